"""The linear stack of a dense decoder as one replayable unit: every packed projection of every layer, run in order.

This is the per-token hot path the reference walks with one Python call per linear (decode/spec_decode.py:3982-3998
-> every q/k/v/o/gate/up/down ``forward``) and wraps in CUDA graphs to hide launch cost
(decode/proj_graph.py, decode/layer_graph.py).  Here the whole stack is captured once into a CUDA graph and replayed;
the packs stay resident in HBM and every replay streams each of them exactly once.

Projections of one layer and their inputs (d = d_model, kv = kv heads x head_dim, f = MLP width):

    q (d -> q_out)  k (d -> kv)  v (d -> kv)   read the attention input x_attn (M, d)
    o (q_out -> d)                              reads x_o (M, q_out)
    gate (d -> f)   up (d -> f)                 read the MLP input x_mlp (M, d)
    down (f -> d)                               reads x_down (M, f)

Attention, norms and activations between them are not part of this path; the stack feeds every projection a
resident activation buffer of the right shape.

Projections that read the same input (q/k/v; gate/up) are fused into one pack and one launch by default, as the
reference fuses its entropy-coded linears (formats/qvb8r/fuse.py:1-60); the members' outputs are views of the fused
output and every compressed byte is still streamed exactly once per step.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import fuse as _fuse
from . import lib as _lib
from . import synth


@dataclass(frozen=True)
class StackConfig:
    name: str
    layers: int
    d_model: int
    q_out: int
    kv_out: int
    mlp: int
    tau: float
    config_id: int

    def projections(self):
        """(name, Q, P, input buffer) of one layer, in execution order."""
        d, f = self.d_model, self.mlp
        return [("q", self.q_out, d, "x_attn"), ("k", self.kv_out, d, "x_attn"), ("v", self.kv_out, d, "x_attn"),
                ("o", d, self.q_out, "x_o"), ("gate", f, d, "x_mlp"), ("up", f, d, "x_mlp"), ("down", d, f, "x_down")]

    def weights_per_layer(self) -> int:
        return sum(q * p for _, q, p, _ in self.projections())


# shapes of the benchmark configurations
DENSE_9B = StackConfig("9b-dense", 32, 4096, 4096, 1024, 12288, 1e-3, 2)
DENSE_27B = StackConfig("27b-dense", 64, 5120, 5120, 1024, 17408, 2e-3, 3)
DENSE_65B = StackConfig("65b-dense", 80, 8192, 8192, 1024, 28672, 1e-3, 5)
CONFIGS = {c.name: c for c in (DENSE_9B, DENSE_27B, DENSE_65B)}


ROW_PARALLEL = ("o", "down")      # sharded by input columns when world > 1; the others by output rows


def _lib_max_jobs() -> int:
    return 128                    # jobs one launch of the streaming kernel takes (MAX_JOBS of the kernel source)


MAX_GROUP_LAYERS = 32             # layers behind one launch at most (four fused projections each)


class LinearStack:
    """Packs of `layers` decoder layers resident on one device + activation / output buffers + a captured graph.

    rank / world: q/k/v and gate/up are sharded by OUTPUT ROWS (column-parallel): rank r holds rows
    [r*Q/world, (r+1)*Q/world), which for a QVB8 pack is a slice of the per-row vectors and a byte range of the ids
    (rows are independent, reference formats/qvb8/module.py:126-160).  Their consumers o and down are sharded by
    INPUT COLUMNS (row-parallel): rank r holds columns [r*P/world, (r+1)*P/world) of every row, cut out of the whole
    pack's bytes (``fuse.column_shard``), reads the matching slice of the activation and produces a partial (M, Q)
    sum; one all-reduce per column->row pair is the only exchange (two per layer, or one per launch when several
    layers run behind one launch).

    shard="rows": EVERY projection is sharded by output rows, the reference's own cut (``row_subset``).  The shards of o
    and down keep their full-length rows -- eight times fewer, eight times longer tiles than the column shards at
    world 8, which the streaming kernel runs markedly faster at M = 1 -- at the price of more exchanges: o and down
    need their whole input, so the ranks all-gather their slices of the attention output and the MLP activation as
    well as the slices of the o and down outputs (four all-gathers per layer in a model; here one all-gather per
    launch carrying all four slices of the launch's layers)."""

    def __init__(self, cfg: StackConfig, M: int, device, layers: int | None = None, seed_base: int | None = None,
                 rank: int = 0, world: int = 1, policy: str = "escape_outliers", x_dtype=torch.bfloat16,
                 fuse_same_input: bool = True, shard: str = "pairs"):
        if shard not in ("pairs", "rows"):
            raise ValueError("shard must be 'pairs' or 'rows'")
        self.shard = shard
        self.cfg, self.M, self.device = cfg, int(M), torch.device(device)
        self.layers = cfg.layers if layers is None else int(layers)
        self.rank, self.world = rank, world
        self.fused = bool(fuse_same_input)
        self.launches = []       # [layer][launch] -> (name, QVB8Pack, struct, keepalive (+ plan), input name, member names)
        self.compressed_bytes = 0
        self.n_weights = 0
        self.width_hist: dict = {}
        self.n_escapes = 0
        seed_base = 1000 * cfg.config_id if seed_base is None else seed_base
        groups = dict(_fuse.SAME_INPUT_GROUPS) if self.fused else {}
        member_group = {m: g for g, ms in groups.items() for m in ms}
        for layer in range(self.layers):
            made = {}
            for j, (name, Q, P, xname) in enumerate(cfg.projections()):
                # every rank encodes the WHOLE weight (a deployment would read the whole pack file) and cuts its shard
                # out of the pack's bytes: rows for the column-parallel projections, input columns for the row-parallel
                W = synth.synth_weight(Q, P, seed_base + layer * 16 + j, device=self.device)
                pk = synth.encode_qvb8(W, tau=cfg.tau, policy=policy)
                del W
                if world > 1:
                    if name in ROW_PARALLEL and shard == "pairs":
                        if P % (128 * world):
                            raise ValueError(f"{name}: {P} columns do not split over {world} ranks in 128-column units")
                        pk = _fuse.column_shard(pk, rank * (P // world), (rank + 1) * (P // world))
                    else:
                        if Q % world:
                            raise ValueError(f"{name}: {Q} rows do not split over {world} ranks")
                        pk = _fuse.row_shard(pk, rank * (Q // world), (rank + 1) * (Q // world))
                made[name] = (pk, xname)
            row, done = [], set()
            for name, _, _, xname in cfg.projections():
                if name in done:
                    continue
                g = member_group.get(name)
                members = [m for m in groups[g] if m in made] if g else [name]
                if len(members) > 1:
                    pk, _ = _fuse.concat_packs([made[m][0] for m in members])
                    lname = g
                else:
                    pk, lname = made[name][0], name
                done.update(members)
                st, keep = _lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx,
                                            pk.esc_vals)
                plan = _lib.build_plan(st, keep)
                row.append((lname, pk, st, keep + [plan], xname, members))
                self.compressed_bytes += pk.weight_bytes()
                self.n_weights += pk.Q * pk.P
                self.n_escapes += int(pk.esc_idx.numel())
                for b, n in pk.stats["nbits_hist"].items():
                    self.width_hist[b] = self.width_hist.get(b, 0) + n
            del made
            self.launches.append(row)
        d, f = cfg.d_model, cfg.mlp
        # row-parallel projections read only this rank's slice of their input
        cut = world if shard == "pairs" else 1
        shapes = {"x_attn": d, "x_o": cfg.q_out // cut, "x_mlp": d, "x_down": f // cut}
        self.x = {k: synth.synth_activation(self.M, p, seed=7 + i, device=self.device, dtype=x_dtype)
                  for i, (k, p) in enumerate(shapes.items())}
        # one output buffer per launch; y[layer][name] are the members' views of it.  The outputs of the row-parallel
        # projections (partial sums that the ranks exchange) lie side by side in ONE buffer, layer after layer, so that
        # the partial sums of several layers can be exchanged by a single all-reduce.
        n_rp = sum(1 for name, *_ in self.launches[0] if name in ROW_PARALLEL)
        d_out = d if shard == "pairs" else d // world
        if shard == "pairs":
            self.y_rowpar = torch.empty((self.layers * n_rp, self.M, d_out), dtype=torch.float32, device=self.device)
            rp_out = [self.y_rowpar[i] for i in range(self.layers * n_rp)]
        else:
            # everything split by output rows: what a rank must hand to the others, per layer, is its slice of the o and
            # down outputs and its slice of their inputs (attention output, MLP activation -- produced outside this
            # path, random here).  One contiguous part per layer, so a launch's layers are exchanged by one all-gather.
            extra = self.M * (cfg.q_out + f) // world
            self.part = torch.randn((self.layers, n_rp * self.M * d_out + extra), dtype=torch.float32, device=self.device,
                                    generator=torch.Generator(device=self.device).manual_seed(11 + rank))
            self.gathered = None
            rp_out = [self.part[i // n_rp, (i % n_rp) * self.M * d_out:(i % n_rp + 1) * self.M * d_out].view(self.M, d_out)
                      for i in range(self.layers * n_rp)]
        self.y_launch = []
        for li, row in enumerate(self.launches):
            outs, k = [], 0
            for name, pk, *_ in row:
                if name in ROW_PARALLEL and pk.Q == d_out:
                    outs.append(rp_out[li * n_rp + k])
                    k += 1
                else:
                    outs.append(torch.empty((self.M, pk.Q), dtype=torch.float32, device=self.device))
            self.y_launch.append(outs)
        self._n_rp = n_rp
        self.y = []
        for row, outs in zip(self.launches, self.y_launch):
            views = {}
            for (lname, pk, _, _, _, members), out in zip(row, outs):
                sizes = pk.stats.get("members", [pk.Q]) if len(members) > 1 else [pk.Q]
                for m, t in zip(members, torch.split(out, sizes, dim=1)):
                    views[m] = t
            self.y.append(views)
        for row in self.launches:
            for _, pk, *_ in row:
                _lib.reserve_scratch(self.device, self.M, pk.Q, pk.P)
        self.graph = None
        self.reduce = False      # all-reduce the row-parallel projections' partial sums (set by enable_collectives)
        self.peer = None         # the NVLink push all-reduce, when enabled
        self.launches_per_step = sum(len(row) for row in self.launches)
        self.pdl = True
        self._host_in = self._host_out = None
        self.group_layers = 0    # > 0: this many layers' projections behind one launch (set_grouping)
        self._groups = None

    # ---- execution ------------------------------------------------------------------------------------
    def enable_collectives(self, peer: bool = True) -> None:
        """The shard boundaries: after o and after down the ranks all-reduce their partial (M, d_model) sums, captured
        into the graph with the launches.  peer=True: the push kernel over NVLink peer memory (qvb8_b200.peer); False:
        NCCL on the compute stream.  q/k/v and gate/up need no exchange: their consumers work on the local slice."""
        import torch.distributed as dist
        self.reduce = self.world > 1 and dist.is_initialized()
        self.peer = None
        if self.reduce and peer:
            from .peer import PeerAllReduce
            # the largest exchange: the row-parallel outputs of up to MAX_GROUP_LAYERS layers at once (see set_grouping)
            if self.shard == "pairs":
                cap = max(max(t.numel() for row in self.y_launch for t in row),
                          min(self.layers, MAX_GROUP_LAYERS) * self._n_rp * self.M * self.cfg.d_model)
            else:
                cap = min(self.layers, MAX_GROUP_LAYERS) * self.part.shape[1]
            self.peer = PeerAllReduce(dist.group.WORLD, cap, self.device)
        if self.reduce and self.shard == "rows":
            self.gathered = torch.empty((self.world, min(self.layers, MAX_GROUP_LAYERS) * self.part.shape[1]), dtype=torch.float32,
                                        device=self.device)

    def _allgather(self, l0: int, l1: int) -> None:
        """Exchange the parts of layers [l0, l1): afterwards gathered[r] holds rank r's."""
        part = self.part[l0:l1].view(-1)
        out = self.gathered.view(-1)[:self.world * part.numel()]
        if self.peer is not None and part.numel() % 4 == 0:
            self.peer.allgather(part, out, flags=_lib.FLAG_PDL if self.pdl else 0)
        else:
            import torch.distributed as dist
            dist.all_gather_into_tensor(out, part)

    def _allreduce(self, t: torch.Tensor) -> None:
        if self.peer is not None and t.numel() % 4 == 0:
            self.peer.allreduce(t, flags=_lib.FLAG_PDL if self.pdl else 0)
        else:
            import torch.distributed as dist
            dist.all_reduce(t)

    def set_grouping(self, layers_per_launch: int) -> None:
        """Run the projections of `layers_per_launch` consecutive layers as ONE launch each (``qvb8_small_m_group``):
        inside a launch the weight stream never drains between projections.  The stack's projections read resident
        activation buffers and write separate outputs, so they are independent jobs.  0 = one launch per projection.
        With several ranks the partial sums of a launch's row-parallel projections (o and down of its layers) are
        exchanged by ONE all-reduce after the launch."""
        self.group_layers = min(int(layers_per_launch), MAX_GROUP_LAYERS)
        self._groups = None
        self.graph = None
        if self.group_layers > 0:
            per = max(1, min(self.group_layers, _lib_max_jobs() // max(1, len(self.launches[0]))))
            self._groups, self._group_layers = [], []
            for l0 in range(0, self.layers, per):
                items = []
                self._group_layers.append((l0, min(self.layers, l0 + per)))
                for li in range(l0, min(self.layers, l0 + per)):
                    for j, (name, pk, st, keep, xname, _) in enumerate(self.launches[li]):
                        items.append((st, keep, keep[-1], self.x[xname], self.y_launch[li][j]))
                self._groups.append(_lib.JobList(items))
            self.launches_per_step = len(self._groups)
        else:
            self.launches_per_step = sum(len(row) for row in self.launches)

    def kernels_per_step(self) -> int:
        """Kernels of this library one step launches: per list launch the streaming kernel, the escape pre-pass when a
        pack of the list carries escapes, and the exchange kernel when ranks exchange; per single launch one (a lower
        bound: a list whose jobs do not all fit one launch is cut into several)."""
        extra = 1 if self.reduce else 0
        if self._groups is not None:
            n = 0
            for l0, l1 in self._group_layers:
                esc = any(pk.esc_idx.numel() > 0 for li in range(l0, l1) for _, pk, *_ in self.launches[li])
                n += 1 + (1 if esc else 0) + extra
            return n
        per_layer_exchanges = (self._n_rp if self.shard == "pairs" else 1) * extra
        return sum(len(row) + per_layer_exchanges for row in self.launches)

    def run_eager(self) -> None:
        """One pass over every launch of every layer on the current stream."""
        if self._groups is not None:
            for g, (l0, l1) in zip(self._groups, self._group_layers):
                _lib.small_m_group(g, flags=_lib.FLAG_PDL if self.pdl else 0)
                if self.reduce and self.shard == "rows":
                    self._allgather(l0, l1)
                elif self.reduce:
                    self._allreduce(self.y_rowpar[l0 * self._n_rp:l1 * self._n_rp].view(-1))
            return
        for li, row in enumerate(self.launches):
            for j, (name, pk, st, keep, xname, _) in enumerate(row):
                _lib.small_m(st, keep, self.x[xname], out=self.y_launch[li][j], plan=keep[-1],
                             flags=_lib.FLAG_PDL if self.pdl else 0)
                if self.reduce and name in ROW_PARALLEL and self.shard == "pairs":
                    self._allreduce(self.y_launch[li][j])
            if self.reduce and self.shard == "rows":
                self._allgather(li, li + 1)

    def capture(self) -> None:
        # warm-up (shared-memory opt-in, scratch) on the stream the capture will use: scratch buffers are kept per
        # stream, so everything the captured calls need exists before the capture begins
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.run_eager()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            self.run_eager()
        self.graph = g

    def step(self) -> None:
        """One decode step of the stack with the activations already resident in HBM."""
        if self.graph is None:
            self.capture()
        self.graph.replay()

    # ---- the host-buffer API (end-to-end: pinned host activations in, last layer's outputs back) --------
    def _host_buffers(self):
        if self._host_in is None:
            self._host_in = {k: torch.empty_like(v, device="cpu").pin_memory() for k, v in self.x.items()}
            for k, v in self.x.items():
                self._host_in[k].copy_(v)
            last = self.y_launch[-1]
            self._host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in last]
        return self._host_in, self._host_out

    def step_host(self, x_host: dict | None = None):
        """Activations from pinned host memory -> one stack step -> the last layer's projection outputs on the host.
        Returns the list of host tensors (valid after this call returns: it synchronises)."""
        hin, hout = self._host_buffers()
        if x_host is not None:
            for k, v in x_host.items():
                hin[k].copy_(v)
        for k in self.x:
            self.x[k].copy_(hin[k], non_blocking=True)
        self.step()
        for t, h in zip(self.y_launch[-1], hout):
            h.copy_(t, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return hout

    def h2d_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.x.values())

    def d2h_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.y_launch[-1])
