"""``QVBandLinearV8R``: a linear layer whose weight exists on the device only as an entropy-coded QVB8R pack.

Public surface of the reference module of the same name (formats/qvb8r/module.py:57-325): constructed from a parsed
``.qvb8r`` dict or ``from_packfile``; ``forward`` picks a kernel by the row count M of the flattened input; ``dense``
returns the exact weight for audits.

    M = 1        ``gemv``    fp32 band value x fp32 activation
    M = 2..8     ``multi``   the same for several rows (bf16 activations are read as they are: exact in fp32)
    M = 9..16    ``tc``      band value rounded once to fp16 x activation narrowed to saturated fp16
    M = 17..48   equal passes of at most 16 rows through ``tc``
    M > 48       the weight is restored to fp16 and multiplied by one library GEMM per chunk

Escapes (weights stored exactly because the band could not certify them) are added after every kernel product as
``y[m, q] += sum_e x[m, c_e] * (exact_e - band_e)`` in stored order; the differences are kept twice, against the fp32
band value (``gemv`` / ``multi``) and against its fp16 rounding (``tc``).

Many rows, this library's way: a B200 holds any single weight of the model families in scope dense in 16 bits next to
the packs (the largest, a 248k x 5120 vocabulary projection, is 2.5 GB), so the whole weight is restored straight
into ORIGINAL row order by one decode launch and multiplied by one GEMM; only weights above ``RESTORE_BYTES`` fall back
to chunks of whole blocks in sorted row order (the reference's scheme for small cards, module.py:127-161, 249-277).
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch
import torch.nn as nn

from . import packs, rans
from .ext_qvb8r import TILES_PER_BLOCK, core_tensors, ext

ROWS_PER_TC_PASS = 16
MAX_KERNEL_ROWS = 48
_FP32_BUFFERS = ("min_s", "tau_s", "esc_val", "esc_delta", "esc_delta16", "chunk_esc_val")


@dataclasses.dataclass(frozen=True)
class Chunk:
    """A run of whole blocks restored together: blocks [block0, block0 + nblocks) hold the sorted rows
    [row0, row0 + rows); its escapes are entries [esc0, esc1) of the chunk-ordered escape arrays."""
    block0: int
    nblocks: int
    row0: int
    rows: int
    esc0: int
    esc1: int


def plan_chunks(tiles: np.ndarray, blocks: np.ndarray, row_budget: int) -> list[tuple[int, int, int, int]]:
    """Cuts the block schedule into runs of at most `row_budget` sorted rows (a single block may exceed it).  Returns
    (first block, blocks, first sorted row, rows) per run.  Works on the cumulative row count: the end of a run is the
    last block whose cumulative end stays within the budget counted from the run's start."""
    tiles = np.asarray(tiles, np.int64).reshape(-1, 3)
    blocks = np.asarray(blocks, np.int64).reshape(-1, 3)
    tile_end = np.cumsum(tiles[:, 2])
    block_end = tile_end[blocks[:, 1] + blocks[:, 2] - 1]              # sorted rows covered up to and including a block
    block_begin = np.concatenate([[0], block_end[:-1]])
    runs, b, nb = [], 0, len(blocks)
    while b < nb:
        limit = block_begin[b] + max(1, int(row_budget))
        e = int(np.searchsorted(block_end, limit, side="right"))       # first block that would overflow the budget
        e = max(e, b + 1)
        runs.append((b, e - b, int(block_begin[b]), int(block_end[e - 1] - block_begin[b])))
        b = e
    return runs


def escape_tables(d: dict):
    """Host arrays for the escape pass, from a parsed file: rows that have escapes, their ranges (CSR), columns, the
    stored differences and the differences against the fp16-rounded band value; all sorted by (row, column)."""
    P = int(d["P"])
    pos = np.asarray(d["esc_idx"], np.int64)
    order = np.argsort(pos, kind="stable")
    pos = pos[order]
    exact = np.asarray(d["esc_val"], np.float32)[order]
    delta = np.asarray(d["esc_delta"], np.float32)[order]
    band = exact - delta                                               # the fp32 band value the difference was taken from
    delta16 = exact - band.astype(np.float16).astype(np.float32)
    rows, first = np.unique(pos // P, return_index=True)
    ranges = np.append(first, pos.size).astype(np.int64)
    return dict(esc_uq=rows.astype(np.int64), esc_ptr=ranges, esc_c=(pos % P).astype(np.int64), esc_delta=delta,
                esc_delta16=delta16.astype(np.float32), esc_flat=pos, esc_val=exact)


class QVBandLinearV8R(nn.Module):
    RESTORE_BYTES = 4 << 30        # dense fp16 bytes restored at once in the many-rows route
    CHUNK_BYTES = None             # test hook: a smaller budget forces the chunked route

    def __init__(self, d: dict, bias=None, device="cuda", path: str | None = None):
        super().__init__()
        self.path = path
        Q, P = int(d["Q"]), int(d["P"])
        self.out_features, self.in_features, self.T = Q, P, int(d["T"])
        dev = torch.device(device)
        for name, t in zip(("words", "off", "states", "tiles", "blocks8", "tab", "perm", "min_s", "tau_s", "drow"),
                           core_tensors(d, dev)):
            self.register_buffer(name, t, persistent=False)

        def put(name, a, dt):
            self.register_buffer(name, torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(dev), persistent=False)
        esc = escape_tables(d)
        for name, a in esc.items():
            put(name, a, np.float32 if a.dtype == np.float32 else np.int64)
        self.bias = nn.Parameter(torch.as_tensor(bias).detach().to(dev), requires_grad=False) if bias is not None else None

        # the chunked route's tables (used only above the restore budget): per chunk its blocks and sorted rows, the
        # original rows of those sorted rows, and the chunk's escapes as positions inside the chunk
        tiles = np.asarray(d["tiles"], np.int64).reshape(-1, 3)
        blocks = rans.blocks_for(tiles, TILES_PER_BLOCK)
        budget_bytes = self.CHUNK_BYTES if self.CHUNK_BYTES is not None else self.RESTORE_BYTES
        runs = plan_chunks(tiles, blocks, max(1, int(budget_bytes) // (2 * P)))
        perm = np.asarray(d["perm"], np.int64)
        sorted_pos_of = np.empty(Q, np.int64)
        sorted_pos_of[perm] = np.arange(Q)
        esc_sorted_row = sorted_pos_of[esc["esc_flat"] // P] if esc["esc_flat"].size else np.zeros(0, np.int64)
        by_sorted = np.argsort(esc_sorted_row, kind="stable")
        srow, scol, sval = esc_sorted_row[by_sorted], (esc["esc_flat"] % P)[by_sorted], esc["esc_val"][by_sorted]
        starts = np.asarray([r[2] for r in runs], np.int64)
        cut = np.searchsorted(srow, np.append(starts, Q), side="left")
        which = np.searchsorted(starts, srow, side="right") - 1 if srow.size else np.zeros(0, np.int64)
        self.chunks = [Chunk(b0, nb, r0, nr, int(cut[i]), int(cut[i + 1])) for i, (b0, nb, r0, nr) in enumerate(runs)]
        put("chunk_rows", perm, np.int64)                               # sorted position -> original row
        put("chunk_esc_pos", (srow - starts[which]) * P + scol if srow.size else srow, np.int64)
        put("chunk_esc_val", sval, np.float32)
        self.whole = len(self.chunks) == 1

    @classmethod
    def from_packfile(cls, path: str, *, bias=None, tau: float | None = None, device: str = "cuda",
                      blob: bytes | None = None) -> "QVBandLinearV8R":
        """The loader's entry point.  `tau` is accepted and unused: every file states its own certified tau."""
        if blob is None:
            with open(path, "rb") as fh:
                blob = fh.read()
        return cls(packs.read_qvb8r(blob, str(path)), bias=bias, device=device, path=path)

    def _apply(self, fn, recurse=True):
        """Casts of the module never touch the fp32 data of the format; it only follows the stream to a new device."""
        held = {n: self._buffers.pop(n) for n in _FP32_BUFFERS}
        try:
            super()._apply(fn, recurse)
        finally:
            dev = self._buffers["words"].device
            for n, t in held.items():
                self._buffers[n] = t if t.device == dev else t.to(dev)
        return self

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"tile_rows={self.T}")

    # ---- kernel routes --------------------------------------------------------------------------------------
    def core(self) -> tuple:
        """The ten tensors every entry point of the extension takes after its activations."""
        return (self.words, self.off, self.states, self.tiles, self.blocks8, self.tab, self.perm, self.min_s,
                self.tau_s, self.drow)

    def _add_escapes(self, x32: torch.Tensor, y: torch.Tensor, differences: torch.Tensor) -> torch.Tensor:
        y = y if y.is_contiguous() else y.contiguous()
        ext.fix_escapes(x32, self.esc_uq, self.esc_ptr, self.esc_c, differences, y)
        return y

    def _few_rows(self, x2: torch.Tensor) -> torch.Tensor:
        """1..16 rows through the decoding kernels, escapes added."""
        M = x2.shape[0]
        x32 = x2.float().contiguous()
        if M == 1:
            return self._add_escapes(x32, ext.gemv(x32.reshape(-1), *self.core()).reshape(1, -1), self.esc_delta)
        if M <= 8:
            xin = x2.contiguous() if x2.dtype == torch.bfloat16 else x32
            return self._add_escapes(x32, ext.multi(xin, *self.core()), self.esc_delta)
        x16 = x32.clamp(min=-65504.0, max=65504.0).to(torch.float16)
        return self._add_escapes(x32, ext.tc(x16, *self.core(), self.T), self.esc_delta16)

    def _many_rows(self, x2: torch.Tensor) -> torch.Tensor:
        """Restore to fp16 + library GEMM with fp32 accumulation and fp32 result."""
        x16 = x2.float().clamp(min=-65504.0, max=65504.0).to(torch.float16)
        P = self.in_features
        if self.whole:
            # one decode launch writes every row at its original index; escapes by their original positions
            W = ext.decode(*self.core(), P, 0, 0, self.blocks8.shape[0], -1, 0)
            if self.esc_flat.numel():
                W.view(-1)[self.esc_flat] = self.esc_val.to(torch.float16)
            return torch.mm(x16, W.t(), out_dtype=torch.float32)
        y = torch.empty((x2.shape[0], self.out_features), dtype=torch.float32, device=x2.device)
        for c in self.chunks:
            W = ext.decode(*self.core(), P, 0, c.block0, c.nblocks, c.row0, c.rows)       # sorted rows, compact
            if c.esc1 > c.esc0:
                W.view(-1)[self.chunk_esc_pos[c.esc0:c.esc1]] = self.chunk_esc_val[c.esc0:c.esc1].to(torch.float16)
            y[:, self.chunk_rows[c.row0:c.row0 + c.rows]] = torch.mm(x16, W.t(), out_dtype=torch.float32)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).to(self.words.device)
        result_dtype = x.dtype
        if x2.dtype == torch.float32 and torch.is_autocast_enabled(x2.device.type):
            cast_to = torch.get_autocast_dtype(x2.device.type)          # behave like nn.Linear under autocast
            if cast_to in (torch.float16, torch.bfloat16):
                x2, result_dtype = x2.to(cast_to), cast_to
        M = x2.shape[0]
        if M == 0:
            return torch.empty(*lead, self.out_features, dtype=result_dtype, device=x2.device)
        if M <= ROWS_PER_TC_PASS:
            y = self._few_rows(x2)
        elif M <= MAX_KERNEL_ROWS:
            passes = -(-M // ROWS_PER_TC_PASS)
            y = torch.cat([self._few_rows(part) for part in torch.tensor_split(x2, passes, dim=0)])
        else:
            y = self._many_rows(x2)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.to(result_dtype).reshape(*lead, self.out_features)

    def dense(self, dtype=torch.bfloat16) -> torch.Tensor:
        """The exact (Q, P) weight rounded to `dtype`, escapes written over: for audits, not a product path."""
        code = 0 if dtype == torch.float16 else 1 if dtype == torch.bfloat16 else 2
        W = ext.decode(*self.core(), self.in_features, code, 0, self.blocks8.shape[0], -1, 0)
        if self.esc_flat.numel():
            W.view(-1)[self.esc_flat] = self.esc_val.to(W.dtype)
        return W if W.dtype == dtype else W.to(dtype)


class QVBandLinearV8RShard(nn.Module):
    """One rank's share of an entropy-coded linear split over `world` ranks by TILES (the only cut a ``.qvb8r`` tensor
    allows without re-encoding, :func:`qvb8_b200.fuse.qvb8r_tile_shard`): the rank decodes and multiplies a contiguous
    run of tiles -- about 1 / world of the coded words -- and the ranks' output rows, which lie scattered over the whole
    tensor, are exchanged by one all-gather (padded to the largest shard) and put in place.

    `group`: a torch.distributed group, or None for a shard used on its own (``forward`` then returns the local rows and
    ``rows`` says which rows of the whole tensor they are)."""

    def __init__(self, d: dict, rank: int, world: int, *, bias=None, device="cuda", group=None):
        super().__init__()
        from . import fuse
        if not (0 <= rank < world):
            raise ValueError("rank outside the world")
        bounds = fuse.qvb8r_shard_bounds(d, world)
        self.rank, self.world, self.group = int(rank), int(world), group
        self.out_features, self.in_features = int(d["Q"]), int(d["P"])
        shard, rows = fuse.qvb8r_tile_shard(d, bounds[rank], bounds[rank + 1])
        self.local = QVBandLinearV8R(shard, device=device) if shard["Q"] else None
        dev = torch.device(device)
        self.register_buffer("rows", torch.from_numpy(np.ascontiguousarray(rows, dtype=np.int64)).to(dev), persistent=False)
        # every rank's rows (the same on all ranks: the bounds follow from the file alone), padded to the largest shard
        all_rows = [fuse.qvb8r_tile_shard(d, bounds[r], bounds[r + 1])[1] for r in range(world)] if world > 1 else [rows]
        self.pad = max(1, max(len(r) for r in all_rows))
        place = np.full((world, self.pad), self.out_features, np.int64)          # padding lands in a spare column
        for r, rr in enumerate(all_rows):
            place[r, :len(rr)] = rr
        self.register_buffer("place", torch.from_numpy(place.reshape(-1)).to(dev), persistent=False)
        self.bias = nn.Parameter(torch.as_tensor(bias).detach().to(dev), requires_grad=False) if bias is not None else None

    def local_product(self, x: torch.Tensor) -> torch.Tensor:
        """(.., rows.numel()) -- this rank's output rows, in the order of ``rows``."""
        if self.local is None:
            return torch.zeros(*x.shape[:-1], 0, dtype=x.dtype, device=self.rows.device)
        return self.local(x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local_product(x)
        if self.world > 1 and self.group is None:
            return y                                                     # a shard on its own: the local rows
        out = gather_rows(y, self.place, self.pad, self.world, self.out_features, self.group)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out


def gather_rows(y: torch.Tensor, place: torch.Tensor, pad: int, world: int, out_features: int, group) -> torch.Tensor:
    """The whole (.., out_features) product from every rank's local rows y (.., n_r): one all-gather of the rows padded
    to `pad` columns, then every column put where `place` (world * pad positions, `out_features` = discard) says."""
    lead = y.shape[:-1]
    padded = torch.zeros(*lead, pad, dtype=y.dtype, device=y.device)
    padded[..., :y.shape[-1]] = y
    if world > 1:
        import torch.distributed as dist
        parts = torch.empty(world, *lead, pad, dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(parts.view(-1), padded.contiguous().view(-1), group=group)   # (1-D: every backend takes it)
        flat = parts.movedim(0, -2).reshape(*lead, world * pad)
    else:
        flat = padded
    out = torch.empty(*lead, out_features + 1, dtype=y.dtype, device=y.device)
    out[..., place] = flat
    return out[..., :out_features]
