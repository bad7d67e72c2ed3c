#!/usr/bin/env python
"""Benchmark of the fused decode-in-matmul over a QVB8 linear stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L] [--rows M]

Metric: compressed-weight bytes streamed per second at M = 1 (GB/s, the packs' own bytes: bit-packed ids + per-row
metadata + escape entries), over the 9B-class dense decoder linear stack (32 layers: q/k/v/o 4096->4096/1024/1024/
4096, gate/up 4096->12288, down 12288->4096; weights N(0, 0.02) with 0.1% +-10 sigma outliers, QVB8 tau = 1e-3,
seeded).  One step = one pass over every projection of every layer = one decode token.

  value   whole-job GB/s with the activations resident in HBM (CUDA-graph replay, CUDA events, max over ranks)
  e2e     the same through LinearStack.step_host: pinned host activations -> device, the step, outputs -> host
  N > 1   below 8 tokens every projection is sharded by output rows and the ranks all-gather the slices of the o / down
          outputs and inputs; from 8 tokens q/k/v and gate/up by output rows, o and down by input columns, partial sums
          all-reduced (--shard).  One exchange per list launch, by this library's push kernels over peer memory (checked
          against NCCL first; --nccl-allreduce uses NCCL).  Total bytes stay fixed ("strong")
  other workloads (--workload): single, qvb8r, moe, prefill -- each prints its own JSON line

--impl reference times the CPU path the reference itself would run for this op (it ships no CPU GEMV): restore the
pack to bf16 weights, then torch.matmul on the host cores -- here through the CPU oracle's restatement of the
reference decoder, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "compressed_weight_stream_m1"
UNIT = "GB/s"


DRAM_TRAFFIC_RATIO = 89.7 / 89.3      # (dram__bytes_read + dram__bytes_write) / algorithmic bytes, ncu, one launch


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period: float = 0.01):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {}
        for n in ("HwSlowdown", "HwThermalSlowdown", "SwThermalSlowdown", "SwPowerCap", "HwPowerBrakeSlowdown"):
            v = getattr(nv, "nvmlClocksEventReason" + n, None) or getattr(nv, "nvmlClocksThrottleReason" + n, None)
            if v is not None:
                names[int(v)] = n
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                if get is not None:
                    r = int(get(self.h))
                    for bit, n in names.items():
                        if r & bit:
                            self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        def snake(n):
            return "".join("_" + c.lower() if c.isupper() else c for c in n).lstrip("_")
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(snake(r) for r in self.reasons), "samples": len(self.samples)}


def cpu_reference_step(sample, threads: int):
    """One bounded CPU sample: restore each pack of `sample` to bf16 with the oracle's restatement of the reference
    decoder, then torch.matmul with the bf16 activation on the host cores.  Returns bytes processed."""
    import numpy as np
    import oracle
    nbytes = 0
    for pk, x in sample:
        bits = oracle.decode_16(pk["ids"], pk["nbits"], pk["bit_off"], pk["min_s"], pk["tau_s"], pk["Q"], pk["P"],
                                pk["esc_idx"], pk["esc_vals"], "bf16")
        W = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)
        y = torch.matmul(x, W.t())
        nbytes += pk["bytes"]
        del W, y
    return nbytes


def build_cpu_sample(cfg, rows_cap: int = 4096):
    """The first layer's q/k/v/o packs of the workload (seeded as on the GPU), on the host, as oracle dicts."""
    from qvb8_b200 import synth
    sample = []
    for j, (name, Q, P, _) in enumerate(cfg.projections()[:4]):
        pk = synth.synth_pack(min(Q, rows_cap), P, 1000 * cfg.config_id + j, tau=cfg.tau)
        d = dict(Q=pk.Q, P=pk.P, ids=pk.ids.numpy(), nbits=pk.nbits.numpy(), bit_off=pk.bit_off.numpy(),
                 min_s=pk.min_s.numpy(), tau_s=pk.tau_s.numpy(), esc_idx=pk.esc_idx.numpy(),
                 esc_vals=pk.esc_vals.numpy(), bytes=pk.weight_bytes())
        x = synth.synth_activation(1, P, seed=7)
        sample.append((d, x))
    return sample


def run_reference_arm(args, cfg):
    """CPU arm: rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.num_threads()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    sample = build_cpu_sample(cfg)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(sample, threads)
    t0 = time.perf_counter()
    nbytes = 0
    for _ in range(args.steps):
        nbytes += cpu_reference_step(sample, threads)
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    desc = "layer-0 q,k,v,o packs of the workload (4096x4096, 2x 1024x4096, 4096x4096), M=1, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{cfg.name} linear stack, decode M=1 (CPU sample)", "sample": desc},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_moe(args):
    """One mixture-of-experts layer of the 35B-A3B-class configuration: 128 experts, top-8 routing from a seeded
    softmax over N(0, 1) logits, d_model 2048, expert FFN 768, QVB8 tau = 1e-3 with the outliers kept in band (expert
    stacks carry no escapes).  Metric: bytes of the DISTINCT selected experts' gate_up and down packs per second.
    N > 1: expert parallelism -- rank r holds experts [r E/N, (r+1) E/N), every rank sees all tokens and the routing,
    the fp32 partial outputs are all-reduced by the push kernel over peer memory (strong scaling: one layer's work is
    split)."""
    from qvb8_b200 import experts, lib, synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    E, topk, d, f, M = 128, 8, 2048, 768, args.rows
    if E % world:
        raise SystemExit(f"bench.py: {E} experts do not split over {world} ranks")
    per = E // world
    mine = range(rank * per, (rank + 1) * per)
    ups = [synth.encode_qvb8(synth.synth_weight(2 * f, d, 4000 + e, device=dev), tau=1e-3, policy="inband") for e in mine]
    dns = [synth.encode_qvb8(synth.synth_weight(d, f, 5000 + e, device=dev), tau=1e-3, policy="inband") for e in mine]
    per_expert = torch.zeros(E, dtype=torch.int64, device=dev)
    per_expert[rank * per:(rank + 1) * per] = torch.tensor([u.weight_bytes() + v.weight_bytes() for u, v in zip(ups, dns)],
                                                           device=dev)
    if world > 1:
        dist.all_reduce(per_expert)
    per_expert = per_expert.tolist()
    mod = experts.QVBandExpertsV8(ups, dns, num_experts=per, first_expert=rank * per, total_experts=E)
    sample = (ups[:], dns[:]) if rank == 0 else None             # the CPU baseline restores a few of these below
    del ups, dns
    exchange = None
    if world > 1:
        from qvb8_b200.peer import PeerAllReduce
        peer = PeerAllReduce(dist.group.WORLD, M * d, dev)
        probe = torch.randn(M * d, device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
        got, ref = peer.allreduce(probe.clone()), probe.clone()
        dist.all_reduce(ref)
        ok = torch.tensor([int(torch.allclose(got, ref, rtol=1e-5, atol=1e-5))], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1 and (M * d) % 4 == 0:
            mod.set_reduce(lambda t: peer.allreduce(t.view(-1)).view_as(t))
            exchange = "peer push all-reduce (checked against NCCL)"
        else:
            mod.set_reduce(lambda t: dist.all_reduce(t))
            exchange = "nccl all-reduce"
    g = torch.Generator(device="cpu").manual_seed(11)
    w, idx = torch.topk(torch.softmax(torch.randn(M, E, generator=g), -1), topk, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float()
    X = synth.synth_activation(M, d, seed=7, device=dev)
    host = [X.cpu().pin_memory(), idx.pin_memory(), w.pin_memory()]
    idx_d, w_d = idx.to(dev), w.to(dev)
    distinct = sorted(set(idx.flatten().tolist()))
    nbytes = sum(per_expert[e] for e in distinct)
    warm = max(3, args.warmup)
    s = torch.cuda.Stream(dev)
    with torch.cuda.stream(s):
        for _ in range(warm):
            mod(X, idx_d, w_d)
    s.synchronize()
    graph = torch.cuda.CUDAGraph()                              # the launches of the layer (+ the exchange), replayed
    with torch.cuda.graph(graph, stream=s, capture_error_mode="thread_local"):
        out = mod(X, idx_d, w_d)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    with ClockSampler(local) as clocks:
        for a, b in ev:
            flush.zero_()                                     # the selected experts (<= 250 MB) would otherwise sit in L2
            a.record(); graph.replay(); b.record()
        barrier()
    ms = sum(a.elapsed_time(b) for a, b in ev) / args.steps
    # end to end: activations, routing and weights from pinned host memory, the layer's output back to the host
    out_host = torch.empty_like(out, device="cpu").pin_memory()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        X.copy_(host[0], non_blocking=True); idx_d.copy_(host[1], non_blocking=True); w_d.copy_(host[2], non_blocking=True)
        graph.replay()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    status = lib.device_status(dev)
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    # CPU baseline on a bounded sample: restore the first token's experts that rank 0 holds (C restatement of the
    # reference decoder) and run the expert MLP on them in numpy
    import numpy as np
    import oracle

    def pack_np(pk):
        c = lambda t: t.detach().cpu().numpy()
        return dict(Q=pk.Q, P=pk.P, ids=c(pk.ids), nbits=c(pk.nbits), bit_off=c(pk.bit_off), min_s=c(pk.min_s),
                    tau_s=c(pk.tau_s), esc_idx=c(pk.esc_idx), esc_vals=c(pk.esc_vals))
    chosen = [e for e in idx[0].tolist() if e < per][:4] or [0]
    host_packs = [(pack_np(sample[0][e]), pack_np(sample[1][e])) for e in chosen]
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < min(args.cpu_seconds, 10.0):
        upd = np.stack([oracle.qvb8_dense(u) for u, _ in host_packs])
        dnd = np.stack([oracle.qvb8_dense(v) for _, v in host_packs])
        oracle.moe_experts(X[:1].float().cpu().numpy(), np.arange(len(chosen))[None, :],
                           np.full((1, len(chosen)), 1.0 / len(chosen), np.float32), upd, dnd)
        reps += 1
    cpu_s = (time.perf_counter() - t0) / reps
    cpu_gbs = sum(per_expert[e] for e in chosen) / cpu_s / 1e9
    peak, peak_kind = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    launches = 4 + (1 if world > 1 else 0)
    print(json.dumps({
        "metric": "moe_distinct_expert_bytes_per_s", "value": gbs, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"35B-A3B-class expert layer, E={E}, top-{topk}, d_model {d}, expert FFN {f}, M={M} tokens",
                   "distinct_experts": len(distinct), "bytes": nbytes, "l2": "256 MB written between steps",
                   "parallelism": (f"experts split {per} per rank x{world}, tokens and routing replicated, fp32 partial "
                                   f"outputs exchanged by one {exchange} per layer") if world > 1 else "single GPU",
                   "device_status": status},
        "clocks": clocks.summary(), "gpu_launches": launches * args.steps,
        "e2e": {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
                "d2h_bytes_per_step": out_host.numel() * out_host.element_size()},
        "roofline": {"bound": "hbm", "achieved": gbs * (1.0 / world), "peak": peak, "unit": "GB/s",
                     "frac": gbs / world / peak, "traffic": None, "peak_kind": peak_kind, "kernel": "moe_rows_kernel",
                     "note": "per GPU: distinct-expert bytes of the layer / ranks / step time"},
        "cpu_baseline": {"value": cpu_gbs, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                         "sample": f"{len(chosen)} experts of the first token: restore gate_up and down (C restatement "
                                   f"of the reference decoder) + the expert MLP in numpy, {reps} repetitions in "
                                   f"{cpu_s * reps:.1f} s"}}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill(args):
    """Prefill of one 27B-class layer's MLP projections (gate+up fused 34816 x 5120, down 5120 x 17408) for M tokens
    (default 2048) through the tcgen05 kernel: QVB8 packs at tau = 2e-3, outliers escaped.  Metric: dense-equivalent
    TFLOP/s (2 M Q P per projection) over the whole call, i.e. the fp16 narrowing of X, the main kernel and the
    escape pass; beside it the same projections through dense restore + library GEMM."""
    from qvb8_b200 import fuse, lib, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    M = args.rows if args.rows > 1 else 2048
    d, f = 5120, 17408
    gate = synth.encode_qvb8(synth.synth_weight(f, d, 6001, device=dev), tau=2e-3, policy=args.policy)
    up = synth.encode_qvb8(synth.synth_weight(f, d, 6002, device=dev), tau=2e-3, policy=args.policy)
    down = synth.encode_qvb8(synth.synth_weight(d, f, 6003, device=dev), tau=2e-3, policy=args.policy)
    packs = [fuse.concat_packs([gate, up])[0], down]
    del gate, up
    work = []
    for pk in packs:
        st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
        work.append((pk, st, keep, lib.build_plan(st, keep), synth.synth_activation(M, pk.P, seed=pk.Q, device=dev)))
    flops = sum(2.0 * M * pk.Q * pk.P for pk in packs)

    def fused():
        return [lib.prefill(st, keep, X, plan=plan) for _, st, keep, plan, X in work]

    def dense():
        return [torch.mm(X.to(torch.float16), lib.decode(st, keep, torch.float16).t(), out_dtype=torch.float32)
                for _, st, keep, _, X in work]

    def timed(fn, steps, clocks_on):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        with ClockSampler(0) as clocks:
            for a, b in ev:
                a.record(); fn(); b.record()
            torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in ev) / steps, clocks.summary() if clocks_on else None

    ms, clk = timed(fused, args.steps, True)
    ms_dense, _ = timed(dense, max(3, args.steps // 2), False)
    # end to end: X from pinned host memory, one value of every result read back
    hx = [X.cpu().pin_memory() for *_, X in work]
    def e2e_step():
        outs = []
        for (pk, st, keep, plan, _), h in zip(work, hx):
            outs.append(lib.prefill(st, keep, h.to(dev, non_blocking=True), plan=plan))
        return float(sum(o[0, 0] for o in outs))
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) / args.steps * 1e3
    peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json"))) \
        if os.path.exists(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "prefill_dense_equivalent_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32", "data": "synthetic",
        "config": {"workload": f"27B-class MLP projections (gate+up 34816x5120, down 5120x17408), prefill M={M}, QVB8 tau=2e-3, "
                               f"policy {args.policy}", "l2": "weights + activations (> 400 MB) exceed L2",
                   "dense_restore_plus_library_gemm_ms": ms_dense},
        "clocks": clk, "gpu_launches": sum(4 + (1 if pk.esc_idx.numel() else 0) for pk in packs) * args.steps,
        "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(sum(h.numel() * h.element_size() for h in hx)), "d2h_bytes_per_step": 8},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                     "peak_kind": "measured (burst)" if peaks else "fallback", "kernel": "prefill_kernel"}}), flush=True)


def run_single(args):
    """One linear layer (default 4096 x 4096, the single-layer configuration; --shape QxP for others) at M = --rows:
    `copies` distinct packs of that shape are multiplied back to back per step, so that a step streams more bytes than
    the L2 holds.  One launch per pack (the reference-shaped call path).  Also the committed driver of the profiler
    summaries under profiles/."""
    import oracle
    from qvb8_b200 import lib, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Q, P = (int(v) for v in args.shape.lower().split("x"))
    M = args.rows
    one = synth.synth_pack(Q, P, 1000, tau=1e-3, device=dev, policy=args.policy)
    copies = max(2, -(-(300 << 20) // max(1, one.weight_bytes())))          # > 2 x L2 per step
    packs = [one] + [synth.synth_pack(Q, P, 1000 + c, tau=1e-3, device=dev, policy=args.policy) for c in range(1, copies)]
    work = []
    X = synth.synth_activation(M, P, seed=7, device=dev)
    for pk in packs:
        st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
        work.append((st, keep, lib.build_plan(st, keep), torch.empty(M, Q, device=dev)))
    lib.reserve_scratch(dev, M, Q, P)
    nbytes = sum(pk.weight_bytes() for pk in packs)

    def step():
        for st, keep, plan, Y in work:
            lib.small_m(st, keep, X, out=Y, plan=plan, flags=lib.FLAG_PDL)
    s = torch.cuda.Stream(dev)
    with torch.cuda.stream(s):
        lib.reserve_scratch(dev, M, Q, P)
        step()
    s.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        step()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(args.steps):
            graph.replay()
        ev1.record()
        torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    # parity of what was just timed: pack 0 against the CPU oracle
    d = dict(Q=one.Q, P=one.P, ids=one.ids.cpu().numpy(), nbits=one.nbits.cpu().numpy(), bit_off=one.bit_off.cpu().numpy(),
             min_s=one.min_s.cpu().numpy(), tau_s=one.tau_s.cpu().numpy(), esc_idx=one.esc_idx.cpu().numpy(),
             esc_vals=one.esc_vals.cpu().numpy())
    want = oracle.matmul_f32w(X.float().cpu().numpy(), oracle.qvb8_dense(d), narrow_x=True)
    got = work[0][3].cpu().numpy()
    import numpy as np
    err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    # end to end: X from pinned host memory, the last pack's result back to the host
    hx, hy = X.cpu().pin_memory(), torch.empty_like(work[-1][3], device="cpu").pin_memory()
    def e2e_step():
        X.copy_(hx, non_blocking=True)
        graph.replay()
        hy.copy_(work[-1][3], non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
    # CPU baseline: the oracle's restatement of the reference decoder restoring pack 0 to bf16 + torch matmul
    threads = oracle.num_threads()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    sample = [(dict(d, bytes=one.weight_bytes()), X.cpu())]
    cpu_reference_step(sample, threads)
    t0 = time.perf_counter()
    nb = reps = 0
    while time.perf_counter() - t0 < args.cpu_seconds:
        nb += cpu_reference_step(sample, threads)
        reps += 1
    dt = time.perf_counter() - t0
    peak, peak_kind = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"single linear {Q}x{P}, M={M}, QVB8 tau=1e-3, policy={args.policy}: {copies} distinct packs "
                               "per step, one launch each", "bytes_per_step": nbytes, "us_per_launch": ms * 1e3 / copies,
                   "l2": "a step streams more than twice the L2", "rel_fro_vs_oracle": err},
        "clocks": clocks.summary(), "gpu_launches": copies * args.steps,
        "e2e": {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": hx.numel() * hx.element_size(),
                "d2h_bytes_per_step": hy.numel() * hy.element_size(), "ms_per_step": e2e_ms},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "peak_kind": peak_kind, "kernel": "small_m_kernel"},
        "cpu_baseline": {"value": nb / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"pack 0 restored to bf16 by the C restatement of the reference decoder + torch.matmul, "
                                   f"{reps} repetitions in {dt:.1f} s"}}), flush=True)


def run_qvb8r(args):
    """The entropy-coded format: the seven projections of one 27B-class layer (d_model 5120, MLP 17408, q/o 5120, k/v
    1024) as QVB8R packs at tau = 2e-3, products at M = --rows (1 = gemv, 2..8 = multi, 9..16 = tc) with the escape
    pass.  Metric: bytes of the coded stream and its tables per second (the kernel is bound by the decoder's
    dependency chain, not by HBM: the fraction is reported for completeness).  --layers scales the rows down for quick
    runs (rows / layers)."""
    import numpy as np
    from qvb8_b200 import fuse, rans, synth
    from qvb8_b200.linear_r import QVBandLinearV8R, QVBandLinearV8RShard
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    M = args.rows
    div = max(1, args.layers or 1)
    d, f = 5120, 17408
    shapes = [("q", 5120, d), ("k", 1024, d), ("v", 1024, d), ("o", d, 5120), ("gate", f, d), ("up", f, d), ("down", d, f)]
    t0 = time.perf_counter()
    mods, nbytes, nweights = [], 0, 0
    for j, (name, Q, P) in enumerate(shapes):
        Q = max(64, Q // div)
        # every rank codes the whole tensor (a deployment reads the whole file) and keeps its run of tiles
        enc = synth.encode_qvb8r(synth.synth_weight(Q, P, 3000 + j), tau=2e-3, K=4, T=max(1, -(-Q // 4096)))
        nt = len(enc["tiles"])
        nb8 = len(rans.blocks_for(enc["tiles"], 8))
        nbytes += 4 * enc["words"].size + 256 * nt + 8 * (nt + 1) + 24 * nt + 12 * nb8 + 16384 * int(enc["K"]) + 16 * Q \
            + 20 * len(enc["esc_idx"])
        nweights += Q * P
        mod = QVBandLinearV8R(enc, device=dev) if world == 1 else \
            QVBandLinearV8RShard(enc, rank, world, device=dev, group=dist.group.WORLD)
        mods.append((name, mod, synth.synth_activation(M, P, seed=7 + j, device=dev)))
    t_build = time.perf_counter() - t0

    def eager_step():
        return [m(x) for _, m, x in mods]

    # The seven products of a layer are independent (each has its own input): one CUDA graph with a branch per
    # projection, so that small launches (a tensor has at most 4096 tiles = warps) share the machine, replayed per step.
    # Multi-rank runs stay eager (a library all-gather per projection).
    replay = "eager"
    step = eager_step
    if world == 1:
        try:
            for _ in range(2):
                eager_step()
            torch.cuda.synchronize(dev)
            main_s = torch.cuda.Stream(dev)
            side = [torch.cuda.Stream(dev) for _ in mods]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=main_s, capture_error_mode="thread_local"):
                cur = torch.cuda.current_stream(dev)
                graph_outs = []
                for (_, m, x), st in zip(mods, side):
                    st.wait_stream(cur)
                    with torch.cuda.stream(st):
                        graph_outs.append(m(x))
                for st in side:
                    cur.wait_stream(st)
            torch.cuda.synchronize(dev)
            # the replayed graph must give what the eager calls give
            want = eager_step()
            graph.replay()
            torch.cuda.synchronize(dev)
            if all(torch.equal(a, b) for a, b in zip(graph_outs, want)):
                replay = "one CUDA graph, a branch per projection"

                def step():
                    graph.replay()
                    return graph_outs
        except RuntimeError as e:
            print(f"[bench] qvb8r: graph capture unavailable ({str(e)[:120]}); eager launches", file=sys.stderr, flush=True)
            torch.cuda.synchronize(dev)
    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    hx = [x.cpu().pin_memory() for *_, x in mods]
    def e2e_step():
        if replay != "eager":
            for (_, _, x), h in zip(mods, hx):
                x.copy_(h, non_blocking=True)
            return step()[-1].float().cpu()
        outs = [m(h.to(dev, non_blocking=True)) for (_, m, _), h in zip(mods, hx)]
        return outs[-1].float().cpu()
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        if rank != 0:
            finish(world, dist)
            return
    peak, peak_kind = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "qvb8r_coded_stream_bytes_per_s", "value": gbs, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"27B-class layer, 7 projections as QVB8R packs (tau 2e-3), M={M}" + (f", rows / {div}" if div > 1 else ""),
                   "weights": nweights, "bytes": nbytes, "bits_per_weight": 8.0 * nbytes / nweights,
                   "weights_per_s": nweights / (ms * 1e-3), "pack_build_s": round(t_build, 1),
                   "l2": "coded streams of the layer exceed the L2" if nbytes > (126 << 20) else "working set fits the L2",
                   "launches": replay,
                   "parallelism": (f"every tensor split by tiles into {world} runs of about equal coded words; the ranks' "
                                   "output rows exchanged by one NCCL all-gather per projection") if world > 1 else "single GPU"},
        "clocks": clocks.summary(), "gpu_launches": 2 * len(mods) * args.steps,
        "e2e": {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": int(sum(h.numel() * h.element_size() for h in hx)),
                "d2h_bytes_per_step": int(mods[-1][1].out_features * M * 4), "ms_per_step": e2e_ms},
        "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "qvb8r_kernel",
                     "note": "bound by the entropy decoder's per-lane dependency chain, not by HBM"}}), flush=True)
    finish(world, dist)


def finish(world, dist):
    """Leave a multi-rank run without tearing NCCL down: communicators referenced by captured graphs make
    destroy_process_group wait for ever, so the ranks meet at a barrier, flush and exit."""
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="9b-dense")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--rows", type=int, default=1, help="activation rows M (1 = decode)")
    ap.add_argument("--policy", default="escape_outliers")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--shape", default="4096x4096", help="--workload single: QxP")
    ap.add_argument("--workload", default="stack", choices=["stack", "moe", "prefill", "single", "qvb8r"],
                    help="stack: the dense linear stack (headline); moe: one 35B-A3B-class expert layer; "
                         "prefill: 27B-class MLP projections for 2048 tokens on the tcgen05 kernel")
    ap.add_argument("--no-fuse", action="store_true", help="one launch per projection (no same-input fusion)")
    ap.add_argument("--group-layers", type=int, default=-1,
                    help="layers whose projections run behind one launch (0 = one launch per projection; "
                         "-1 = default: 32)")
    ap.add_argument("--shard", default="auto", choices=["auto", "pairs", "rows"],
                    help="N > 1: column/row-parallel pairs + all-reduce, or every projection by output rows + all-gather "
                         "(auto: rows below 8 activation rows, where the full-length rows stream faster; pairs from 8)")
    ap.add_argument("--nccl-allreduce", action="store_true", help="N > 1: NCCL all-reduce instead of the peer push kernel")
    ap.add_argument("--no-alt-policy", action="store_true", help="skip the second measurement with the in-band encoder policy")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from qvb8_b200 import stack as S
    cfg = S.CONFIGS[args.config]
    if args.workload == "moe" and args.impl != "reference":
        run_moe(args)
        return
    if args.workload == "prefill" and args.impl != "reference":
        run_prefill(args)
        return
    if args.workload == "single" and args.impl != "reference":
        run_single(args)
        return
    if args.workload == "qvb8r" and args.impl != "reference":
        run_qvb8r(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the kernels have no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from qvb8_b200 import lib
    lib.load()
    t_build = time.perf_counter()
    shard = args.shard if args.shard != "auto" else ("rows" if args.rows < 8 else "pairs")
    if world == 1:
        shard = "pairs"
    st = S.LinearStack(cfg, args.rows, dev, layers=args.layers, rank=rank, world=world, policy=args.policy,
                       fuse_same_input=not args.no_fuse, shard=shard)
    torch.cuda.synchronize(dev)
    t_build = time.perf_counter() - t_build

    allreduce_kind = None
    if world > 1:
        # all-reduce after o and after down: the only exchanges of a layer.  The push kernel over peer memory is checked
        # once against NCCL on seeded data; if the peers cannot map each other's memory the stack keeps NCCL.
        allreduce_kind = "nccl"
        if not args.nccl_allreduce:
            try:
                st.enable_collectives(peer=True)
                # two sizes: one (M, d_model) block and the largest exchange of a list launch (several blocks of the
                # push kernel), each twice so that both flag parities are used
                good = True
                for numel in (args.rows * cfg.d_model, st.peer.cap, st.peer.cap, args.rows * cfg.d_model):
                    probe = torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(rank + numel))
                    mine = st.peer.allreduce(probe.clone())
                    ref = probe.clone()
                    dist.all_reduce(ref)
                    torch.cuda.synchronize(dev)
                    good = good and bool(torch.allclose(mine, ref, rtol=1e-5, atol=1e-5))
                    got = st.peer.allgather(probe, torch.empty(world * numel, device=dev))
                    want = torch.empty(world * numel, device=dev)
                    dist.all_gather_into_tensor(want, probe)
                    torch.cuda.synchronize(dev)
                    good = good and bool(torch.equal(got, want))
                good = good and lib.device_status() == 0
                ok = torch.tensor([1 if good else 0], device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if int(ok.item()) == 1:
                    allreduce_kind = "peer push kernel (checked against NCCL)"
                else:
                    st.peer = None
            except RuntimeError as e:
                if rank == 0:
                    print(f"[bench] peer all-reduce unavailable ({e}); using NCCL", file=sys.stderr, flush=True)
                st.enable_collectives(peer=False)
        else:
            st.enable_collectives(peer=False)

    group_layers = args.group_layers if args.group_layers >= 0 else 32
    if group_layers > 0:
        st.set_grouping(group_layers)

    def one_step():
        st.step()

    st.capture()
    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    # The timed block is exactly --steps steps between two CUDA events.  A block of a few dozen milliseconds is too
    # short to read clocks by, so blocks are repeated until about a second has passed (the same number on every rank)
    # and the MEDIAN block is reported, with the spread and the clock samples of the whole second.
    block_ms = []
    with ClockSampler(local) as clocks:
        t_start = time.perf_counter()
        while True:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            ev0.record()
            for _ in range(args.steps):
                one_step()
            ev1.record()
            torch.cuda.synchronize(dev)
            block_ms.append(ev0.elapsed_time(ev1))
            go_on = torch.tensor([1 if (time.perf_counter() - t_start < 1.0 and len(block_ms) < 400) else 0], device=dev)
            if world > 1:
                dist.broadcast(go_on, 0)
            if int(go_on.item()) == 0:
                break
    if world > 1:                                        # per block the slowest rank, then the median block
        t = torch.tensor(block_ms, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        block_ms = t.tolist()
    ms = statistics.median(block_ms)
    if world > 1:
        tot = torch.tensor([st.compressed_bytes, st.n_weights, st.launches_per_step, st.kernels_per_step()], device=dev,
                           dtype=torch.int64)
        dist.all_reduce(tot)
        total_bytes, total_weights, launches, kernels = (int(v) for v in tot.tolist())
    else:
        total_bytes, total_weights, launches = st.compressed_bytes, st.n_weights, st.launches_per_step
        kernels = st.kernels_per_step()
    ms_step = ms / args.steps
    gbs = total_bytes / (ms_step * 1e-3) / 1e9

    # end to end through the host-buffer API
    for _ in range(3):
        st.step_host()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        st.step_host()
    e2e_s = (time.perf_counter() - t0) / args.steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_gbs = total_bytes / e2e_s / 1e9

    # the same stack with the encoder's other policy (outliers kept in band: 8-bit rows, no escape list), one GPU only
    alt = None
    if world == 1 and args.policy == "escape_outliers" and not args.no_alt_policy:
        st2 = S.LinearStack(cfg, args.rows, dev, layers=args.layers, policy="inband", fuse_same_input=not args.no_fuse)
        if group_layers > 0:
            st2.set_grouping(group_layers)
        st2.capture()
        for _ in range(args.warmup):
            st2.step()
        blocks = []
        t_start = time.perf_counter()
        while time.perf_counter() - t_start < 0.5 or len(blocks) < 3:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            e0.record()
            for _ in range(args.steps):
                st2.step()
            e1.record()
            torch.cuda.synchronize(dev)
            blocks.append(e0.elapsed_time(e1) / args.steps)
        ms2 = statistics.median(blocks)
        alt = {"policy": "inband (8-bit rows, no escapes)", "ms_per_step": ms2, "compressed_bytes": st2.compressed_bytes,
               "value": st2.compressed_bytes / (ms2 * 1e-3) / 1e9, "unit": UNIT,
               "bits_per_weight": 8.0 * st2.compressed_bytes / max(1, st2.n_weights), "tokens_per_s": 1e3 / ms2 * args.rows}
        del st2

    if rank != 0:
        finish(world, dist)
        return

    peak, peak_kind = measured_peaks()
    if alt is not None:
        alt["frac_of_hbm_peak"] = alt["value"] / peak
    per_launch_bytes = total_bytes / max(1, launches)
    line = {
        "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"{cfg.name} linear stack ({st.layers} layers x q,k,v,o,gate,up,down), decode M={args.rows}, "
                        f"QVB8 tau={cfg.tau}, policy={args.policy}",
            "launches_per_step": st.launches_per_step,
            "projections_per_launch": (f"{st.group_layers} layers x 4 fused projections behind one launch (the stack's "
                                       "projections read resident inputs and are independent)") if st._groups else "one",
            "timed_blocks": {"blocks": len(block_ms), "steps_per_block": args.steps, "reported": "median",
                             "min_ms_per_step": min(block_ms) / args.steps, "max_ms_per_step": max(block_ms) / args.steps},
            "same_input_fusion": "q+k+v and gate+up each run as one pack and one launch" if st.fused else "off",
            "weights": total_weights, "compressed_bytes": total_bytes,
            "bits_per_weight": 8.0 * total_bytes / max(1, total_weights),
            "row_width_hist": {str(k): v for k, v in sorted(st.width_hist.items())}, "escapes": st.n_escapes,
            "parallelism": ((f"column/row-parallel pairs x{world}; the partial sums of o and down are exchanged by "
                             f"{'one all-reduce per launch' if st._groups else 'two all-reduces per layer'} ({allreduce_kind})")
                            if shard == "pairs" else
                            (f"every projection split by output rows x{world}; each rank's slices of the o and down outputs "
                             f"and of their inputs are exchanged by one all-gather per "
                             f"{'launch' if st._groups else 'layer'} ({allreduce_kind})"))
                           if world > 1 else "single GPU",
            "l2": "working set (packs) far larger than L2; every step streams all of it",
            "tokens_per_s": 1e3 / ms_step * args.rows, "pack_build_s": round(t_build, 1),
            "other_encoder_policy": alt,
        },
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_gbs, "unit": UNIT, "h2d_bytes_per_step": st.h2d_bytes(), "d2h_bytes_per_step": st.d2h_bytes(),
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": kernels * args.steps,
        "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                     # dram bytes per launch: ncu measured 89.6 MB read + 0.1 MB written for the 89.3 MB launch (gate+up,
                     # 24576 x 4096); traffic grows with the streamed bytes, so the ratio is applied to the average launch
                     "traffic": per_launch_bytes * DRAM_TRAFFIC_RATIO, "traffic_kind": "scaled from one ncu capture",
                     "peak_kind": peak_kind, "kernel": "small_m_kernel",
                     "bytes_per_launch_avg": per_launch_bytes,
                     "launches_per_step": launches // max(1, world), "avg_launch_us": ms_step * 1e3 / max(1, launches // max(1, world)),
                     "note": "achieved = algorithmic (compressed) bytes per launch / average launch duration, the latter "
                             "= CUDA-event step time / launches of the step (back-to-back launches of the one kernel, gaps "
                             "included)"},
    }
    if world == 1:
        import oracle
        threads = oracle.num_threads()
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        sample = build_cpu_sample(cfg)
        cpu_reference_step(sample, threads)
        t0 = time.perf_counter()
        nb = 0
        reps = 0
        while time.perf_counter() - t0 < args.cpu_seconds:
            nb += cpu_reference_step(sample, threads)
            reps += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": nb / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"layer-0 q,k,v,o packs, M=1, restore to bf16 (C restatement of the reference "
                                          f"decoder, OpenMP) + torch.matmul on CPU, {reps} repetitions in {dt:.1f} s"}
    print(json.dumps(line), flush=True)
    finish(world, dist)


if __name__ == "__main__":
    main()
