"""Grouped expert MLP (reference qvb8_moe_experts_forward / _relu2_forward, qvb8_cuda.cu:949-1058) against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import experts, synth
from qvb8_b200.ext_qvb8 import ext
from util import pack_np, random_pack, rel_fro

DEV = "cuda:0"
TOL = 1e-2          # stated tolerance: relative Frobenius against the reference kernel / a dense product
TIGHT = 2e-4        # what fp32 accumulation actually gives


def _experts(E, Qup, P, Qdn, hidden, widths, seed):
    ups = [random_pack(Qup, P, widths, seed=seed + e) for e in range(E)]
    dns = [random_pack(Qdn, hidden, widths, seed=seed + 100 + e) for e in range(E)]
    return ups, dns


def _routing(M, E, topk, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(M, E, generator=g)
    w, idx = torch.topk(torch.softmax(logits, -1), topk, dim=-1)
    return idx.to(torch.int64), (w / w.sum(-1, keepdim=True)).float()


def test_stack_layout_cpu():
    ups, _ = _experts(3, 16, 64, 64, 8, (5, 7), seed=1)
    st = experts.stack_packs(ups)
    assert st["min_s"].shape == (3, 16) and st["bit_off"].shape == (3, 16) and st["ids"].numel() % 16 == 0
    for e, m in enumerate(ups):
        base = int(st["bit_off"][e, 0]) // 8
        assert base % 16 == 0
        n = m.ids.numel() - 8
        assert torch.equal(st["ids"][base:base + n], m.ids[:n])
        assert torch.equal(st["bit_off"][e] - base * 8, m.bit_off)
    bad = random_pack(16, 64, (7,), seed=9, esc_frac=0.01)
    with pytest.raises(ValueError):
        experts.stack_packs([ups[0], bad])


def test_expert_range_of_a_rank_cpu():
    """a rank's module names its experts' place in the whole layer; ranges outside the layer are refused"""
    ups, dns = _experts(4, 16, 64, 64, 8, (5, 7), seed=3)
    whole = experts.QVBandExpertsV8(ups, dns, num_experts=4)
    assert not whole.sharded and whole.first_expert == 0 and whole.total_experts == 4
    part = experts.QVBandExpertsV8(ups[2:], dns[2:], num_experts=2, first_expert=2, total_experts=4)
    assert part.sharded and part.up["min_s"].shape == (2, 16)
    part.set_reduce(None)
    with pytest.raises(ValueError):
        experts.QVBandExpertsV8(ups[2:], dns[2:], num_experts=2, first_expert=3, total_experts=4)
    with pytest.raises(ValueError):
        experts.QVBandExpertsV8(ups, dns, num_experts=3)


@pytest.mark.gpu
@pytest.mark.parametrize("act", ["silu", "relu2"])
@pytest.mark.parametrize("M,dtype", [(1, torch.bfloat16), (5, torch.float16), (19, torch.float32)])
def test_moe_matches_oracle(cuda_lib, act, M, dtype):
    E, topk, P, hidden, Qdn = 10, 3, 256, 96, 256
    Qup = 2 * hidden if act == "silu" else hidden
    ups, dns = _experts(E, Qup, P, Qdn, hidden, (4, 6, 7, 8, 10), seed=40 + M)
    mod = experts.QVBandExpertsV8([u.to(DEV) for u in ups], [d.to(DEV) for d in dns], num_experts=E, act=act)
    idx, w = _routing(M, E, topk, seed=M)
    X = synth.synth_activation(M, P, seed=3, device=DEV, dtype=dtype) * 0.5
    out = mod(X, idx.to(DEV), w.to(DEV))
    assert out.dtype == dtype and tuple(out.shape) == (M, Qdn)
    upd = np.stack([oracle.qvb8_dense(pack_np(u)) for u in ups])
    dnd = np.stack([oracle.qvb8_dense(pack_np(d)) for d in dns])
    want = oracle.moe_experts(X.float().cpu().numpy(), idx.numpy(), w.numpy(), upd, dnd, act)
    err = rel_fro(out.float().cpu().numpy(), want)
    tol = TIGHT if dtype == torch.float32 else 6e-3          # bf16 / fp16 outputs carry their own rounding
    assert err < TOL and err < tol, err
    again = mod(X, idx.to(DEV), w.to(DEV))
    assert torch.equal(out, again)                           # fixed summation order


@pytest.mark.gpu
@pytest.mark.parametrize("act", ["silu", "relu2"])
@pytest.mark.parametrize("M,dtype", [(1, torch.bfloat16), (3, torch.float32), (8, torch.float16), (8, torch.float32)])
def test_streaming_route_matches_oracle(cuda_lib, act, M, dtype):
    """up to 8 tokens and column counts that are multiples of 128: every distinct expert runs as a job of the streaming
    kernel from a job table written on the device; hidden activations are scaled by powers of two around the fp16
    staging (checked here with inputs large enough that unscaled hidden values would leave the fp16 range)"""
    import ctypes
    from qvb8_b200 import lib
    E, topk, P, hidden, Qdn = 12, 4, 256, 128, 256
    Qup = 2 * hidden if act == "silu" else hidden
    ups, dns = _experts(E, Qup, P, Qdn, hidden, (4, 6, 7, 8, 10), seed=60 + M)
    mod = experts.QVBandExpertsV8([u.to(DEV) for u in ups], [d.to(DEV) for d in dns], num_experts=E, act=act)
    u, d = mod.up, mod.down
    ust = lib.expert_stack_struct(u["ids"], u["min_s"], u["tau_s"], u["nbits"], u["bit_off"], u["Q"], u["P"])
    dst = lib.expert_stack_struct(d["ids"], d["min_s"], d["tau_s"], d["nbits"], d["bit_off"], d["Q"], d["P"])
    assert lib.load().qvb8_moe_streams(M, topk, E, ctypes.byref(ust[0]), ctypes.byref(dst[0])) == 1
    idx, w = _routing(M, E, topk, seed=M + 1)
    scale = 200.0 if dtype != torch.float16 else 4.0           # hidden values of 1e5 and more: beyond the fp16 range
    X = synth.synth_activation(M, P, seed=4, device=DEV, dtype=dtype) * scale
    out = mod(X, idx.to(DEV), w.to(DEV))
    assert out.dtype == dtype and tuple(out.shape) == (M, Qdn)
    upd = np.stack([oracle.qvb8_dense(pack_np(a)) for a in ups])
    dnd = np.stack([oracle.qvb8_dense(pack_np(b)) for b in dns])
    want = oracle.moe_experts(X.float().cpu().numpy(), idx.numpy(), w.numpy(), upd, dnd, act)
    assert np.isfinite(want).all()
    err = rel_fro(out.float().cpu().numpy(), want)
    tol = 1e-3 if dtype == torch.float32 else 6e-3           # fp32: the 2^-11 rounding of the hidden values
    assert err < TOL and err < tol, err
    assert torch.equal(out, mod(X, idx.to(DEV), w.to(DEV)))  # fixed summation order
    assert lib.device_status() == 0


@pytest.mark.gpu
def test_moe_config_shape_and_bad_index(cuda_lib):
    """The benchmark's expert shapes (d_model 2048, expert FFN 768) at a few tokens; an out-of-range expert index is
    reported and touches nothing out of range."""
    from qvb8_b200 import lib
    E, topk, P, hidden = 16, 8, 2048, 768
    ups, dns = _experts(E, 2 * hidden, P, P, hidden, (6, 7), seed=7)
    mod = experts.QVBandExpertsV8([u.to(DEV) for u in ups], [d.to(DEV) for d in dns], num_experts=E)
    M = 8
    idx, w = _routing(M, E, topk, seed=11)
    X = synth.synth_activation(M, P, seed=5, device=DEV) * 0.25
    out = mod(X, idx.to(DEV), w.to(DEV))
    upd = np.stack([oracle.qvb8_dense(pack_np(u)) for u in ups])
    dnd = np.stack([oracle.qvb8_dense(pack_np(d)) for d in dns])
    want = oracle.moe_experts(X.float().cpu().numpy(), idx.numpy(), w.numpy(), upd, dnd, "silu")
    assert rel_fro(out.float().cpu().numpy(), want) < 6e-3
    # bad index
    L = lib.load()
    u, d = mod.up, mod.down
    ust = lib.expert_stack_struct(u["ids"], u["min_s"], u["tau_s"], u["nbits"], u["bit_off"], u["Q"], u["P"])
    dst = lib.expert_stack_struct(d["ids"], d["min_s"], d["tau_s"], d["nbits"], d["bit_off"], d["Q"], d["P"])
    bad_idx = idx.clone()
    bad_idx[0, 0] = E + 5
    import ctypes
    nbytes = int(L.qvb8_moe_scratch_bytes(M, topk, E, u["P"], u["Q"], d["Q"], 0))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    o = torch.empty(M, d["Q"], dtype=X.dtype, device=DEV)
    bi, wd = bad_idx.to(DEV), w.to(DEV)
    rc = L.qvb8_moe_experts(X.data_ptr(), lib.dtype_code(X.dtype), M, bi.data_ptr(), wd.data_ptr(), topk, E,
                            ctypes.byref(ust[0]), ctypes.byref(dst[0]), 0, o.data_ptr(), scratch.data_ptr(), nbytes,
                            lib.stream_ptr(torch.device(DEV)))
    assert rc == 0
    flag = ctypes.c_int(0)
    assert L.qvb8_moe_bad_index(scratch.data_ptr(), M, topk, E, u["P"], u["Q"], d["Q"], 0, ctypes.byref(flag)) == 0
    assert flag.value == 1
    assert lib.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_shards_sum_to_the_whole(cuda_lib, world):
    """experts split over `world` ranks (here: modules on one device, run one after the other), tokens and routing
    replicated: the ranks' fp32 partial outputs add up to the unsharded layer's output, and a shard asked alone returns
    only its own experts' contributions"""
    E, topk, P, hidden, M = 8, 3, 256, 64, 6
    ups, dns = _experts(E, 2 * hidden, P, P, hidden, (5, 7, 8), seed=21)
    ups, dns = [u.to(DEV) for u in ups], [d.to(DEV) for d in dns]
    whole = experts.QVBandExpertsV8(ups, dns, num_experts=E)
    idx, w = _routing(M, E, topk, seed=3)
    X = synth.synth_activation(M, P, seed=8, device=DEV, dtype=torch.float32) * 0.5
    want = whole(X, idx.to(DEV), w.to(DEV))
    per = E // world
    parts = []
    for r in range(world):
        shard = experts.QVBandExpertsV8(ups[r * per:(r + 1) * per], dns[r * per:(r + 1) * per], num_experts=per,
                                        first_expert=r * per, total_experts=E)
        assert shard.sharded
        parts.append(shard(X, idx.to(DEV), w.to(DEV)))
        # the same shard with the other ranks' pairs given weight zero on the whole layer
        mask = ((idx >= r * per) & (idx < (r + 1) * per)).float()
        alone = whole(X, idx.to(DEV), (w * mask).to(DEV))
        assert float((parts[-1] - alone).abs().max()) <= 1e-5 * float(want.abs().max())
    total = torch.stack(parts).sum(0)
    assert float((total - want).abs().max()) <= 1e-5 * float(want.abs().max())
    # the reduce hook receives the fp32 partial sums; the result comes back in the activations' type
    seen = []
    shard.set_reduce(lambda t: seen.append(t.dtype) or t * 2)
    out = shard(X.to(torch.bfloat16), idx.to(DEV), w.to(DEV))
    assert seen == [torch.float32] and out.dtype == torch.bfloat16
    from qvb8_b200 import lib
    assert lib.device_status() == 0


@pytest.mark.gpu
def test_moe_full_size_properties(cuda_lib):
    """The 35B-A3B-class layer at its full size (128 experts, top-8, d_model 2048, expert FFN 768, 32 tokens): too
    large for the oracle, so size-independent properties are checked: doubling the routing weights doubles the result
    exactly; reordering the tokens reorders the rows bit for bit; a token computed alone agrees with its row."""
    E, topk, d, f, M = 128, 8, 2048, 768, 32
    ups = [synth.encode_qvb8(synth.synth_weight(2 * f, d, 4000 + e, device=DEV), tau=1e-3, policy="inband") for e in range(E)]
    dns = [synth.encode_qvb8(synth.synth_weight(d, f, 5000 + e, device=DEV), tau=1e-3, policy="inband") for e in range(E)]
    mod = experts.QVBandExpertsV8(ups, dns, num_experts=E)
    idx, w = _routing(M, E, topk, seed=3)
    idx, w = idx.to(DEV), w.to(DEV)
    X = synth.synth_activation(M, d, seed=9, device=DEV, dtype=torch.float32)
    out = mod(X, idx, w)
    assert out.shape == (M, d) and bool(torch.isfinite(out).all())
    assert torch.equal(mod(X, idx, w * 2), out * 2)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(1)).to(DEV)
    assert torch.equal(mod(X[perm].contiguous(), idx[perm].contiguous(), w[perm].contiguous()), out[perm])
    for t in (0, 17, 31):
        one = mod(X[t:t + 1].contiguous(), idx[t:t + 1].contiguous(), w[t:t + 1].contiguous())
        # (a single token takes the streaming route: its hidden activations pass through fp16 with 2^-11 rounding)
        assert rel_fro(one.cpu().numpy(), out[t:t + 1].cpu().numpy()) < 1e-3
    # eight tokens, the streaming route at full size: the same properties
    X8, idx8, w8 = X[:8].contiguous(), idx[:8].contiguous(), w[:8].contiguous()
    out8 = mod(X8, idx8, w8)
    assert rel_fro(out8.cpu().numpy(), out[:8].cpu().numpy()) < 1e-3
    assert torch.equal(mod(X8, idx8, w8 * 2), out8 * 2)
    p8 = torch.randperm(8, generator=torch.Generator().manual_seed(2)).to(DEV)
    assert torch.equal(mod(X8[p8].contiguous(), idx8[p8].contiguous(), w8[p8].contiguous()), out8[p8])
    from qvb8_b200 import lib
    assert lib.device_status() == 0
