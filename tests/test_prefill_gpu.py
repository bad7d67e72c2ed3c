"""The tcgen05 prefill kernel (many tokens) against the oracle's dense fp32 product on the restored weights."""
import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import lib, synth
from util import pack_np, random_pack, rel_fro

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2          # the stated tolerance
TIGHT = 1e-4        # what exact products with fp32 accumulation give


def _run(pk, M, dtype, seed):
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
    plan = lib.build_plan(st, keep)
    X = synth.synth_activation(M, pk.P, seed=seed, device=DEV, dtype=dtype)
    Y = lib.prefill(st, keep, X, plan=plan)
    torch.cuda.synchronize()
    want = oracle.matmul_f32w(X.float().cpu().numpy(), oracle.qvb8_dense(pack_np(pk)), narrow_x=True)
    return Y, want


@pytest.mark.parametrize("Q,P,M,widths,esc", [
    (128, 64, 32, (7,), 0.0),                      # one CTA, one K block
    (256, 512, 100, (6, 7, 8), 0.0),               # two row tiles, ragged token tile
    (200, 1024, 300, (3, 5, 7, 8), 0.002),         # ragged rows, two token tiles, escapes
    (384, 256, 257, (4, 9, 12), 0.001),            # 12-bit rows are recomputed in fp32
    (300, 1280, 520, (1, 2, 10, 11, 14), 0.0),     # every unpack mode; 20 K blocks wrap the stage ring several times
    (1000, 2048, 64, (7,), 0.001),                 # one width: eight row tiles, deep K
    (130, 320, 40, (3, 6, 7, 8), 0.0),             # five K blocks: a partial super-stage, an odd last pair
    (64, 192, 16, (5, 7), 0.0),                    # rows that do not start on 16 bytes take the id-by-id path
])
def test_prefill_matches_oracle(cuda_lib, Q, P, M, widths, esc):
    pk = random_pack(Q, P, widths, seed=Q + M, esc_frac=esc, device=DEV)
    Y, want = _run(pk, M, torch.bfloat16, seed=M)
    err = rel_fro(Y.cpu().numpy(), want)
    assert err < TOL and err < TIGHT, err
    assert lib.device_status() == 0


def test_prefill_dtypes_and_determinism(cuda_lib):
    pk = random_pack(256, 512, (6, 7), seed=3, esc_frac=0.001, device=DEV)
    for dt in (torch.float16, torch.float32):
        Y, want = _run(pk, 64, dt, seed=9)
        assert rel_fro(Y.cpu().numpy(), want) < TIGHT
    a, _ = _run(pk, 200, torch.bfloat16, seed=4)
    b, _ = _run(pk, 200, torch.bfloat16, seed=4)
    assert torch.equal(a, b)
    assert lib.device_status() == 0


def test_prefill_full_size_agrees_with_the_streaming_kernel(cuda_lib):
    """27B-class down projection, 2048 tokens: too large for the oracle, so the tcgen05 kernel is checked against the
    streaming kernel (itself oracle-checked at small sizes) on sampled tokens, and on size-independent properties:
    zero activations give exactly zero, and f(2x) = 2 f(x) exactly (a power of two passes through every rounding)."""
    Q, P, M = 5120, 17408, 2048
    pk = synth.encode_qvb8(synth.synth_weight(Q, P, 77, device=DEV), tau=2e-3)
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
    plan = lib.build_plan(st, keep)
    X = synth.synth_activation(M, P, seed=5, device=DEV, dtype=torch.float16)
    X[X.abs() < 1e-3] = 0                                 # keep 2x exact: no fp16 subnormals
    Y = lib.prefill(st, keep, X, plan=plan)
    rows = torch.tensor([0, 1, 255, 256, 1000, 1535, 2046, 2047], device=DEV)
    Ys = lib.small_m(st, keep, X[rows].contiguous(), plan=plan)
    err = float((Y[rows] - Ys).norm() / Ys.norm())
    assert err < TIGHT, err
    assert torch.count_nonzero(lib.prefill(st, keep, torch.zeros_like(X), plan=plan)) == 0
    assert torch.equal(lib.prefill(st, keep, X * 2, plan=plan), Y * 2)
    assert lib.device_status() == 0
