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
