"""The embedding row gather against the reference's arithmetic (min_s + id * tau_s, escapes written over, one cast)."""
import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import lib
from qvb8_b200.embedding import QVBandEmbeddingV8
from util import pack_np, random_pack

DEV = "cuda:0"


def _expected(pk, rows, dtype):
    d = pack_np(pk)
    ids = oracle.unpack_ids(d["ids"], d["nbits"], d["bit_off"], d["Q"], d["P"]).astype(np.float32)     # (Q, P)
    W = (d["min_s"].astype(np.float32)[:, None] + ids * d["tau_s"].astype(np.float32)[:, None]).astype(np.float32)
    W.reshape(-1)[d["esc_idx"]] = d["esc_vals"]
    return torch.from_numpy(W[rows]).to(dtype)


def test_module_keeps_fp32_metadata_on_cpu():
    pk = random_pack(40, 64, (5, 7), seed=2, esc_frac=0.01)
    emb = QVBandEmbeddingV8.from_pack(pk)
    emb.to(torch.bfloat16)
    assert emb.min_s.dtype == torch.float32 and emb.esc_vals.dtype == torch.float32
    with pytest.raises(RuntimeError):
        emb(torch.tensor([1, 2]))                       # no CUDA device: the product path refuses, it does not fall back


@pytest.mark.gpu
@pytest.mark.parametrize("widths,esc", [((7,), 0.0), ((3, 6, 8, 11, 14), 0.01)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rows_bit_exact(cuda_lib, widths, esc, dtype):
    Q, P = 300, 320
    pk = random_pack(Q, P, widths, seed=len(widths), esc_frac=esc, device=DEV)
    emb = QVBandEmbeddingV8.from_pack(pk, out_dtype=dtype)
    idx = torch.tensor([[0, 299, 17], [17, 5, 128]], device=DEV)
    got = emb(idx)
    assert got.shape == (2, 3, P) and got.dtype == dtype
    want = _expected(pk, idx.reshape(-1).cpu().numpy(), dtype)
    assert torch.equal(got.reshape(-1, P).cpu(), want)
    assert torch.equal(emb.weight.cpu(), _expected(pk, np.arange(Q), dtype))
    with pytest.raises(IndexError):
        emb(torch.tensor([Q], device=DEV))
    assert lib.device_status() == 0
