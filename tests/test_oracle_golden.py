"""The CPU oracle against the golden fixtures (outputs of the reference's own Python decoders)."""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN, golden_cases
from qvb8_b200 import packs


def _load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return z, packs.read_qvb8(z["blob"].tobytes())


@pytest.mark.parametrize("name", golden_cases())
def test_ids_match_reference_unpack(name):
    z, pk = _load(name)
    ids = oracle.unpack_ids(pk["ids"], pk["nbits"], pk["bit_off"], pk["Q"], pk["P"])
    assert np.array_equal(ids, z["ids"])


@pytest.mark.parametrize("name", golden_cases())
def test_restore_bit_exact_with_reference_reconstruct(name):
    z, pk = _load(name)
    w = oracle.qvb8_dense(pk, table="bf16")            # the fixture applies the pack's full escape list
    assert np.array_equal(w.view(np.uint32), z["w32"].view(np.uint32))


@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_dense_16bit_restore(name, kind):
    z, pk = _load(name)
    got = oracle.decode_16(pk["ids"], pk["nbits"], pk["bit_off"], pk["min_s"], pk["tau_s"], pk["Q"], pk["P"],
                           pk["esc_idx_bf16"], pk["esc_vals_bf16"], kind)
    assert np.array_equal(got, z["w16_bits" if kind == "f16" else "wbf_bits"])


@pytest.mark.parametrize("name", golden_cases())
def test_certificate_holds(name):
    z, pk = _load(name)
    src = torch.from_numpy(z["source_bits"].view(np.int16)).view(torch.bfloat16).double().numpy()
    w16 = z["w16_bits"].view(np.float16).astype(np.float64)
    assert np.abs(w16 - src).max() <= pk["tau"] * (1 + 1e-6)


def test_rounding_helpers_match_numpy_and_torch():
    rng = np.random.default_rng(5)
    a = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  6.1e-5, 5.96e-8, np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.f32_to_f16_bits(a), a.astype(np.float16).view(np.uint16))
    want = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_bits(a), want)
    sat = oracle.sat_half(a)
    with np.errstate(over="ignore"):
        ref = np.clip(a, -65504, 65504).astype(np.float16).astype(np.float32)
    assert np.array_equal(sat, ref)


def test_matmul_oracle_matches_float64():
    rng = np.random.default_rng(1)
    W = rng.standard_normal((37, 96)).astype(np.float32)
    X = rng.standard_normal((5, 96)).astype(np.float32)
    got = oracle.matmul_f32w(X, W, narrow_x=True)
    Xn = X.astype(np.float16).astype(np.float64)
    assert np.allclose(got, Xn @ W.astype(np.float64).T, rtol=1e-12, atol=1e-12)
