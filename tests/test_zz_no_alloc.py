"""qvb8_small_m_static: the streaming product with its scratch in a fixed array of the loaded module (no allocation
anywhere in the call).  Named to be collected last; passes alone and after every other GPU test."""
import ctypes

import pytest
import torch

from qvb8_b200 import synth
from util import random_pack

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, L, st, plan, X, Y, flags=0):
    with torch.cuda.device(X.device):
        return L.qvb8_small_m_static(ctypes.byref(st), plan.data_ptr(), X.data_ptr(), lib.dtype_code(X.dtype), 0,
                                     X.shape[0], Y.data_ptr(), flags, lib.stream_ptr(X.device))


def test_static_scratch_matches_the_regular_entry_point(cuda_lib):
    from qvb8_b200 import lib
    L = lib.load()
    assert L.qvb8_small_m_static_max_scratch() == 4 << 20
    # M = 8 at P = 4096: the staged activations do not fit beside the rings, so K is split into ranges and the
    # kernel really uses partial-result slots and tickets
    pk = random_pack(512, 4096, (6, 7, 8), seed=77, esc_frac=0.002, device=DEV)
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
    plan = lib.build_plan(st, keep)
    need = int(L.qvb8_small_m_scratch_bytes(8, pk.Q, pk.P))
    assert 0 < need <= 4 << 20
    for seed in (1, 2):                                   # two consecutive calls: the array is reused as it was left
        X = synth.synth_activation(8, pk.P, seed=seed, device=DEV)
        want = lib.small_m(st, keep, X, plan=plan)
        got = torch.full_like(want, float("nan"))
        rc = _call_static(lib, L, st, plan, X, got)
        assert rc == 0, L.qvb8_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    # a shape that needs no scratch at all goes through as well
    X1 = synth.synth_activation(1, pk.P, seed=3, device=DEV)
    want1 = lib.small_m(st, keep, X1, plan=plan)
    got1 = torch.empty_like(want1)
    assert _call_static(lib, L, st, plan, X1, got1) == 0
    torch.cuda.synchronize()
    assert torch.equal(got1, want1)
    assert lib.device_status() == 0


def test_static_scratch_refuses_what_does_not_fit(cuda_lib):
    from qvb8_b200 import lib
    L = lib.load()
    Q, P, M = 32768, 4096, 48
    assert int(L.qvb8_small_m_scratch_bytes(M, Q, P)) > 4 << 20
    # only the sizes matter for the refusal: a pack header with the big Q over small buffers is never dereferenced
    pk = random_pack(64, P, (7,), seed=5, device=DEV)
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
    big = type(st)(st.ids, st.ids_bytes, st.min_s, st.tau_s, st.nbits, st.bit_off, Q, P, None, None, 0)
    plan = lib.build_plan(st, keep)
    X = synth.synth_activation(M, P, seed=1, device=DEV)
    Y = torch.zeros(M, 64, device=DEV)
    rc = _call_static(lib, L, big, plan, X, Y)
    assert rc != 0
    msg = L.qvb8_last_error().decode()
    assert "built-in array" in msg and "qvb8_small_m_ex" in msg
    torch.cuda.synchronize()
    assert float(Y.abs().sum()) == 0.0                    # nothing was launched
