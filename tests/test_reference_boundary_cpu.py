"""The drop-in boundary against the REFERENCE's own modules (build container only: skipped where the reference
checkout is absent, e.g. on a GPU box).

The reference's ``QVBandLinearV8`` / ``QVBandLinearV8R`` fetch their kernels through ``_load_ext()``;
``ext_qvb8.install()`` / ``ext_qvb8r.install()`` rebind that loader.  Here the reference modules are imported
unmodified, the loaders are rebound, and a recording stand-in with THIS package's extension signatures answers the
calls with oracle-computed values on the CPU: every call the reference makes must bind to the shim's signature, and the
module's result must be the product with the restored weight.  Separately, the entry-point names registered in the
reference's ``PYBIND11_MODULE`` blocks (read from the .cu text) must all exist on the shims.
"""
import inspect
import os
import re
import sys

import numpy as np
import pytest
import torch

import oracle
from oracle import build_ref
from qvb8_b200 import ext_qvb8, ext_qvb8r, packs, rans, synth

REF = build_ref.reference_root()
pytestmark = pytest.mark.skipif(REF is None, reason="reference checkout not present on this machine")


@pytest.fixture(scope="module")
def ref_modules():
    sys.path.insert(0, os.path.join(REF, "src"))
    try:
        import qv_band.formats.qvb8.module as m8
        import qv_band.formats.qvb8r.module as m8r
        yield m8, m8r
    finally:
        sys.path.remove(os.path.join(REF, "src"))


def _registered(cu_path):
    text = open(cu_path).read()
    block = text[text.index("PYBIND11_MODULE"):]
    return re.findall(r'm\.def\("(\w+)"', block)


def test_every_registered_entry_point_exists_on_the_shims():
    q = _registered(os.path.join(REF, "src/qv_band/formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu"))
    r = _registered(os.path.join(REF, "src/qv_band/formats/qvb8r/backends/cuda_qvb8r/qvb8r_cuda.cu"))
    assert len(q) >= 10 and len(r) >= 9
    for name in q:
        assert callable(getattr(ext_qvb8.ext, name, None)), f"qvb8 shim lacks {name}"
    for name in r:
        assert callable(getattr(ext_qvb8r.ext, name, None)), f"qvb8r shim lacks {name}"
    assert "bf16" in (ext_qvb8.ext.mma_multi.__doc__ or "")           # the reference module looks for this word


class Recorder:
    """Stands in for the kernels on a machine without a GPU: binds every call to the real shim's signature, records
    it, and answers with values computed by the CPU oracle."""

    def __init__(self, shim, answers):
        self.shim, self.answers, self.calls = shim, answers, []

    def __getattr__(self, name):
        real = getattr(self.shim, name)                                # AttributeError for names the shim lacks

        def call(*args, **kwargs):
            inspect.signature(real).bind(*args, **kwargs)              # TypeError if the reference's call does not fit
            self.calls.append(name)
            return self.answers[name](*args, **kwargs)
        call.__doc__ = real.__doc__
        return call


def test_reference_qvb8_linear_runs_on_the_rebound_loader(ref_modules, monkeypatch):
    m8, _ = ref_modules
    Q, P = 48, 256
    pk, _W = synth.synth_pack(Q, P, 77, return_weight=True)
    from util import pack_np
    Wd = oracle.qvb8_dense(pack_np(pk))

    def product(X, ids, min_s, nbits, bit_off, P_, tau_s, esc_idx, esc_vals):
        assert ids.dtype == torch.uint8 and nbits.dtype == torch.uint8 and bit_off.dtype == torch.int64
        return torch.from_numpy(oracle.matmul_f32w(X.float().numpy().reshape(-1, P), Wd, narrow_x=True).astype(np.float32))

    def dense16(ids, min_s, nbits, bit_off, P_, tau_s, esc_idx, esc_vals):
        return torch.from_numpy(Wd).to(torch.float16)
    rec = Recorder(ext_qvb8.ext, dict(forward=product, gemv_multi=product, gemv=product, decode=dense16))
    monkeypatch.setattr(ext_qvb8, "ext", rec)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)   # no driver on a CPU-only machine
    ext_qvb8.install()
    assert m8._load_ext() is rec
    lin = m8.QVBandLinearV8.from_packfile(None, device="cpu", blob=pk.to_blob("QVBD"))
    for M in (1, 5, 20):
        X = synth.synth_activation(M, P, seed=M, dtype=torch.float32)
        y = lin(X)
        want = oracle.matmul_f32w(X.numpy(), Wd, narrow_x=True)
        assert y.shape == (M, Q)
        assert np.linalg.norm(y.double().numpy() - want) / np.linalg.norm(want) < 2e-3     # fp16 weights above 8 rows
    assert set(rec.calls) <= {"forward", "gemv_multi", "gemv", "decode"} and "forward" in rec.calls


def test_reference_qvb8r_linear_runs_on_the_rebound_loader(ref_modules, monkeypatch):
    _, m8r = ref_modules
    Q, P = 40, 256
    d = synth.encode_qvb8r(synth.synth_weight(Q, P, 5), tau=2e-3, K=2, T=4)
    blob = packs.write_qvb8r(d, Q=Q, P=P, min_s=d["min_s"], tau_s=d["tau_s"], esc_idx=d["esc_idx"], esc_val=d["esc_val"],
                             esc_delta=d["esc_delta"], cert=dict(tau=2e-3, max_err=d["max_err"], restore="fp16"))
    words = np.concatenate([d["words"], np.zeros(rans.PAD_WORDS, np.uint32)])
    ids = oracle.rans_decode_ids(words, d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64),
                                 oracle.slot_tables(d["freq"]), d["perm"], d["drow"].astype(np.int32), Q, P)
    band = oracle.rans_restore_f32(ids, d["min_s"], d["tau_s"])

    def check_core(core):
        want = (torch.int32, torch.int64, torch.int64, torch.int64, torch.int32, torch.int32, torch.int32, torch.float32,
                torch.float32, torch.int32)
        assert tuple(t.dtype for t in core) == want

    def gemv(X, *core):
        check_core(core)
        return torch.from_numpy((X.double().numpy().reshape(1, P) @ band.astype(np.float64).T).astype(np.float32)).reshape(-1)

    def multi(X, *core):
        check_core(core)
        return torch.from_numpy((X.double().numpy() @ band.astype(np.float64).T).astype(np.float32))

    def tc(X, *core_T):
        check_core(core_T[:-1])
        W16 = band.astype(np.float16).astype(np.float64)
        return torch.from_numpy((X.double().numpy() @ W16.T).astype(np.float32))

    def fix(X, uq, ptr, ec, ed, Y):
        for u in range(uq.numel()):
            for e in range(int(ptr[u]), int(ptr[u + 1])):
                Y[:, uq[u]] += X[:, ec[e]] * ed[e]
    rec = Recorder(ext_qvb8r.ext, dict(gemv=gemv, multi=multi, tc=tc, fix_escapes=fix))
    monkeypatch.setattr(ext_qvb8r, "ext", rec)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    ext_qvb8r.install()
    assert m8r._load_ext() is rec
    lin = m8r.QVBandLinearV8R.from_packfile("w.qvb8r", device="cpu", blob=blob)
    W = band.astype(np.float64).copy()
    W.reshape(-1)[d["esc_idx"]] = d["esc_val"]
    for M, tol in ((1, 1e-5), (6, 1e-5), (14, 2e-3)):
        X = synth.synth_activation(M, P, seed=M, dtype=torch.float32)
        y = lin(X)
        want = X.double().numpy() @ W.T
        assert np.linalg.norm(y.double().numpy() - want) / np.linalg.norm(want) < tol
    assert {"gemv", "multi", "tc", "fix_escapes"} <= set(rec.calls)


def test_install_binds_the_live_extension_object(ref_modules):
    m8, m8r = ref_modules
    ext_qvb8.install()
    ext_qvb8r.install()
    assert m8._load_ext() is ext_qvb8.ext and m8r._load_ext() is ext_qvb8r.ext
    import qv_band.formats.qvb8.backends_experts as be
    assert be._load_ext() is ext_qvb8.ext
