"""GPU parity tests of the QVB8 kernels (through the C ABI via the reference-shaped extension object).

Bars: restored weights bit-exact with the oracle and with the reference decoder's golden outputs; small-M products
within 1e-2 relative Frobenius of the oracle (the stated tolerance) -- in practice they sit near 1e-6, and the tests
also hold them to 1e-4 so that an indexing slip cannot hide inside the loose bound.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN, golden_cases
from qvb8_b200 import packs, synth
from qvb8_b200.ext_qvb8 import ext
from util import bits16, ext_args, pack_np, random_pack, rel_fro

pytestmark = pytest.mark.gpu

TOL = 1e-2          # relative Frobenius tolerance of the small-M outputs (stated by the benchmark definition)
TIGHT = 1e-4        # what an fp32-accumulating implementation actually achieves, with margin
DEV = "cuda:0"


def _golden_pack(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    d = packs.read_qvb8(z["blob"].tobytes())
    return z, synth.QVB8Pack.from_parsed(d, DEV)


# ------------------------------------------------------------------------------------------------------------
# dense restore: bit-exact

@pytest.mark.parametrize("name", golden_cases())
def test_decode_matches_reference_golden(cuda_lib, name):
    z, pk = _golden_pack(name)
    args = ext_args(pk, "bf16")                     # the fixtures apply the pack's full escape list
    assert np.array_equal(bits16(ext.decode(*args)), z["w16_bits"])
    assert np.array_equal(bits16(ext.decode_bf16(*args)), z["wbf_bits"])
    w32 = ext.decode_f32(*args).cpu().numpy()
    assert np.array_equal(w32.view(np.uint32), z["w32"].view(np.uint32))


@pytest.mark.parametrize("Q,P,widths,esc", [
    (300, 1024, (6, 7), 0.001),
    (130, 512, (4, 5, 6, 7, 8), 0.01),
    (77, 256, tuple(range(1, 15)), 0.002),
    (16, 4096, (7,), 0.0),
    (5, 136, (3, 6, 9), 0.01),             # P % 8 == 0 but not % 128
    (9, 100, (5, 7, 11), 0.01),            # P % 8 != 0: rows start at arbitrary bits
    (1, 8, (14,), 0.0),
])
def test_decode_random_widths_vs_oracle(cuda_lib, Q, P, widths, esc):
    pk = random_pack(Q, P, widths, seed=Q * 7 + P, esc_frac=esc, device=DEV)
    d = pack_np(pk)
    for kind, fn in (("f16", ext.decode), ("bf16", ext.decode_bf16)):
        want = oracle.decode_16(d["ids"], d["nbits"], d["bit_off"], d["min_s"], d["tau_s"], Q, P, d["esc_idx"],
                                d["esc_vals"], kind)
        assert np.array_equal(bits16(fn(*ext_args(pk))), want), kind
    want32 = oracle.qvb8_dense(d)
    got32 = ext.decode_f32(*ext_args(pk)).cpu().numpy()
    assert np.array_equal(got32.view(np.uint32), want32.view(np.uint32))


def test_decode_empty(cuda_lib):
    pk = random_pack(0, 128, (7,), seed=1, device=DEV)
    assert ext.decode(*ext_args(pk)).shape == (0, 128)


# ------------------------------------------------------------------------------------------------------------
# small-M product

def _oracle_y(pk, X, narrow=True):
    W = oracle.qvb8_dense(pack_np(pk))
    return oracle.matmul_f32w(X.float().cpu().numpy(), W, narrow_x=narrow)


SHAPES = [
    # Q, P, widths, escape fraction
    (256, 1024, (6, 7), 0.001),
    (200, 512, (3, 4, 5, 6, 7, 8), 0.0),
    (130, 128, (7,), 0.01),                      # one chunk, ragged row block
    (17, 2048, (6, 7, 8), 0.0),                  # fewer rows than one tile pair
    (384, 640, tuple(range(1, 15)), 0.002),      # every width: fragment classes and the per-element class
    (1024, 4096, (7,), 0.0005),
]


@pytest.mark.parametrize("Q,P,widths,esc", SHAPES)
@pytest.mark.parametrize("M", [1, 2, 3, 8])
def test_small_m_vs_oracle(cuda_lib, Q, P, widths, esc, M):
    pk = random_pack(Q, P, widths, seed=Q + P + M, esc_frac=esc, device=DEV)
    X = synth.synth_activation(M, P, seed=7 + M, device=DEV)
    y = ext.forward(X, *ext_args(pk))
    assert y.shape == (M, Q) and y.dtype == torch.float32
    want = _oracle_y(pk, X)
    err = rel_fro(y.cpu().numpy(), want)
    assert err < TOL and err < TIGHT, err


@pytest.mark.parametrize("M", [9, 16, 17, 33, 48])
def test_verify_rows_vs_oracle(cuda_lib, M):
    pk = random_pack(272, 768, (5, 6, 7), seed=M, esc_frac=0.001, device=DEV)
    X = synth.synth_activation(M, 768, seed=M, device=DEV)
    perm = torch.argsort(pk.nbits.to(torch.int16), stable=True).to(torch.int32)
    tile_nb = torch.zeros((272 + 15) // 16, dtype=torch.int32, device=DEV)
    y = ext.mma_multi(X, *ext_args(pk), perm, tile_nb)
    err = rel_fro(y.cpu().numpy(), _oracle_y(pk, X))
    assert err < TOL and err < TIGHT, err


@pytest.mark.parametrize("xdt", [torch.float16, torch.bfloat16, torch.float32])
def test_activation_dtypes_and_saturation(cuda_lib, xdt):
    pk = random_pack(128, 256, (6, 7), seed=3, device=DEV)
    X = synth.synth_activation(4, 256, seed=2, device=DEV, dtype=torch.float32)
    if xdt != torch.float16:
        X[1, 5] = 7.0e4                          # beyond fp16: must clamp to 65504, not turn into inf
        X[2, 9] = -1.0e5
    X = X.to(xdt)
    y = ext.gemv_multi(X, *ext_args(pk))
    assert torch.isfinite(y).all()
    err = rel_fro(y.cpu().numpy(), _oracle_y(pk, X))
    assert err < TIGHT, err


def test_generic_path_agrees(cuda_lib):
    from qvb8_b200 import lib
    pk = random_pack(96, 200, (2, 6, 7, 12), seed=9, esc_frac=0.01, device=DEV)      # P % 128 != 0 -> generic kernel
    X = synth.synth_activation(5, 200, seed=1, device=DEV)
    y = ext.forward(X, *ext_args(pk))
    assert rel_fro(y.cpu().numpy(), _oracle_y(pk, X)) < TIGHT
    pk2 = random_pack(160, 384, (6, 7), seed=10, esc_frac=0.01, device=DEV)
    X2 = synth.synth_activation(3, 384, seed=1, device=DEV)
    st, keep = lib.pack_struct(pk2.ids, pk2.min_s, pk2.tau_s, pk2.nbits, pk2.bit_off, pk2.P, pk2.esc_idx, pk2.esc_vals)
    a = lib.small_m(st, keep, X2)
    b = lib.small_m(st, keep, X2, generic=True)
    assert rel_fro(a.cpu().numpy(), b.cpu().numpy()) < 1e-5


@pytest.mark.parametrize("fill,force_s,nstg,cps", [(100, 0, 0, 0), (25, 1, 2, 4), (300, 3, 3, 8), (50, 12, 8, 4), (100, 2, 2, 16),
                                                    (100, 0, 3, 12)])
@pytest.mark.parametrize("M", [1, 5, 16])
def test_plan_kernel_configurations(cuda_lib, fill, force_s, nstg, cps, M):
    """The streaming kernel under different grid sizes, K splits, ring depths and stage lengths, with escapes, gives the oracle's
    product; so does the layout-agnostic kernel (no plan)."""
    from qvb8_b200 import lib
    pk = random_pack(300, 1536, (4, 6, 7, 8, 11), seed=31 + M, esc_frac=0.004, device=DEV)
    X = synth.synth_activation(M, 1536, seed=M, device=DEV)
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
    plan = lib.build_plan(st, keep)
    want = _oracle_y(pk, X)
    try:
        lib.load().qvb8_small_m_set_tuning(fill, force_s, nstg, cps, 0)
        for flags in (0, lib.FLAG_PDL):
            y = lib.small_m(st, keep, X, plan=plan, flags=flags)
            err = rel_fro(y.cpu().numpy(), want)
            assert err < TIGHT, (err, flags)
    finally:
        lib.load().qvb8_small_m_set_tuning(0, 0, 0, 0, 0)
    y_noplan = lib.small_m(st, keep, X)
    assert rel_fro(y_noplan.cpu().numpy(), want) < TIGHT


def test_plan_contents(cuda_lib):
    """Tile descriptors: rows sorted by width (stable), 16 per tile, padding marked; escapes regrouped by row."""
    from qvb8_b200 import lib
    Q, P = 100, 256
    pk = random_pack(Q, P, (5, 7, 7, 7, 12), seed=5, device=DEV)
    idx = torch.tensor([3 * P + 7, 3 * P + 200, 40 * P + 1], dtype=torch.int64, device=DEV)
    val = torch.tensor([0.25, -0.5, 0.125], device=DEV)
    pk.esc_idx, pk.esc_vals = idx, val
    st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, idx, val)
    plan = lib.build_plan(st, keep).cpu()
    ntiles = int(plan[:4].view(torch.int32)[0])
    nbits = pk.nbits.cpu().numpy().astype(int)
    cls = np.where((nbits >= 3) & (nbits <= 8), nbits - 3, 6)
    want_tiles = sum((int((cls == c).sum()) + 15) // 16 for c in range(7))
    assert ntiles == want_tiles
    ptr = plan[256: 256 + (Q + 1) * 4].view(torch.int32).tolist()
    assert ptr[:4] == [0, 0, 0, 0] and ptr[4] == 2 and ptr[40] == 2 and ptr[41] == 3 and ptr[Q] == 3
    up = lambda v: (v + 255) // 256 * 256
    tiles_off = 256 + up((Q + 1) * 4) + 2 * up(3 * 4)
    seen = []
    for t in range(ntiles):
        d = plan[tiles_off + 400 * t: tiles_off + 400 * (t + 1)].view(torch.int32)
        nb, cnt = int(d[0]), int(d[1])
        rows = d[4:20].tolist()
        assert all(r >= 0 for r in rows[:cnt]) and all(r == -1 for r in rows[cnt:])
        assert rows[:cnt] == sorted(rows[:cnt])
        for r in rows[:cnt]:
            assert (nbits[r] if 3 <= nbits[r] <= 8 else 0) == nb
        seen += rows[:cnt]
    assert sorted(seen) == list(range(Q))
    X = synth.synth_activation(2, P, seed=1, device=DEV)
    y = lib.small_m(st, keep, X, plan=plan.to(DEV))
    assert rel_fro(y.cpu().numpy(), _oracle_y(pk, X)) < TIGHT


def test_fused_stack_equals_separate_launches(cuda_lib):
    """q/k/v and gate/up fused into one pack and one launch each give bit-identical outputs to one launch per
    projection (each row's sum is computed the same way), and the oracle's product."""
    from qvb8_b200 import stack
    cfg = stack.StackConfig("tiny", 1, 512, 512, 128, 1024, 1e-3, 9)
    for M in (1, 3):
        a = stack.LinearStack(cfg, M, DEV, fuse_same_input=True)
        b = stack.LinearStack(cfg, M, DEV, fuse_same_input=False)
        assert a.launches_per_step == 4 and b.launches_per_step == 7
        assert a.compressed_bytes == b.compressed_bytes
        a.step(); b.step()
        torch.cuda.synchronize()
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            assert torch.equal(a.y[0][name], b.y[0][name]), name
        for (lname, pk, _, _, xname, _), y in zip(b.launches[0], b.y_launch[0]):
            assert rel_fro(y.cpu().numpy(), _oracle_y(pk, b.x[xname])) < TIGHT, lname


def test_small_m_is_deterministic(cuda_lib):
    pk = random_pack(512, 4096, (6, 7), seed=21, esc_frac=0.001, device=DEV)        # several K-ranges
    X = synth.synth_activation(8, 4096, seed=3, device=DEV)
    a = ext.forward(X, *ext_args(pk))
    for _ in range(3):
        assert torch.equal(a, ext.forward(X, *ext_args(pk)))


def test_no_wait_ever_gave_up(cuda_lib):
    """Runs late in this file: the device-side error word must still be zero after every kernel above."""
    from qvb8_b200 import lib
    assert lib.device_status() == 0


def test_gemv_m1_entry_point(cuda_lib):
    pk = random_pack(256, 512, (7,), seed=4, device=DEV)
    x = synth.synth_activation(1, 512, seed=5, device=DEV, dtype=torch.float16).view(-1)
    y = ext.gemv(x, *ext_args(pk))
    assert y.shape == (1, 256)
    assert rel_fro(y.cpu().numpy(), _oracle_y(pk, x.view(1, -1))) < TIGHT
    with pytest.raises(RuntimeError):
        ext.gemv(x.float(), *ext_args(pk))           # the reference insists on fp16 here


def test_argument_errors_are_runtime_errors(cuda_lib):
    pk = random_pack(64, 256, (7,), seed=4, device=DEV)
    with pytest.raises(RuntimeError):
        ext.gemv_multi(synth.synth_activation(9, 256, device=DEV), *ext_args(pk))
    with pytest.raises(RuntimeError):
        ext.forward(synth.synth_activation(2, 128, device=DEV), *ext_args(pk))
    with pytest.raises(RuntimeError):
        ext.decode(pk.ids.cpu(), pk.min_s, pk.nbits, pk.bit_off, pk.P, pk.tau_s, pk.esc_idx, pk.esc_vals)
    with pytest.raises(RuntimeError):
        ext.mma_multi(synth.synth_activation(49, 256, device=DEV), *ext_args(pk), torch.empty(0), torch.empty(0))


def test_prefill_rows_route(cuda_lib):
    pk = random_pack(192, 512, (6, 7), seed=8, esc_frac=0.001, device=DEV)
    X = synth.synth_activation(80, 512, seed=2, device=DEV)
    y = ext.forward(X, *ext_args(pk))
    assert y.dtype == torch.float32 and y.shape == (80, 192)
    assert rel_fro(y.cpu().numpy(), _oracle_y(pk, X)) < TOL


# ------------------------------------------------------------------------------------------------------------
# the benchmark's single-layer configuration, through size-independent properties

def test_full_size_layer_properties(cuda_lib):
    Q = P = 4096
    pk, W = synth.synth_pack(Q, P, seed=1000, device=DEV, return_weight=True)
    w16 = ext.decode(*ext_args(pk))
    assert float((w16.double() - W.double()).abs().max()) <= pk.tau            # the certificate, every element
    w32 = ext.decode_f32(*ext_args(pk))
    assert torch.equal(w32, synth.reference_dense(pk, torch.float32))           # integer-op restatement on the GPU
    assert torch.equal(w16, synth.reference_dense(pk, torch.float16))
    assert torch.equal(ext.decode_bf16(*ext_args(pk, "bf16")), synth.reference_dense(pk, torch.bfloat16))
    x = synth.synth_activation(1, P, seed=7, device=DEV)
    y = ext.forward(x, *ext_args(pk))
    xs = x.float().clamp(-65504, 65504).half().double()
    want = xs @ w32.double().t()
    assert rel_fro(y.cpu().numpy(), want.cpu().numpy()) < TIGHT
    # linearity in X: f(a + b) == f(a) + f(b) up to rounding, on values exactly representable in fp16
    a = torch.randint(-8, 9, (1, P), device=DEV).to(torch.float16)
    b = torch.randint(-8, 9, (1, P), device=DEV).to(torch.float16)
    ya, yb, yab = (ext.forward(t, *ext_args(pk)) for t in (a, b, a + b))
    assert rel_fro(yab.cpu().numpy(), (ya + yb).cpu().numpy()) < 1e-5


# ------------------------------------------------------------------------------------------------------------
# activations that keep their range (the reference's bf16 mode of the verify kernel, qvb8_cuda.cu:1755-1775, 1861-1862;
# module.py:375-400 passes bf16=True with the bf16 escape table for bf16-certified packs)

@pytest.mark.parametrize("M", [8, 16, 48])
def test_bf16_mode_rows_vs_oracle(cuda_lib, M):
    pk = synth.synth_pack(272, 768, seed=60 + M, tau=2e-3, device=DEV, restore="fp16+bf16")
    X = synth.synth_activation(M, 768, seed=M, device=DEV, dtype=torch.bfloat16)
    perm = torch.argsort(pk.nbits.to(torch.int16), stable=True).to(torch.int32)
    tile_nb = torch.zeros((272 + 15) // 16, dtype=torch.int32, device=DEV)
    y = ext.mma_multi(X, *ext_args(pk, "bf16"), perm, tile_nb, True)
    d = pack_np(pk)
    band = oracle.restore_f32(oracle.unpack_ids(d["ids"], d["nbits"], d["bit_off"], pk.Q, pk.P), d["min_s"], d["tau_s"],
                              np.zeros(0, np.int64), np.zeros(0, np.float32))
    # the reference multiplies bf16(band) (escapes from the bf16 table); this library the un-narrowed band value
    Wb = torch.from_numpy(band).to(torch.bfloat16).float().numpy()
    Wb.reshape(-1)[d["esc_idx_bf16"]] = d["esc_vals_bf16"]
    Wf = band.copy()
    Wf.reshape(-1)[d["esc_idx_bf16"]] = d["esc_vals_bf16"]
    Xn = X.float().cpu().numpy()
    assert rel_fro(y.cpu().numpy(), oracle.matmul_f32w(Xn, Wb, narrow_x=False)) < TOL          # the reference's contract
    assert rel_fro(y.cpu().numpy(), oracle.matmul_f32w(Xn, Wf, narrow_x=False)) < TIGHT        # what is computed here


@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float32])
def test_bf16_mode_keeps_the_range(cuda_lib, xdt):
    """x_mode 1: a token with values far beyond fp16's range is prescaled by a power of two, not clamped; the other
    tokens are untouched; runs through the streaming kernel (P % 128 == 0, plan)"""
    pk = random_pack(160, 1024, (5, 6, 7, 8), seed=4, esc_frac=0.002, device=DEV)
    X = synth.synth_activation(9, 1024, seed=3, device=DEV, dtype=torch.float32)
    X[2] *= 3.0e6
    X[5, 17] = -2.5e8
    X[7] *= 1.0e-3
    X = X.to(xdt)
    perm = torch.argsort(pk.nbits.to(torch.int16), stable=True).to(torch.int32)
    tile_nb = torch.zeros(10, dtype=torch.int32, device=DEV)
    y = ext.mma_multi(X, *ext_args(pk), perm, tile_nb, True)
    assert torch.isfinite(y).all()
    W = oracle.qvb8_dense(pack_np(pk))
    want = oracle.matmul_f32w(X.float().cpu().numpy(), W, narrow_x=False)
    got = y.cpu().numpy()
    for m in range(9):                                   # row by row: a huge token must not hide the others
        # fp16 staging after the prescale keeps 11 bits of every activation: 5e-4 per element at worst
        assert rel_fro(got[m], want[m]) < 1e-3, (m, rel_fro(got[m], want[m]))
    # the clamping mode on the same input saturates token 2 and differs there, as documented
    y0 = ext.mma_multi(X, *ext_args(pk), perm, tile_nb, False)
    assert rel_fro(y0.cpu().numpy()[2], want[2]) > 0.1
    want0 = oracle.matmul_f32w(X.float().cpu().numpy()[:1], W, narrow_x=True)      # its own contract: fp16-narrowed activations
    assert rel_fro(y0.cpu().numpy()[0], want0[0]) < TIGHT


def test_config1_single_layer_against_the_oracle(cuda_lib):
    """the 4096 x 4096 single-layer configuration, product and restore against the CPU oracle itself"""
    Q = P = 4096
    pk = synth.synth_pack(Q, P, seed=1000, device=DEV)
    d = pack_np(pk)
    W = oracle.qvb8_dense(d)
    assert np.array_equal(ext.decode_f32(*ext_args(pk)).cpu().numpy().view(np.uint32), W.view(np.uint32))
    for M in (1, 8):
        X = synth.synth_activation(M, P, seed=7, device=DEV)
        y = ext.forward(X, *ext_args(pk))
        want = oracle.matmul_f32w(X.float().cpu().numpy(), W, narrow_x=True)
        assert rel_fro(y.cpu().numpy(), want) < TIGHT


# ------------------------------------------------------------------------------------------------------------
# several products behind one launch

def _job_items(shapes, M, seed, x_dtype=torch.bfloat16, widths=None, esc=0.001):
    from qvb8_b200 import lib
    items, packs_ = [], []
    for k, (Q, P) in enumerate(shapes):
        pk = random_pack(Q, P, widths or (6, 7), seed=seed + k, esc_frac=esc, device=DEV)
        st, keep = lib.pack_struct(pk.ids, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off, pk.P, pk.esc_idx, pk.esc_vals)
        X = synth.synth_activation(M, P, seed=seed + 10 * k, device=DEV, dtype=x_dtype)
        Y = torch.full((M, Q), float("nan"), device=DEV)
        items.append((st, keep, lib.build_plan(st, keep), X, Y))
        packs_.append(pk)
    return items, packs_


@pytest.mark.parametrize("M", [1, 2, 4, 8])
@pytest.mark.parametrize("shapes", [
    [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)],              # one 9B-class layer
    [(256, 512), (48, 1024), (16, 128), (1024, 256), (300, 384), (7, 2048), (512, 512)],     # small and ragged
    [(512, 1024)] * 131,                                                     # more jobs than one launch takes
])
def test_job_list_equals_separate_calls(cuda_lib, shapes, M):
    from qvb8_b200 import lib
    items, packs_ = _job_items(shapes, M, seed=100 * M)
    jl = lib.JobList(items)
    lib.small_m_group(jl)
    torch.cuda.synchronize()
    for (st, keep, plan, X, Y), pk in zip(items, packs_):
        want = lib.small_m(st, keep, X, plan=plan)
        # the same kernel on the same bytes; only the grouping of the fixed-order fp32 partial sums differs (a list cuts
        # its stream of tiles into per-CTA ranges of its own, and adds the escape corrections in a pre-pass)
        assert rel_fro(Y.cpu().numpy(), want.cpu().numpy()) < 1e-5
    # and against the oracle for the first and the last job
    for k in (0, len(items) - 1):
        assert rel_fro(items[k][4].cpu().numpy(), _oracle_y(packs_[k], items[k][3])) < TIGHT
    # a second run over the same list (barrier phases, exchange buffers start afresh) gives the same bits
    first = [it[4].clone() for it in items]
    lib.small_m_group(jl, flags=lib.FLAG_PDL)
    torch.cuda.synchronize()
    assert all(torch.equal(a, it[4]) for a, it in zip(first, items))
    assert lib.device_status(DEV) == 0


def test_job_list_escapes_by_pre_pass_and_in_line(cuda_lib):
    """a list's escapes are applied by the pre-pass kernel; the tuning alternative sums them on the consumer warps, tile
    by tile (here with more entries per tile than travel with a descriptor: the rest comes from global memory) -- the
    same results"""
    from qvb8_b200 import lib
    L = lib.load()
    for M in (1, 3, 4, 8):
        items, packs_ = _job_items([(256, 4096), (200, 1024), (48, 12288), (512, 512)], M, seed=40 + M, esc=0.02)
        jl = lib.JobList(items)
        lib.small_m_group(jl)
        torch.cuda.synchronize()
        first = [it[4].clone() for it in items]
        for y, (st, keep, plan, X, Y), pk in zip(first, items, packs_):
            assert rel_fro(y.cpu().numpy(), _oracle_y(pk, X)) < TIGHT
        try:
            L.qvb8_small_m_set_tuning(0, 0, 0, 0, 32)                      # in line (8 tokens: still the pre-pass)
            lib.small_m_group(jl)
            torch.cuda.synchronize()
            second = [it[4].clone() for it in items]
            lib.small_m_group(jl, flags=lib.FLAG_PDL)
            torch.cuda.synchronize()
            assert all(torch.equal(a, it[4]) for a, it in zip(second, items))     # one sum order
        finally:
            L.qvb8_small_m_set_tuning(0, 0, 0, 0, 0)
        for y, pk, it in zip(first, packs_, items):
            assert rel_fro(it[4].cpu().numpy(), y.cpu().numpy()) < 1e-5
            assert rel_fro(it[4].cpu().numpy(), _oracle_y(pk, it[3])) < TIGHT
    assert lib.device_status(DEV) == 0


def test_job_list_mixed_widths_and_range_mode(cuda_lib):
    from qvb8_b200 import lib
    shapes = [(320, 1024), (160, 512), (640, 1024), (96, 2048), (320, 1024)]
    items, packs_ = _job_items(shapes, 9, seed=7, x_dtype=torch.float32, widths=(3, 4, 5, 6, 7, 8, 11), esc=0.003)
    items[2][3].mul_(1.0e6)                                                # beyond fp16: needs the prescale of x_mode 1
    jl = lib.JobList(items, x_mode=1)
    lib.small_m_group(jl)
    torch.cuda.synchronize()
    for (st, keep, plan, X, Y), pk in zip(items, packs_):
        assert rel_fro(Y.cpu().numpy(), lib.small_m(st, keep, X, x_mode=1, plan=plan).cpu().numpy()) < 1e-5
        W = oracle.qvb8_dense(pack_np(pk))
        assert rel_fro(Y.cpu().numpy(), oracle.matmul_f32w(X.cpu().numpy(), W, narrow_x=False)) < 1e-3
    assert lib.device_status(DEV) == 0


@pytest.mark.parametrize("M,shapes", [
    (16, [(512, 12288), (1024, 4096)]),                    # 16 tokens: six and two column ranges
    (8, [(640, 8192), (96, 28672), (2048, 512)]),          # two ranges, seven ranges, whole
    (24, [(320, 4096), (160, 2048)]),
    (3, [(200, 28672), (64, 128)]),
])
def test_job_list_with_column_ranges(cuda_lib, M, shapes):
    """activations that would crowd the copy rings out of shared memory are staged a column range at a time: the pack
    runs as consecutive jobs of the list, one per range, and every thread adds the later ranges to what it wrote for
    the first"""
    from qvb8_b200 import lib
    items, packs_ = _job_items(shapes, M, seed=3 + M, esc=0.002)
    jl = lib.JobList(items)
    L = lib.load()
    refs = [lib.small_m(st, keep, X, plan=plan) for st, keep, plan, X, Y in items]      # every job on its own
    torch.cuda.synchronize()
    for budget_kb in (0, 20):                                              # the default budget, and a small one: more ranges
        try:
            L.qvb8_small_m_set_tuning(0, budget_kb, 0, 0, 0)
            jl = lib.JobList(items)                                        # (a list sizes its scratch when it is made)
            lib.small_m_group(jl)
            torch.cuda.synchronize()
            first = [it[4].clone() for it in items]
            lib.small_m_group(jl, flags=lib.FLAG_PDL)
            torch.cuda.synchronize()
        finally:
            L.qvb8_small_m_set_tuning(0, 0, 0, 0, 0)
        assert all(torch.equal(a, it[4]) for a, it in zip(first, items))   # one sum order, run after run
        for (st, keep, plan, X, Y), pk, ref in zip(items, packs_, refs):
            assert rel_fro(Y.cpu().numpy(), ref.cpu().numpy()) < 1e-5
            assert rel_fro(Y.cpu().numpy(), _oracle_y(pk, X)) < TIGHT
    # with the cut switched off the large jobs run on their own (K split across CTAs): the same results
    try:
        L.qvb8_small_m_set_tuning(0, 0, 0, 0, 128)
        jl = lib.JobList(items)
        lib.small_m_group(jl)
        torch.cuda.synchronize()
    finally:
        L.qvb8_small_m_set_tuning(0, 0, 0, 0, 0)
    for (st, keep, plan, X, Y), ref in zip(items, refs):
        assert rel_fro(Y.cpu().numpy(), ref.cpu().numpy()) < 1e-5
    assert lib.device_status(DEV) == 0
