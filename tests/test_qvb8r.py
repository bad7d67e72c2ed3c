"""QVB8R (entropy-coded QVB8): the synthetic encoder against the oracle decoder, the container round trip, and the
CUDA kernels against the oracle on seeded packs.  The oracle decoder, the encoder, the container code and the kernels
are pinned on files written and decoded by the reference itself in tests/test_qvb8r_golden.py."""
import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import packs, rans, synth

DEV = "cuda:0"
TOL = 1e-2
TIGHT = 2e-5


def _pack(Q, P, seed, K=3, T=None, tau=2e-3):
    W = synth.synth_weight(Q, P, seed)
    return W, synth.encode_qvb8r(W, tau=tau, K=K, T=T)


def _dense(d):
    """fp32 restored weights with the exact escapes written over (what a dense reader produces)."""
    return oracle.qvb8r_dense(d)


def test_encoder_roundtrip_and_certificate():
    W, d = _pack(80, 256, seed=11, K=3, T=4)
    tab = rans.slot_tables(d["freq"])
    assert np.array_equal(tab, oracle.slot_tables(d["freq"]))
    assert int(d["freq"].astype(np.int64).sum(1).min()) == 4096 and int(d["freq"].max()) <= 1024
    words = np.concatenate([d["words"], np.zeros(rans.PAD_WORDS, np.uint32)])
    ids = oracle.rans_decode_ids(words, d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64), tab,
                                 d["perm"], d["drow"].astype(np.int32), 80, 256)
    band = oracle.rans_restore_f32(ids, d["min_s"], d["tau_s"])
    Wd = _dense(d)
    # every weight within tau of the source after the fp16 rounding the certificate is stated on
    err = np.abs(Wd.astype(np.float16).astype(np.float64) - W.float().numpy().astype(np.float64))
    assert float(err.max()) <= 2e-3
    # the stored differences are exact - band at the escaped positions
    ei = d["esc_idx"]
    assert np.array_equal((d["esc_val"] - band.reshape(-1)[ei]).astype(np.float32), d["esc_delta"])
    assert d["words"].size * 32 / (80 * 256) < 8.0       # it does compress


def test_container_roundtrip():
    _, d = _pack(48, 128, seed=5, K=2, T=8)
    blob = packs.write_qvb8r(d, Q=d["Q"], P=d["P"], min_s=d["min_s"], tau_s=d["tau_s"], esc_idx=d["esc_idx"],
                             esc_val=d["esc_val"], esc_delta=d["esc_delta"], cert=dict(tau=d["tau"], max_err=d["max_err"]))
    r = packs.read_qvb8r(blob)
    for k in ("perm", "freq", "tiles", "tile_off", "states", "words", "drow", "min_s", "tau_s", "esc_idx", "esc_val", "esc_delta"):
        assert np.array_equal(np.asarray(r[k]), np.asarray(d[k]).astype(np.asarray(r[k]).dtype)), k
    assert np.array_equal(_dense(r).view(np.uint32), _dense(d).view(np.uint32))
    bad = bytearray(blob); bad[200] ^= 1
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8r(bytes(bad))


def test_blocks_schedule():
    tiles = np.array([[0, 0, 4]] * 10 + [[1, 40, 4]] * 3, np.int64)
    b = rans.blocks_for(tiles, 8)
    assert b.tolist() == [[0, 0, 8], [0, 8, 2], [1, 10, 3]]


@pytest.mark.gpu
@pytest.mark.parametrize("Q,P,K,T", [(80, 256, 3, 4), (300, 1024, 2, 1), (64, 4096, 1, 8), (1000, 512, 4, 3)])
def test_gpu_ids_and_decode(cuda_lib, Q, P, K, T):
    from qvb8_b200.ext_qvb8r import core_tensors, ext
    _, d = _pack(Q, P, seed=Q + P, K=K, T=T)
    core = core_tensors(d, DEV)
    tab = rans.slot_tables(d["freq"])
    words = np.concatenate([d["words"], np.zeros(rans.PAD_WORDS, np.uint32)])
    want_ids = oracle.rans_decode_ids(words, d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64), tab,
                                      d["perm"], d["drow"].astype(np.int32), Q, P)
    got = ext.ids(P, *core)
    assert np.array_equal(got.cpu().numpy(), want_ids)                       # bit-exact
    band = oracle.rans_restore_f32(want_ids, d["min_s"], d["tau_s"])
    nblk = core[4].numel() // 3
    for code, dt, ref in ((2, torch.float32, band),
                          (0, torch.float16, torch.from_numpy(band).to(torch.float16).numpy()),
                          (1, torch.bfloat16, None)):
        Wg = ext.decode(*core, P, code, 0, nblk, -1, 0)
        assert Wg.dtype == dt
        if ref is None:
            assert torch.equal(Wg.cpu(), torch.from_numpy(band).to(torch.bfloat16))
        else:
            assert np.array_equal(Wg.cpu().numpy().view(np.uint16 if code == 0 else np.uint32),
                                  ref.view(np.uint16 if code == 0 else np.uint32))
    # a block range as a compact chunk in sorted order
    b0, nb = nblk // 3, max(1, nblk // 2)
    blocks = core[4].cpu().numpy().reshape(-1, 3)
    tiles = np.asarray(d["tiles"]).reshape(-1, 3)
    t_first, t_last = blocks[b0][1], blocks[b0 + nb - 1][1] + blocks[b0 + nb - 1][2] - 1
    row_base = int(tiles[t_first][1]); nrows = int(tiles[t_last][1] + tiles[t_last][2]) - row_base
    chunk = ext.decode(*core, P, 2, b0, nb, row_base, nrows)
    want_chunk = band[np.asarray(d["perm"])[row_base:row_base + nrows]]
    assert np.array_equal(chunk.cpu().numpy().view(np.uint32), want_chunk.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 3, 8, 13])
def test_gpu_products(cuda_lib, M):
    from qvb8_b200.ext_qvb8r import core_tensors, escape_csr, ext
    Q, P = 260, 1024
    _, d = _pack(Q, P, seed=70 + M, K=3, T=2)
    core = core_tensors(d, DEV)
    Wd = _dense(d)                                                           # exact escapes written over
    X = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.float32)
    want = oracle.matmul_f32w(X.cpu().numpy(), Wd, narrow_x=False)
    if M == 1:
        y = ext.gemv(X.reshape(-1), *core).reshape(1, -1)
    elif M <= 8:
        y = ext.multi(X, *core)
        yb = ext.multi(X.to(torch.bfloat16), *core)                           # bf16 X is exact in fp32
        ext.fix_escapes(X.to(torch.bfloat16).float(), *escape_csr(d, DEV), yb)
        wb = oracle.matmul_f32w(X.to(torch.bfloat16).float().cpu().numpy(), Wd, narrow_x=False)
        assert np.linalg.norm(yb.cpu().numpy() - wb) / np.linalg.norm(wb) < TIGHT
    else:
        y = None
    if y is not None:
        ext.fix_escapes(X, *escape_csr(d, DEV), y)
        err = np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want)
        assert err < TOL and err < TIGHT, err
    # tensor-core contract: band rounded once to fp16, fp16 X
    Xh = X.to(torch.float16)
    yt = ext.tc(Xh, *core, 8)
    ids = oracle.rans_decode_ids(np.concatenate([d["words"], np.zeros(rans.PAD_WORDS, np.uint32)]),
                                 d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64),
                                 rans.slot_tables(d["freq"]), d["perm"], d["drow"].astype(np.int32), Q, P)
    W16 = oracle.rans_restore_f32(ids, d["min_s"], d["tau_s"]).astype(np.float16).astype(np.float32)
    wt = oracle.matmul_f32w(Xh.float().cpu().numpy(), W16, narrow_x=False)
    errt = np.linalg.norm(yt.cpu().numpy() - wt) / np.linalg.norm(wt)
    assert errt < TOL and errt < TIGHT, errt
    assert torch.equal(yt, ext.tc(Xh, *core, 8))                              # fixed summation order


def test_linear_module_builds_on_cpu_and_chunks_cover_all_rows():
    """Host-side logic of the module: buffers, escape CSR, chunk plan (no kernel call)."""
    from qvb8_b200.linear_r import QVBandLinearV8R, plan_chunks
    _, d = _pack(100, 256, seed=21, K=3, T=4)
    mod = QVBandLinearV8R(d, device="cpu")
    assert mod.whole and len(mod.chunks) == 1 and mod.chunks[0].rows == 100
    assert sorted(mod.chunk_rows.tolist()) == list(range(100))
    assert int(mod.esc_ptr[-1]) == len(d["esc_idx"]) == mod.esc_delta16.numel()
    small = type("Small", (QVBandLinearV8R,), {"CHUNK_BYTES": 2 * 256 * 16})     # 16 rows of fp16 per chunk
    m2 = small(d, device="cpu")
    assert len(m2.chunks) > 1 and not m2.whole
    assert sum(c.rows for c in m2.chunks) == 100 and m2.chunks[-1].esc1 == m2.chunk_esc_pos.numel() == len(d["esc_idx"])
    assert all(a.row0 + a.rows == b.row0 and a.block0 + a.nblocks == b.block0 for a, b in zip(m2.chunks, m2.chunks[1:]))
    # every chunk escape lands on the element it names: sorted row (row0 + pos // P) is original row chunk_rows[...]
    P = 256
    got = set()
    for c in m2.chunks:
        for pos in m2.chunk_esc_pos[c.esc0:c.esc1].tolist():
            assert 0 <= pos < c.rows * P
            got.add(int(m2.chunk_rows[c.row0 + pos // P]) * P + pos % P)
    assert got == set(int(v) for v in d["esc_idx"])
    tiles = np.array([[0, 0, 4], [0, 4, 4], [0, 8, 4], [1, 12, 2], [1, 14, 2]], np.int64)
    blocks = rans.blocks_for(tiles, 2)
    assert plan_chunks(tiles, blocks, 8) == [(0, 1, 0, 8), (1, 2, 8, 8)]
    assert plan_chunks(tiles, blocks, 1) == [(0, 1, 0, 8), (1, 1, 8, 4), (2, 1, 12, 4)]
    mod.to(torch.bfloat16)
    assert mod.min_s.dtype == torch.float32 and mod.esc_delta.dtype == torch.float32


@pytest.mark.gpu
@pytest.mark.parametrize("M,chunk_rows", [(1, None), (5, None), (12, None), (40, None), (130, None), (130, 32)])
def test_linear_module_forward(cuda_lib, M, chunk_rows):
    from qvb8_b200.linear_r import QVBandLinearV8R
    Q, P = 260, 1024
    _, d = _pack(Q, P, seed=31, K=3, T=2)
    cls = QVBandLinearV8R if chunk_rows is None else type("Small", (QVBandLinearV8R,), {"CHUNK_BYTES": 2 * P * chunk_rows})
    bias = torch.linspace(-1, 1, Q)
    mod = cls(d, bias=bias, device=DEV)
    X = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.bfloat16)
    y = mod(X.reshape(1, M, P))
    assert y.shape == (1, M, Q) and y.dtype == torch.bfloat16
    want = oracle.matmul_f32w(X.float().cpu().numpy(), _dense(d), narrow_x=False) + bias.numpy()[None, :]
    err = np.linalg.norm(y.float().cpu().numpy().reshape(M, Q) - want) / np.linalg.norm(want)
    assert err < TOL, err                                 # bf16 output rounding: ~2e-3
    yf = mod(X.float())
    errf = np.linalg.norm(yf.cpu().numpy() - want) / np.linalg.norm(want)
    assert errf < 1e-3, errf                             # fp16 weight rounding above 8 rows
    Wd = mod.dense(torch.float32)
    assert np.array_equal(Wd.cpu().numpy().view(np.uint32), _dense(d).view(np.uint32))


def test_same_input_fusion_is_the_members_side_by_side():
    """concat_qvb8r: the fused dict restores to the members' weights stacked, bit for bit (oracle decoder, CPU)."""
    from qvb8_b200 import fuse
    _, a = _pack(48, 256, seed=41, K=2, T=4)
    _, b = _pack(80, 256, seed=42, K=3, T=2)
    _, c = _pack(16, 256, seed=43, K=2, T=8)
    fused, splits = fuse.concat_qvb8r([a, b, c])
    assert splits == [48, 128] and fused["Q"] == 144 and fused["K"] == 7
    want = np.vstack([_dense(a), _dense(b), _dense(c)])
    assert np.array_equal(_dense(fused).view(np.uint32), want.view(np.uint32))
    blob = packs.write_qvb8r(fused, Q=fused["Q"], P=fused["P"], min_s=fused["min_s"], tau_s=fused["tau_s"],
                             esc_idx=fused["esc_idx"], esc_val=fused["esc_val"], esc_delta=fused["esc_delta"],
                             cert=dict(tau=fused["tau"], max_err=fused["max_err"]))
    assert np.array_equal(_dense(packs.read_qvb8r(blob)).view(np.uint32), want.view(np.uint32))


def test_tile_shards_are_the_rows_of_the_whole():
    """runs of whole tiles as tensors of their own (no re-encoding): restored, they are the whole tensor's rows; the
    escapes go with their rows; the bounds balance the coded words"""
    from qvb8_b200 import fuse
    _, d = _pack(200, 256, seed=61, K=3, T=4)
    whole = _dense(d)
    for world in (1, 2, 3, 8, 64):
        bounds = fuse.qvb8r_shard_bounds(d, world)
        assert bounds[0] == 0 and bounds[-1] == len(d["tiles"]) and all(a <= b for a, b in zip(bounds, bounds[1:]))
        got, seen, n_esc = np.zeros_like(whole), np.zeros(200, int), 0
        for r in range(world):
            sh, rows = fuse.qvb8r_tile_shard(d, bounds[r], bounds[r + 1])
            assert sh["Q"] == len(rows) and sh["words"].size == int(d["tile_off"][bounds[r + 1]] - d["tile_off"][bounds[r]])
            if sh["Q"]:
                got[rows] = _dense(sh)
            seen[rows] += 1
            n_esc += len(sh["esc_idx"])
            assert np.all(np.diff(sh["esc_idx"]) > 0)
        assert np.array_equal(got.view(np.uint32), whole.view(np.uint32)) and seen.min() == seen.max() == 1
        assert n_esc == len(d["esc_idx"])
        if world in (2, 3):
            sizes = [int(d["tile_off"][b] - d["tile_off"][a]) for a, b in zip(bounds, bounds[1:])]
            assert max(sizes) - min(sizes) <= 2 * int(np.diff(d["tile_off"]).max())
    with pytest.raises(ValueError):
        fuse.qvb8r_tile_shard(d, 3, len(d["tiles"]) + 1)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 9, 40])
def test_tile_sharded_modules_cover_the_whole_product(cuda_lib, M):
    """three shard modules on one device, each with its run of tiles: their local rows, put in place, are the whole
    module's output"""
    from qvb8_b200.linear_r import QVBandLinearV8R, QVBandLinearV8RShard
    P = 512
    _, d = _pack(330, P, seed=71, K=3, T=4)
    X = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.bfloat16)
    want = QVBandLinearV8R(d, device=DEV)(X).float()
    got = torch.full_like(want, float("nan"))
    for r in range(3):
        sh = QVBandLinearV8RShard(d, r, 3, device=DEV)
        got[:, sh.rows] = sh(X).float()
    assert torch.equal(got, want)
    one = QVBandLinearV8RShard(d, 0, 1, device=DEV)
    assert torch.equal(one(X).float(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 6, 14, 70])
def test_same_input_fusion_module(cuda_lib, M):
    """One module over the fused dict gives the members' module outputs side by side."""
    from qvb8_b200 import fuse
    from qvb8_b200.linear_r import QVBandLinearV8R
    P = 512
    ds = [_pack(Q, P, seed=50 + i, K=2, T=2)[1] for i, Q in enumerate((64, 32, 96))]
    fused, splits = fuse.concat_qvb8r(ds)
    X = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.bfloat16)
    y = QVBandLinearV8R(fused, device=DEV)(X).float()
    parts = [QVBandLinearV8R(d, device=DEV)(X).float() for d in ds]
    got = torch.tensor_split(y, splits, dim=-1)
    for g, w in zip(got, parts):
        if M <= 16:
            assert torch.equal(g, w)                     # the same kernels on the same bytes
        else:
            assert torch.allclose(g, w, rtol=2e-2, atol=2e-2)        # library GEMM: the tile shape may differ
