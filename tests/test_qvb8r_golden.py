"""QVB8R against files the REFERENCE wrote and decoded (tests/golden/qvb8r_*.npz, made by make_golden_qvb8r.py with
the reference's container.write / read / runtime_tables / blocks_for, codec.slot_tables and the C++ encode /
embed_rows).  CPU part: this package's reader, writer, tables, encoder and the oracle decoder reproduce them bit for
bit.  GPU part (-m gpu): the kernels do."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN, golden_qvb8r_cases
from qvb8_b200 import packs, rans

CASES = golden_qvb8r_cases()


def _load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return z, packs.read_qvb8r(z["blob"].tobytes(), name)


def test_fixtures_exist():
    assert len(CASES) >= 3


@pytest.mark.parametrize("name", CASES)
def test_oracle_decodes_the_reference_file(name):
    z, d = _load(name)
    tab = oracle.slot_tables(d["freq"])
    assert np.array_equal(tab, z["tab"])
    words = np.concatenate([d["words"], np.zeros(rans.PAD_WORDS, np.uint32)])
    zero = np.zeros(d["Q"], np.int32)
    sym = oracle.rans_decode_ids(words, d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64), tab,
                                 d["perm"], zero, d["Q"], d["P"])
    assert np.array_equal(sym, z["sym"])
    ids = oracle.rans_decode_ids(words, d["tile_off"].astype(np.int64), d["states"], d["tiles"].astype(np.int64), tab,
                                 d["perm"], d["drow"].astype(np.int32), d["Q"], d["P"])
    assert np.array_equal(ids, z["ids"])


@pytest.mark.parametrize("name", CASES)
def test_runtime_tables_match_the_reference(name):
    z, d = _load(name)
    assert np.array_equal(rans.slot_tables(d["freq"]), z["tab"])
    assert np.array_equal(rans.blocks_for(d["tiles"], 8), z["blocks8"])
    assert np.array_equal(rans.blocks_for(d["tiles"], 16), z["blocks16"])


@pytest.mark.parametrize("name", CASES)
def test_encoder_reproduces_the_reference_stream(name):
    """the numpy encoder of this package against the reference's C++ encode: same states, words and tile offsets"""
    z, d = _load(name)
    sym_sorted = z["sym"].astype(np.int64)[d["perm"]]
    states, words, tile_off = rans.encode_symbols(sym_sorted, d["tiles"][:, 0], d["tiles"][:, 2], d["freq"])
    assert np.array_equal(states, d["states"])
    assert np.array_equal(words, d["words"])
    assert np.array_equal(tile_off, d["tile_off"])


@pytest.mark.parametrize("name", CASES)
def test_writer_reproduces_the_reference_file(name):
    z, d = _load(name)
    cert = json.loads(z["cert_json"].tobytes())
    blob = packs.write_qvb8r(d, Q=d["Q"], P=d["P"], min_s=d["min_s"], tau_s=d["tau_s"], esc_idx=d["esc_idx"],
                             esc_val=d["esc_val"], esc_delta=d["esc_delta"], cert=cert)
    assert blob == z["blob"].tobytes()


@pytest.mark.parametrize("name", CASES)
def test_embedding_values_and_stored_differences(name):
    """the reference's embedding restore is a multiplication then an addition (qvb8r_cpu.cpp:44); the stored escape
    difference is taken against the fused form the kernels use (qvb8r_cuda.cu:10)"""
    z, d = _load(name)
    ids = z["ids"].astype(np.float32)
    emb = ids * d["tau_s"][:, None] + d["min_s"][:, None]
    emb.reshape(-1)[d["esc_idx"]] = d["esc_val"]
    assert np.array_equal(emb.view(np.uint32), z["embed_f32"].view(np.uint32))
    band = oracle.rans_restore_f32(z["ids"], d["min_s"], d["tau_s"])
    assert np.array_equal((d["esc_val"] - band.reshape(-1)[d["esc_idx"]]).astype(np.float32), d["esc_delta"])


def test_reader_rejects_damage():
    z, _ = _load(CASES[0])
    blob = bytearray(z["blob"].tobytes())
    for pos in (0, 5, 300, len(blob) - 2):
        bad = bytearray(blob)
        bad[pos] ^= 0x40
        with pytest.raises(packs.PackFormatError):
            packs.read_qvb8r(bytes(bad))
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8r(bytes(blob[:len(blob) // 2]))


# ---------------------------------------------------------------------------------------------------------------
# GPU

def _core(d, dev):
    from qvb8_b200.ext_qvb8r import core_tensors
    return core_tensors(d, dev)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_gpu_ids_and_dense_restore(name, cuda_lib):
    from qvb8_b200.ext_qvb8r import ext
    z, d = _load(name)
    core = _core(d, "cuda:0")
    ids = ext.ids(d["P"], *core).cpu().numpy()
    assert np.array_equal(ids, z["ids"])
    band = oracle.rans_restore_f32(z["ids"], d["min_s"], d["tau_s"])
    nb = core[4].numel() // 3
    w32 = ext.decode(*core, d["P"], 2, 0, nb, -1, 0).cpu().numpy()
    assert np.array_equal(w32.view(np.uint32), band.view(np.uint32))
    w16 = ext.decode(*core, d["P"], 0, 0, nb, -1, 0).cpu().numpy()
    assert np.array_equal(w16.view(np.uint16), band.astype(np.float16).view(np.uint16))
    wbf = ext.decode(*core, d["P"], 1, 0, nb, -1, 0)
    want = torch.from_numpy(band).to(torch.bfloat16)
    assert torch.equal(wbf.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("M", [1, 3, 8, 16])
def test_gpu_products(name, M, cuda_lib):
    from qvb8_b200.ext_qvb8r import escape_csr, ext
    z, d = _load(name)
    dev = "cuda:0"
    core = _core(d, dev)
    g = torch.Generator().manual_seed(100 + M)
    X = torch.randn(M, d["P"], generator=g)
    band = oracle.rans_restore_f32(z["ids"], d["min_s"], d["tau_s"]).astype(np.float64)
    W = band.copy()
    W.reshape(-1)[d["esc_idx"]] = d["esc_val"]
    want = X.double().numpy() @ W.T
    uq, ptr, ec, ed = escape_csr(d, dev)
    Xd = X.to(dev)
    if M == 1:
        y = ext.gemv(Xd.view(-1).contiguous(), *core).view(1, -1)
    elif M <= 8:
        y = ext.multi(Xd, *core)
    else:
        y = None
    if y is not None:
        y = y.contiguous()
        ext.fix_escapes(Xd, uq, ptr, ec, ed, y)
        err = np.linalg.norm(y.cpu().numpy() - want) / np.linalg.norm(want)
        assert err < 2e-5, err
    # the fp16-rounded-weight path for every M <= 16
    W16 = band.astype(np.float32).astype(np.float16).astype(np.float64)
    W16.reshape(-1)[d["esc_idx"]] = d["esc_val"]
    Xh = X.half()
    want16 = Xh.double().numpy() @ W16.T
    y16 = ext.tc(Xh.to(dev).contiguous(), *core, int(d["T"])).contiguous()
    band16 = band.astype(np.float32).astype(np.float16).astype(np.float32).reshape(-1)[d["esc_idx"]]
    ed16 = torch.from_numpy((d["esc_val"] - band16).astype(np.float32)).to(dev)
    ext.fix_escapes(Xh.float().to(dev).contiguous(), uq, ptr, ec, ed16, y16)
    err = np.linalg.norm(y16.cpu().numpy() - want16) / np.linalg.norm(want16)
    assert err < 2e-5, err


@pytest.mark.parametrize("name", CASES)
def test_shim_encode_and_row_hist_match_the_reference_stream(name):
    """the host-side entry points of the reference extension, as the shim offers them (qvb8r_cuda.cu:453-455)"""
    from qvb8_b200.ext_qvb8r import ext
    z, d = _load(name)
    sym_sorted = torch.from_numpy(np.ascontiguousarray(z["sym"][d["perm"]]))
    F = torch.from_numpy(d["freq"].astype(np.int64))
    C = torch.cumsum(F, 1) - F
    if sym_sorted.shape[1] % 128 == 0:
        words, off, states = ext.encode(sym_sorted, torch.from_numpy(d["tiles"].astype(np.int64)), F, C)
        assert np.array_equal(words.numpy().view(np.uint32), d["words"])
        assert np.array_equal(off.numpy(), d["tile_off"].astype(np.int64))
        assert np.array_equal(states.numpy().view(np.uint64), d["states"])
    H = ext.row_hist(sym_sorted, int(d["N"])).numpy()
    want = np.stack([np.bincount(r, minlength=int(d["N"])) for r in sym_sorted.numpy().astype(np.int64)])
    assert np.array_equal(H, want)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_gpu_embedding_rows_match_the_reference_reader(name, cuda_lib):
    """rows decoded on the device against the reference's CPU embed_rows output, bit for bit"""
    from qvb8_b200.embedding import QVBandEmbeddingV8R
    from qvb8_b200.ext_qvb8r import EmbeddingTable
    z, d = _load(name)
    table = EmbeddingTable.from_parsed(d, "cuda:0")
    Q = d["Q"]
    rows = torch.tensor([Q - 1, 0, Q // 2, 0, 1] + list(range(Q)), device="cuda:0")
    got = table.lookup(rows).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), z["embed_f32"][rows.cpu().numpy()].view(np.uint32))
    emb = QVBandEmbeddingV8R(d, out_dtype=torch.float32, device="cuda:0")
    idx = torch.tensor([[1, 2], [Q - 1, 0]])
    assert np.array_equal(emb(idx).cpu().numpy().view(np.uint32), z["embed_f32"][idx.numpy()].view(np.uint32))
    with pytest.raises(IndexError):
        emb(torch.tensor([Q]))
