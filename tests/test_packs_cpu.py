"""Host-side pack logic: byte layouts, readers/writers, the seeded encoder (no GPU)."""
import os

import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import packs, synth
from util import pack_np, random_pack


def test_pack_ids_roundtrip_all_widths():
    pk = random_pack(40, 104, tuple(range(1, 15)), seed=3)
    d = pack_np(pk)
    ids = oracle.unpack_ids(d["ids"], d["nbits"], d["bit_off"], 40, 104)
    again = packs.pack_ids(ids, d["nbits"])
    assert np.array_equal(again, d["ids"])
    assert len(d["ids"]) == packs.payload_bytes(d["nbits"], 104) + packs.PAYLOAD_PAD


def test_torch_packer_equals_host_packer():
    rng = np.random.default_rng(0)
    nbits = rng.integers(1, 15, 64)
    ids = rng.integers(0, 1 << 30, (64, 256)) & ((1 << nbits)[:, None] - 1)
    host = packs.pack_ids(ids, nbits)
    dev, off = synth.pack_payload(torch.from_numpy(ids), torch.from_numpy(nbits))
    assert np.array_equal(dev.numpy(), host)
    assert np.array_equal(off.numpy(), packs.row_bit_offsets(nbits, 256))


@pytest.mark.parametrize("container", ["QVBD", "QVB8"])
def test_blob_roundtrip(container):
    pk = synth.synth_pack(24, 256, seed=5)
    d = packs.read_qvb8(pk.to_blob(container))
    assert (d["Q"], d["P"]) == (24, 256)
    for k in ("min_s", "tau_s", "nbits", "bit_off", "ids", "esc_idx", "esc_vals"):
        assert np.array_equal(d[k], getattr(pk, k).numpy()), k
    assert packs.read_qvb8_shape(pk.to_blob(container)) == (24, 256)


def test_bf16_certified_pack_and_escape_tables(tmp_path):
    pk, W = synth.synth_pack(32, 256, seed=9, tau=2e-3, restore="fp16+bf16", return_weight=True)
    assert pk.esc_idx_bf16.numel() >= pk.esc_idx.numel()
    path = tmp_path / packs.pack_filename("model.layers.0.q_proj.weight", "qvband")
    assert path.name == "model_layers_0_q_proj_weight.qvband"
    path.write_bytes(pk.to_blob())
    # without escape_tables.json: one table (the full list) and the fp16 table is flagged missing
    d = packs.read_qvb8(path.read_bytes(), str(path))
    assert d["restore"] == "fp16+bf16" and d["fp16_table_missing"]
    assert np.array_equal(d["esc_idx"], pk.esc_idx_bf16.numpy())
    keep = np.isin(pk.esc_idx_bf16.numpy(), pk.esc_idx.numpy())
    packs.write_escape_tables(str(tmp_path), {path.name: (pk.esc_idx_bf16.numpy(), keep)})
    d = packs.read_qvb8(path.read_bytes(), str(path))
    assert not d["fp16_table_missing"]
    assert np.array_equal(d["esc_idx"], pk.esc_idx.numpy())
    assert np.array_equal(d["esc_idx_bf16"], pk.esc_idx_bf16.numpy())
    # both certificates
    w = W.double().numpy()
    w16 = oracle.qvb8_dense(d, "fp16").astype(np.float16).astype(np.float64)
    wbf = torch.from_numpy(oracle.qvb8_dense(d, "bf16")).to(torch.bfloat16).double().numpy()
    assert np.abs(w16 - w).max() <= 2e-3 and np.abs(wbf - w).max() <= 2e-3


def test_escape_table_mismatch_is_an_error(tmp_path):
    pk = synth.synth_pack(16, 128, seed=2, restore="fp16+bf16")
    path = tmp_path / "t.qvband"
    path.write_bytes(pk.to_blob())
    idx = pk.esc_idx_bf16.numpy()
    packs.write_escape_tables(str(tmp_path), {"t.qvband": (np.append(idx, 10 ** 6), np.ones(len(idx) + 1, bool))})
    with pytest.raises(packs.EscapeTableError):
        packs.read_qvb8(path.read_bytes(), str(path))


@pytest.mark.parametrize("policy", ["escape_outliers", "inband"])
@pytest.mark.parametrize("tau", [5e-4, 1e-3, 5e-3])
def test_encoder_certifies(policy, tau):
    pk, W = synth.synth_pack(64, 512, seed=int(tau * 1e5), tau=tau, policy=policy, return_weight=True)
    dense = oracle.qvb8_dense(pack_np(pk))
    w = W.double().numpy()
    assert np.abs(dense.astype(np.float16).astype(np.float64) - w).max() <= tau
    assert np.abs(dense.astype(np.float64) - w).max() <= tau
    assert pk.max_err <= tau
    assert int(pk.nbits.max()) <= packs.MAX_CERTIFIED_NBITS
    if policy == "inband":
        assert pk.esc_idx.numel() <= 0.001 * W.numel()          # only rounding stragglers may escape


def test_fp8_escape_pool_and_legacy_versions():
    lut = packs.e4m3_table()
    assert lut[0x38] == 1.0 and lut[0x08] == 2.0 ** -6 and np.isnan(lut[0x7F]) and lut[0x7E] == 448.0
    idx, val = packs.merge_escape_pools(np.array([5, 40]), np.array([1.5, -2.0], np.float32), np.array([17]),
                                        np.array([0x38], np.uint8), np.full(4, 0.25, np.float32), 16)
    assert idx.tolist() == [5, 17, 40] and val.tolist() == [1.5, 0.25, -2.0]


def test_bad_blobs_are_rejected():
    pk = synth.synth_pack(8, 128, seed=1)
    blob = pk.to_blob()
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(b"NOPE" + blob[4:])
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(blob[: len(blob) // 2])
    bad = bytearray(blob); bad[4] = 9                         # version byte
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(bytes(bad))
    bad = bytearray(blob); bad[22] = 1                        # calc_method = table
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(bytes(bad))
    with pytest.raises(ValueError):
        synth.encode_qvb8(torch.full((2, 128), 0.1234567), tau=1e-3)       # not bf16-representable
    with pytest.raises(ValueError):
        synth.encode_qvb8(torch.randn(4, 128).bfloat16() * 1e-5, tau=1e-8)   # below half an fp16 ulp: not certifiable


def test_concat_packs_is_the_members_side_by_side():
    """Same-input fusion (reference formats/qvb8r/fuse.py:22-50 for its entropy-coded format): the fused pack
    restores to the members' dense weights stacked by rows, escapes included."""
    from qvb8_b200 import fuse
    members = [random_pack(40, 256, (5, 7, 8), seed=1, esc_frac=0.01),
               random_pack(17, 256, (3, 6), seed=2, esc_frac=0.0),
               random_pack(64, 256, (7, 11), seed=3, esc_frac=0.02)]
    fused, splits = fuse.concat_packs(members)
    assert fused.Q == 121 and splits == [40, 57]
    want = np.concatenate([oracle.qvb8_dense(pack_np(m)) for m in members], axis=0)
    got = oracle.qvb8_dense(pack_np(fused))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    with pytest.raises(ValueError):
        fuse.concat_packs([members[0], random_pack(8, 128, (7,), seed=4)])


def test_escape_pools_and_tables_match_the_reference(tmp_path):
    """a pack with both escape pools and an escape_tables.json, as the reference's unpack_formula / fp16_list_for /
    select_fp16 read them (fixture made by tests/golden/make_golden.py)"""
    import os
    from conftest import GOLDEN
    z = np.load(os.path.join(GOLDEN, "escpool_32x256.npz"))
    path = tmp_path / "layer_w.qvb8"
    path.write_bytes(z["blob"].tobytes())
    (tmp_path / packs.ESCAPE_TABLES_FILE).write_bytes(z["tables_json"].tobytes())
    d = packs.read_qvb8(z["blob"].tobytes(), str(path))
    assert d["restore"] == "fp16+bf16" and not d["fp16_table_missing"]
    assert np.array_equal(d["esc_idx_bf16"], z["esc_idx"])
    assert np.array_equal(d["esc_vals_bf16"].view(np.uint32), z["esc_vals"].view(np.uint32))
    assert np.array_equal(d["esc_idx"], z["esc_idx_fp16"])
    assert np.array_equal(d["esc_vals"].view(np.uint32), z["esc_vals_fp16"].view(np.uint32))
    # without the tables file the fp16 table is unknown and fp16 runs must be refused later
    d2 = packs.read_qvb8(z["blob"].tobytes(), None)
    assert d2["fp16_table_missing"] and np.array_equal(d2["esc_idx"], z["esc_idx"])


def test_damaged_legacy_blobs_are_refused():
    """the legacy container stores row widths and bit offsets itself: a blob whose fields point outside its payload
    must be refused on the host, never reach a kernel"""
    import struct
    pk = synth.synth_pack(24, 256, 3)
    blob = pk.to_blob("QVB8")
    assert packs.read_qvb8(blob)["Q"] == 24
    with pytest.raises(packs.PackFormatError):                 # payload cut short
        packs.read_qvb8(blob[:len(blob) - 200])
    Q = 24
    nb_at = packs.LEGACY_HEADER_BYTES + 8 * Q
    bad = bytearray(blob); bad[nb_at + 3] = 0                  # a zero-width row
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(bytes(bad))
    bad = bytearray(blob); bad[nb_at + 3] = 15                 # wider than any certified row
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(bytes(bad))
    off_at = nb_at + Q
    bad = bytearray(blob); struct.pack_into("<Q", bad, off_at + 8 * 5, 1 << 40)     # a row far outside the payload
    with pytest.raises(packs.PackFormatError):
        packs.read_qvb8(bytes(bad))
    d = packs.read_qvb8(blob)
    d["esc_idx"] = d["esc_idx"][::-1].copy() if len(d["esc_idx"]) > 1 else np.array([24 * 256], np.int64)
    d["esc_vals"] = d["esc_vals"][:len(d["esc_idx"])] if len(d["esc_vals"]) >= len(d["esc_idx"]) else np.zeros(len(d["esc_idx"]), np.float32)
    with pytest.raises(packs.PackFormatError):
        packs.validate_pack(d)


def test_shards_made_from_pack_bytes_restore_to_slices_of_the_whole():
    """row_shard / column_shard cut a rank's part out of the pack's bytes: no re-encoding, same restored values"""
    import oracle
    from qvb8_b200 import fuse
    from util import pack_np
    pk = synth.synth_pack(96, 512, 8, tau=2e-3, restore="fp16+bf16")
    W = oracle.qvb8_dense(pack_np(pk))
    Wb = oracle.qvb8_dense(pack_np(pk), table="bf16")
    for r0, r1 in ((0, 24), (24, 96), (40, 41)):
        sh = fuse.row_shard(pk, r0, r1)
        assert np.array_equal(oracle.qvb8_dense(pack_np(sh)).view(np.uint32), W[r0:r1].view(np.uint32))
        assert np.array_equal(oracle.qvb8_dense(pack_np(sh), table="bf16").view(np.uint32), Wb[r0:r1].view(np.uint32))
    parts = []
    for c0, c1 in ((0, 128), (128, 256), (256, 512)):
        sh = fuse.column_shard(pk, c0, c1)
        assert (sh.Q, sh.P) == (96, c1 - c0)
        got = oracle.qvb8_dense(pack_np(sh))
        assert np.array_equal(got.view(np.uint32), W[:, c0:c1].view(np.uint32))
        parts.append(got)
        blob = sh.to_blob("QVBD")                                        # a shard is an ordinary pack: it serialises
        assert packs.read_qvb8(blob)["P"] == c1 - c0
    assert np.array_equal(np.hstack(parts), W)
    with pytest.raises(ValueError):
        fuse.column_shard(pk, 4, 128)
