"""Pack directory + manifest: names, keys, round trip, modules built from it (CPU, no kernel call)."""
import json

import numpy as np
import pytest
import torch

from qvb8_b200 import packdir, packs, synth


def _pack(Q, P, seed):
    return synth.encode_qvb8(synth.synth_weight(Q, P, seed), tau=1e-3)


def test_names_and_expert_keys():
    assert packs.pack_filename("model.layers.0.self_attn.q_proj.weight", "qvb8") == "model_layers_0_self_attn_q_proj_weight.qvb8"
    k = packdir.expert_key("model.layers.3.mlp.experts.gate_up_proj", 7)
    assert k.endswith("#expert007") and packdir.split_expert_key(k) == ("model.layers.3.mlp.experts.gate_up_proj", 7)
    assert packdir.split_expert_key("lm_head.weight") == ("lm_head.weight", None)


def test_directory_round_trip(tmp_path):
    tensors = {"model.layers.0.mlp.down_proj.weight": _pack(32, 128, 1),
               packdir.expert_key("model.layers.0.mlp.experts.down_proj", 0): _pack(16, 64, 2),
               packdir.expert_key("model.layers.0.mlp.experts.down_proj", 1): _pack(16, 64, 3)}
    man = packdir.write_pack_dir(str(tmp_path), tensors, fmt="qvb8", tau=1e-3, hf_model="synthetic/9b")
    got = packdir.read_manifest(str(tmp_path))
    assert got == json.loads(json.dumps(man)) and got["format"] == "qvb8" and got["failed"] == []
    e = got["tensors"]["model.layers.0.mlp.down_proj.weight"]
    assert e["pack"] == "model_layers_0_mlp_down_proj_weight.qvb8" and (e["Q"], e["P"]) == (32, 128)
    assert e["bytes"] == (tmp_path / e["pack"]).stat().st_size and e["max_err"] <= 1e-3
    assert packdir.expert_slices(got, "model.layers.0.mlp.experts.down_proj") == [
        "model.layers.0.mlp.experts.down_proj#expert000", "model.layers.0.mlp.experts.down_proj#expert001"]
    lin = packdir.load_linear(str(tmp_path), "model.layers.0.mlp.down_proj.weight", device="cpu")
    pk = tensors["model.layers.0.mlp.down_proj.weight"]
    assert (lin.out_features, lin.in_features) == (32, 128)
    assert torch.equal(lin.ids, pk.ids) and torch.equal(lin.tau_s, pk.tau_s) and torch.equal(lin.esc_idx_bf16, pk.esc_idx_bf16)
    with pytest.raises(KeyError):
        packdir.load_linear(str(tmp_path), "model.layers.9.absent", device="cpu")


def test_qvb8r_directory_and_bad_manifest(tmp_path):
    W = synth.synth_weight(24, 128, 5)
    d = synth.encode_qvb8r(W, tau=2e-3, K=2, T=4)
    packdir.write_pack_dir(str(tmp_path), {"blk.attn.o.weight": d}, fmt="qvb8r", tau=2e-3)
    mod = packdir.load_linear(str(tmp_path), "blk.attn.o.weight", device="cpu")
    assert type(mod).__name__ == "QVBandLinearV8R" and (mod.out_features, mod.in_features) == (24, 128)
    assert np.array_equal(mod.perm.numpy(), np.asarray(d["perm"], np.int32))
    (tmp_path / "manifest.json").write_text(json.dumps({"format": "gguf", "tensors": {}}))
    with pytest.raises(packs.PackFormatError):
        packdir.read_manifest(str(tmp_path))


def _module_dense(mod):
    """restore a QVBandLinearV8's buffers with the oracle (fp16 table written over)"""
    import oracle
    c = lambda t: t.detach().cpu().numpy()
    return oracle.qvb8_dense(dict(Q=mod.out_features, P=mod.in_features, ids=c(mod.ids), nbits=c(mod.nbits),
                                  bit_off=c(mod.bit_off), min_s=c(mod.min_s), tau_s=c(mod.tau_s), esc_idx=c(mod.esc_idx),
                                  esc_vals=c(mod.esc_vals)))


def test_shard_aware_loading(tmp_path):
    """a rank builds only its share of a tensor, cut on the host from the file's bytes: row shards are the whole's rows
    (bias sliced with them), column shards its columns (bias on rank 0), qvb8r shards runs of whole tiles"""
    pk = synth.encode_qvb8(synth.synth_weight(64, 256, 21), tau=1e-3)
    r = synth.encode_qvb8r(synth.synth_weight(40, 128, 22), tau=2e-3, K=2, T=4)
    qdir, rdir = tmp_path / "q", tmp_path / "r"
    qdir.mkdir(); rdir.mkdir()
    packdir.write_pack_dir(str(qdir), {"blk.mlp.up.weight": pk}, fmt="qvb8", tau=1e-3)
    packdir.write_pack_dir(str(rdir), {"blk.mlp.up.weight": r}, fmt="qvb8r", tau=2e-3)
    whole = _module_dense(packdir.load_linear(str(qdir), "blk.mlp.up.weight", device="cpu"))
    bias = torch.arange(64, dtype=torch.float32)
    world = 4
    for rank in range(world):
        rows = packdir.load_linear(str(qdir), "blk.mlp.up.weight", device="cpu", bias=bias, shard=(rank, world, "rows"))
        assert (rows.out_features, rows.in_features) == (16, 256)
        assert np.array_equal(_module_dense(rows).view(np.uint32), whole[rank * 16:(rank + 1) * 16].view(np.uint32))
        assert torch.equal(rows.bias.data, bias[rank * 16:(rank + 1) * 16])
        cols = packdir.load_linear(str(qdir), "blk.mlp.up.weight", device="cpu", bias=bias, shard=(rank, world, "cols"))
        assert (cols.out_features, cols.in_features) == (64, 64)
        assert np.array_equal(_module_dense(cols).view(np.uint32), whole[:, rank * 64:(rank + 1) * 64].view(np.uint32))
        assert (cols.bias is not None) == (rank == 0)
    got = np.zeros((40, 128), np.float32)
    for rank in range(3):
        sh = packdir.load_linear(str(rdir), "blk.mlp.up.weight", device="cpu", shard=(rank, 3))
        assert type(sh).__name__ == "QVBandLinearV8RShard" and sh.out_features == 40
        if sh.local is not None:
            assert sh.local.out_features == sh.rows.numel()
        got[sh.rows.numpy()] = 1.0
    assert got.min() == 1.0                                   # every row belongs to exactly one shard's run of tiles
    with pytest.raises(ValueError):
        packdir.load_linear(str(qdir), "blk.mlp.up.weight", device="cpu", shard=(0, 3, "rows"))   # 64 rows / 3 ranks
    with pytest.raises(ValueError):
        packdir.load_linear(str(qdir), "blk.mlp.up.weight", device="cpu", shard=(4, 4, "rows"))
