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
