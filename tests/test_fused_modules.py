"""Same-input fusion of a loaded model (qvb8_b200.fused_modules): the sharing rules of a group's pending result on CPU,
and on a GPU a small block of packed linears before and after fuse_same_input."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from qvb8_b200 import packs, synth
from qvb8_b200.fused_modules import FusedGroup, FusedMember, fuse_same_input

DEV = "cuda:0"


class _Counting(nn.Module):
    """stands for the fused linear: y = x @ W^T, and counts its calls"""

    def __init__(self, W):
        super().__init__()
        self.W, self.calls = W, 0

    def forward(self, x):
        self.calls += 1
        return x @ self.W.t()


def _group():
    W = torch.arange(6 * 4, dtype=torch.float32).reshape(6, 4)
    g = FusedGroup(_Counting(W), [2, 5])                         # members of 2, 3 and 1 rows
    members = [FusedMember(g, i, in_features=4, out_features=n) for i, n in enumerate((2, 3, 1))]
    return W, g, members


def test_one_product_serves_every_member_once():
    W, g, (a, b, c) = _group()
    x = torch.ones(2, 4)
    ya, yb, yc = a(x), b(x), c(x)
    assert g.lin.calls == 1
    assert torch.equal(torch.cat([ya, yb, yc], -1), x @ W.t())
    assert g._pending is None                                    # input and output released after the last member
    a(x)                                                         # the same tensor again: a new round
    assert g.lin.calls == 2


def test_anything_but_the_same_unchanged_tensor_recomputes():
    W, g, (a, b, c) = _group()
    x = torch.ones(1, 4)
    a(x)
    a(x)                                                         # a member asking twice
    assert g.lin.calls == 2
    b(x)
    assert g.lin.calls == 2
    x.add_(1.0)                                                  # changed in place between two members' calls
    yc = c(x)
    assert g.lin.calls == 3 and torch.equal(yc, (x @ W.t())[:, 5:])
    x2 = x.clone()                                               # an equal tensor is still another tensor
    b(x2)
    assert g.lin.calls == 4


def test_member_adds_its_own_bias():
    W, g, _ = _group()
    m = FusedMember(g, 1, in_features=4, out_features=3, bias=torch.tensor([1.0, 2.0, 3.0]))
    x = torch.ones(1, 4)
    assert torch.equal(m(x), (x @ W.t())[:, 2:5] + torch.tensor([1.0, 2.0, 3.0]))
    assert "member 1" in m.extra_repr()


class _Attn(nn.Module):
    def __init__(self, q, k, v):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = q, k, v


class _Mlp(nn.Module):
    def __init__(self, g, u, d):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = g, u, d


class _Block(nn.Module):
    def __init__(self, attn, mlp):
        super().__init__()
        self.self_attn, self.mlp = attn, mlp


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 5, 20, 130])
def test_fuse_qvb8_block(cuda_lib, M):
    from qvb8_b200.linear import QVBandLinearV8
    P = 512

    def lin(Q, seed, bias=False):
        pk = synth.synth_pack(Q, P, seed=seed, device=DEV)
        b = torch.linspace(-1, 1, Q, device=DEV) if bias else None
        return QVBandLinearV8.from_pack(pk, bias=b)
    blk = _Block(_Attn(lin(128, 1), lin(32, 2, bias=True), lin(32, 3)), _Mlp(lin(256, 4), lin(256, 5), lin(64, 6)))
    model = nn.ModuleList([blk])
    x = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.bfloat16)
    names = [("self_attn", n) for n in ("q_proj", "k_proj", "v_proj")] + [("mlp", n) for n in ("gate_proj", "up_proj")]
    before = {n: getattr(getattr(blk, o), n)(x).float() for o, n in names}
    down = blk.mlp.down_proj
    assert fuse_same_input(model) == 2
    assert blk.mlp.down_proj is down                             # not part of a group: untouched
    for o, n in names:
        m = getattr(getattr(blk, o), n)
        assert isinstance(m, FusedMember)
        got = m(x).float()
        # rows are independent, but a pack of another height may split K differently: equal up to the order of the
        # fp32 sums, i.e. to an ulp of the bf16 product (magnitudes up to 2 here; a member's bias is added after that
        # rounding, so the absolute error does not shrink with the result)
        assert torch.allclose(got, before[n], rtol=2.0 ** -7, atol=2.0 ** -6), n
        assert float((got - before[n]).norm() / before[n].norm()) < 8e-3, n   # (one bf16 ulp is 4e-3 to 8e-3)
    assert blk.self_attn._qvb8_fused.launches == 1 and blk.mlp._qvb8_fused.launches == 1
    assert fuse_same_input(model) == 0                           # nothing left to fuse


@pytest.mark.gpu
def test_fuse_qvb8r_block(cuda_lib, tmp_path):
    from qvb8_b200.linear_r import QVBandLinearV8R
    P = 256
    mods = []
    for i, Q in enumerate((64, 32, 48)):
        d = synth.encode_qvb8r(synth.synth_weight(Q, P, 70 + i), tau=2e-3, K=2, T=2)
        blob = packs.write_qvb8r(d, Q=Q, P=P, min_s=d["min_s"], tau_s=d["tau_s"], esc_idx=d["esc_idx"], esc_val=d["esc_val"],
                                 esc_delta=d["esc_delta"], cert=dict(tau=d["tau"], max_err=d["max_err"]))
        path = tmp_path / f"w{i}.qvb8r"
        path.write_bytes(blob)
        mods.append(QVBandLinearV8R.from_packfile(str(path), device=DEV))
    attn = _Attn(*mods)
    del mods
    wrap = nn.Module()
    wrap.self_attn = attn
    x = synth.synth_activation(3, P, seed=9, device=DEV, dtype=torch.bfloat16)
    before = [getattr(attn, n)(x).float() for n in ("q_proj", "k_proj", "v_proj")]
    assert fuse_same_input(wrap) == 1
    after = [getattr(attn, n)(x).float() for n in ("q_proj", "k_proj", "v_proj")]
    for a, b in zip(after, before):
        assert a.shape == b.shape and torch.allclose(a, b, rtol=2.0 ** -7, atol=2.0 ** -6)
    assert attn._qvb8_fused.launches == 1
