"""Same-input fusion for a LOADED model: sibling packed linears that are fed the same tensor (q/k/v, gate/up, qkv/z)
become members of one fused linear, and the first member called after a new input computes all of them in one launch.

Counterpart of the reference's formats/qvb8r/fuse.py:52-119 (``FusedGroup``, ``FusedMember``, ``fuse_same_input``),
which does this for its entropy-coded modules only.  Here both formats fuse: QVB8 members by concatenating their packs
(:func:`qvb8_b200.fuse.concat_packs`; rows are independent, so every row is computed from the same bytes) and QVB8R
members by concatenating their parsed files (:func:`qvb8_b200.fuse.concat_qvb8r`).

How a result is shared.  A member's ``forward(x)`` asks the group for its slice.  The group keeps ONE pending result: the
input tensor object it was computed from (held, so its storage cannot be handed to another tensor meanwhile), that
tensor's version counter (an in-place change of x between two members' calls must recompute), the fused output, and
which members have not collected yet.  A member that finds its own slice still pending for the very same input takes it;
anything else -- another tensor, a changed version, a member asking twice -- computes afresh.  When the last member has
collected, the input and the output are released.  This is host-side bookkeeping: under CUDA-graph capture every member
call that computes is captured as a launch, and a replay repeats exactly the captured launches.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import fuse as _fuse
from . import packs as _packs
from .linear import QVBandLinearV8
from .linear_r import QVBandLinearV8R
from .synth import QVB8Pack

# attribute of a decoder block -> sibling linears the block's forward feeds the same tensor (module names as the
# reference's loader sees them, formats/qvb8r/fuse.py:16-20)
SAME_INPUT_GROUPS = (
    ("self_attn", ("q_proj", "k_proj", "v_proj")),
    ("linear_attn", ("in_proj_qkv", "in_proj_z")),
    ("mlp", ("gate_proj", "up_proj")),
)


def pack_of(mod: QVBandLinearV8) -> QVB8Pack:
    """The module's buffers as a pack (tensors shared, nothing copied)."""
    shared = mod.esc_idx_bf16 is mod.esc_idx or mod.esc_idx_bf16.data_ptr() == mod.esc_idx.data_ptr()
    return QVB8Pack(Q=mod.out_features, P=mod.in_features, tau=float("nan"),
                    restore="fp16+bf16" if mod.bf16_certified else "fp16", ids=mod.ids, min_s=mod.min_s, tau_s=mod.tau_s,
                    nbits=mod.nbits, bit_off=mod.bit_off, esc_idx=mod.esc_idx, esc_vals=mod.esc_vals,
                    esc_idx_bf16=mod.esc_idx if shared else mod.esc_idx_bf16,
                    esc_vals_bf16=mod.esc_vals if shared else mod.esc_vals_bf16)


class FusedGroup(nn.Module):
    """The fused linear of a same-input group plus the pending result its members share."""

    def __init__(self, linear: nn.Module, splits: list[int]):
        super().__init__()
        self.lin = linear
        self.splits = list(splits)
        self.n_members = len(self.splits) + 1
        self._pending = None          # (input tensor, its version, output slices, members still to collect)
        self.launches = 0             # fused products computed so far (tests and tuning read it)

    @classmethod
    def from_qvb8(cls, members: list[QVBandLinearV8]) -> "FusedGroup":
        if any(m.bf16_certified != members[0].bf16_certified or m.bf16_gemm != members[0].bf16_gemm for m in members):
            raise ValueError("FusedGroup: members must share their restore code and GEMM mode")
        pack, splits = _fuse.concat_packs([pack_of(m) for m in members])
        lin = QVBandLinearV8.from_pack(pack)
        lin.bf16_gemm = members[0].bf16_gemm
        lin.fp16_table_missing = any(m.fp16_table_missing for m in members)
        return cls(lin, splits)

    @classmethod
    def from_qvb8r(cls, parsed: list[dict], device) -> "FusedGroup":
        d, splits = _fuse.concat_qvb8r(parsed)
        return cls(QVBandLinearV8R(d, device=device), splits)

    def get(self, x: torch.Tensor, i: int) -> torch.Tensor:
        p = self._pending
        if p is None or p[0] is not x or p[1] != x._version or i not in p[3]:
            outs = torch.tensor_split(self.lin(x), self.splits, dim=-1)
            self.launches += 1
            p = self._pending = (x, x._version, outs, set(range(self.n_members)))
        p[3].discard(i)
        out = p[2][i]
        if not p[3]:
            self._pending = None
        return out


class FusedMember(nn.Module):
    """Stands where a member linear stood: same ``in_features`` / ``out_features`` / ``bias``, output taken from the
    group."""

    def __init__(self, group: FusedGroup, i: int, in_features: int, out_features: int, bias):
        super().__init__()
        # every member refers to the one group; it is registered once, under the members' owner, not under each member
        object.__setattr__(self, "group", group)
        self.i, self.in_features, self.out_features = int(i), int(in_features), int(out_features)
        self.bias = bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.group.get(x, self.i)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, member {self.i} of a fused launch"


def _fusable(owner, names) -> str | None:
    mods = [getattr(owner, a, None) for a in names]
    if all(isinstance(m, QVBandLinearV8) for m in mods):
        return "qvb8"
    if all(isinstance(m, QVBandLinearV8R) and m.path for m in mods):
        return "qvb8r"
    return None


def fuse_same_input(model: nn.Module, groups=SAME_INPUT_GROUPS) -> int:
    """Replace every same-input group of packed linears in `model` by members of one fused launch; returns the number
    of groups fused.  Called once after the packed modules are in place (the reference's loader calls its counterpart
    through the format's ``finalize`` hook).

    Memory: the owners are collected first, and each group's separate modules are dropped before its fused module is
    built, so at no time does the model exist twice on the device (QVB8R members are re-read from their files; QVB8
    members' byte buffers are concatenated, which needs the group's bytes twice for a moment, not the model's)."""
    todo = []
    for parent in model.modules():
        for sub, names in groups:
            owner = getattr(parent, sub, None)
            if owner is not None and _fusable(owner, names):
                todo.append((owner, names))
    done = 0
    for owner, names in todo:
        kind = _fusable(owner, names)
        if kind is None:                                     # (an owner reachable twice was fused the first time)
            continue
        meta = [(getattr(owner, a).in_features, getattr(owner, a).out_features, getattr(owner, a).bias) for a in names]
        if kind == "qvb8":
            group = FusedGroup.from_qvb8([getattr(owner, a) for a in names])
            for a in names:
                setattr(owner, a, None)
        else:
            device = getattr(owner, names[0]).words.device
            paths = [getattr(owner, a).path for a in names]
            for a in names:                                  # the separate copies go before the fused one arrives
                setattr(owner, a, None)
            if device.type == "cuda":
                torch.cuda.empty_cache()
            parsed = []
            for pth in paths:
                with open(pth, "rb") as fh:
                    parsed.append(_packs.read_qvb8r(fh.read(), str(pth)))
            group = FusedGroup.from_qvb8r(parsed, device)
            del parsed
        owner.add_module("_qvb8_fused", group)
        for i, (a, (n_in, n_out, bias)) in enumerate(zip(names, meta)):
            setattr(owner, a, FusedMember(group, i, n_in, n_out, bias))
        done += 1
    if done and torch.cuda.is_available():
        torch.cuda.empty_cache()
    return done
