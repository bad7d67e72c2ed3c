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
    """Stands where a member linear stood and answers with its slice of the group's product.  Built from the module it
    replaces: it takes over that module's ``in_features`` / ``out_features`` and its bias (added to the slice)."""

    def __init__(self, group: FusedGroup, index: int, replaced: nn.Module | None = None, *, in_features: int | None = None,
                 out_features: int | None = None, bias=None):
        super().__init__()
        self.index = int(index)
        self.in_features = int(in_features if in_features is not None else replaced.in_features)
        self.out_features = int(out_features if out_features is not None else replaced.out_features)
        self.bias = bias if replaced is None else replaced.bias
        # all members point at ONE group, which the owner registers once; a plain attribute here, not a submodule
        self.__dict__["group"] = group

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        part = self.group.get(x, self.index)
        if self.bias is not None:
            part = part + self.bias.to(part.dtype)
        return part

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, member {self.index} of a fused launch"


def _kind_of_group(owner, names) -> str | None:
    """'qvb8' / 'qvb8r' when every named child of `owner` is a packed linear of that format (qvb8r: loaded from a file,
    which the fused tensor is rebuilt from), else None."""
    children = [getattr(owner, a, None) for a in names]
    if all(isinstance(c, QVBandLinearV8) for c in children):
        return "qvb8"
    if all(isinstance(c, QVBandLinearV8R) and c.path for c in children):
        return "qvb8r"
    return None


def _fuse_owner(owner, names, kind: str) -> None:
    """Replace the children `names` of `owner` by members of one fused group (registered on the owner once)."""
    old = [getattr(owner, a) for a in names]
    shapes = [(c.in_features, c.out_features, c.bias) for c in old]
    if kind == "qvb8":
        group = FusedGroup.from_qvb8(old)
    else:
        device, files = old[0].words.device, [c.path for c in old]
        for a in names:                                              # the separate device copies go before the fused one arrives
            setattr(owner, a, None)
        del old
        if device.type == "cuda":
            torch.cuda.empty_cache()
        parsed = []
        for f in files:
            with open(f, "rb") as fh:
                parsed.append(_packs.read_qvb8r(fh.read(), str(f)))
        group = FusedGroup.from_qvb8r(parsed, device)
    owner.add_module("_qvb8_fused", group)
    for i, (a, (n_in, n_out, b)) in enumerate(zip(names, shapes)):
        setattr(owner, a, FusedMember(group, i, in_features=n_in, out_features=n_out, bias=b))


def fuse_same_input(model: nn.Module, groups=SAME_INPUT_GROUPS) -> int:
    """Replace every same-input group of packed linears in `model` by members of one fused launch; returns the number
    of groups fused.  Called once after the packed modules are in place (the reference's loader calls its counterpart
    through the format's ``finalize`` hook).

    Memory: the owners are found first and fused one at a time, and a group's separate modules are dropped before (qvb8r:
    re-read from their files) or right after (qvb8: byte buffers concatenated) its fused module is built, so at no time
    does the model exist twice on the device -- one group's bytes do, for a moment."""
    found = [(getattr(parent, sub), names) for parent in model.modules() for sub, names in groups
             if getattr(parent, sub, None) is not None and _kind_of_group(getattr(parent, sub), names)]
    fused = 0
    for owner, names in found:
        kind = _kind_of_group(owner, names)                   # (an owner reachable twice was fused the first time)
        if kind is not None:
            _fuse_owner(owner, names, kind)
            fused += 1
    if fused and torch.cuda.is_available():
        torch.cuda.empty_cache()
    return fused
