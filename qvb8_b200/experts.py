"""Expert stacks: the stacked layout the grouped expert kernels read, and a mirror of the reference's expert module.

The reference's ``QVBandExpertsV8.build_stack`` (formats/qvb8/backends_experts.py:144-196) concatenates every expert's
packed ids into ONE buffer per projection (16-byte aligned segments, 64 pad bytes), stacks the per-row metadata as
(expert, row) and makes the bit offsets global; it refuses stacks with escapes, differing shapes or P % 8 != 0.
:func:`stack_packs` builds the same layout from :class:`~qvb8_b200.synth.QVB8Pack` objects.
"""
from __future__ import annotations

import torch

from . import ext_qvb8
from .synth import QVB8Pack

STACK_PAD = 64


def stack_packs(members: list[QVB8Pack]) -> dict:
    """{'ids', 'min_s', 'tau_s', 'nbits', 'bit_off', 'Q', 'P'} of all experts of one projection."""
    if not members:
        raise ValueError("stack_packs: no experts")
    Q, P, dev = members[0].Q, members[0].P, members[0].device
    for m in members:
        if (m.Q, m.P) != (Q, P):
            raise ValueError("stack_packs: experts differ in shape")
        if m.esc_idx.numel():
            raise ValueError("stack_packs: an expert carries escape entries (the grouped kernels have no escape pass)")
        if m.device != dev:
            raise ValueError("stack_packs: experts live on different devices")
    if P % 8:
        raise ValueError("stack_packs: P must be a multiple of 8")
    offs, total = [], 0
    for m in members:
        offs.append(total)
        total += (m.ids.numel() + 15) // 16 * 16
    ids_all = torch.zeros(total + STACK_PAD, dtype=torch.uint8, device=dev)
    for off, m in zip(offs, members):
        ids_all[off:off + m.ids.numel()].copy_(m.ids)
    return dict(ids=ids_all, min_s=torch.stack([m.min_s for m in members]).contiguous(),
                tau_s=torch.stack([m.tau_s for m in members]).contiguous(),
                nbits=torch.stack([m.nbits for m in members]).contiguous(),
                bit_off=torch.stack([m.bit_off + o * 8 for m, o in zip(members, offs)]).contiguous(), Q=Q, P=P)


class QVBandExpertsV8(torch.nn.Module):
    """Expert MLP stack over stacked QVB8 packs (fused path of the reference module, backends_experts.py:216-226).

    act: "silu" (gated: the up stack is gate_up with 2 I rows) or "relu2" (non-gated, qvb8_cuda.cu:994-1000)."""

    def __init__(self, up_packs: list[QVB8Pack], down_packs: list[QVB8Pack], *, num_experts: int, act: str = "silu"):
        super().__init__()
        if len(up_packs) != num_experts:
            raise ValueError(f"expected {num_experts} up-projection experts, got {len(up_packs)}")
        if len(down_packs) != num_experts:
            raise ValueError(f"expected {num_experts} down_proj experts, got {len(down_packs)}")
        if act not in ("silu", "relu2"):
            raise ValueError("act must be 'silu' or 'relu2'")
        self.num_experts, self.act = int(num_experts), act
        self.up, self.down = stack_packs(up_packs), stack_packs(down_packs)
        hidden = self.up["Q"] // 2 if act == "silu" else self.up["Q"]
        if hidden != self.down["P"] or self.up["P"] != self.down["Q"]:
            raise ValueError("up and down expert shapes disagree")

    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor):
        u, d = self.up, self.down
        fn = ext_qvb8.ext.moe_experts if self.act == "silu" else ext_qvb8.ext.moe_experts_relu2
        return fn(hidden_states.contiguous(), top_k_index.contiguous(), top_k_weights.float(),
                  u["ids"], u["min_s"], u["tau_s"], u["nbits"], u["bit_off"], u["Q"], u["P"],
                  d["ids"], d["min_s"], d["tau_s"], d["nbits"], d["bit_off"], d["Q"], d["P"])
