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
    """One projection of all experts as the grouped kernels read it: {'ids', 'min_s', 'tau_s', 'nbits', 'bit_off',
    'Q', 'P'}.  Every expert's payload starts on a 16-byte boundary of one shared buffer; its rows keep their own bit
    offsets, shifted by where the expert's payload begins; the per-row vectors become (expert, row) matrices."""
    if not members:
        raise ValueError("stack_packs: no experts")
    first = members[0]
    problems = [f"expert {e}: " + why for e, m in enumerate(members) for ok, why in (
        ((m.Q, m.P) == (first.Q, first.P), f"shape {(m.Q, m.P)} differs from {(first.Q, first.P)}"),
        (m.esc_idx.numel() == 0, "carries escape entries (the grouped kernels have no escape pass)"),
        (m.device == first.device, "lives on another device")) if not ok]
    if first.P % 8:
        problems.append(f"P = {first.P} is not a multiple of 8")
    if problems:
        raise ValueError("stack_packs: " + "; ".join(problems))
    sizes = torch.tensor([m.ids.numel() for m in members], dtype=torch.int64)
    padded = (sizes + 15) // 16 * 16
    starts = torch.cumsum(padded, 0) - padded                           # byte offset of every expert's payload
    payload = torch.zeros(int(padded.sum()) + STACK_PAD, dtype=torch.uint8, device=first.device)
    for m, start in zip(members, starts.tolist()):
        payload.narrow(0, start, m.ids.numel()).copy_(m.ids)
    per_row = lambda field: torch.stack([getattr(m, field) for m in members]).contiguous()
    bit_off = per_row("bit_off") + (starts * 8).to(first.device)[:, None]
    return dict(ids=payload, min_s=per_row("min_s"), tau_s=per_row("tau_s"), nbits=per_row("nbits"),
                bit_off=bit_off.contiguous(), Q=first.Q, P=first.P)


class QVBandExpertsV8(torch.nn.Module):
    """Expert MLP stack over stacked QVB8 packs (fused path of the reference module, backends_experts.py:216-226).

    act: "silu" (gated: the up stack is gate_up with 2 I rows) or "relu2" (non-gated, qvb8_cuda.cu:994-1000).

    Expert parallelism (several devices): a rank holds the experts [first_expert, first_expert + num_experts) of a
    layer with `total_experts`; every rank sees all tokens and the full routing.  ``forward`` renumbers the routing to
    the local stack -- pairs routed to other ranks' experts fall outside it and contribute zero, which the kernels
    guarantee -- computes in fp32, and hands the partial (M, d_model) sums to ``reduce`` (an all-reduce over the ranks,
    set with :meth:`set_reduce`); the result is cast back to the activations' type."""

    def __init__(self, up_packs: list[QVB8Pack], down_packs: list[QVB8Pack], *, num_experts: int, act: str = "silu",
                 first_expert: int = 0, total_experts: int | None = None):
        super().__init__()
        self.first_expert = int(first_expert)
        self.total_experts = int(total_experts) if total_experts is not None else int(num_experts)
        if self.first_expert < 0 or self.first_expert + int(num_experts) > self.total_experts:
            raise ValueError("the local experts must lie inside [0, total_experts)")
        self.reduce = None
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

    @property
    def sharded(self) -> bool:
        return self.total_experts != self.num_experts

    def set_reduce(self, fn) -> None:
        """fn(t) sums the fp32 tensor t over the ranks in place (or returns the sum); None = no exchange."""
        self.reduce = fn

    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor):
        u, d = self.up, self.down
        fn = ext_qvb8.ext.moe_experts if self.act == "silu" else ext_qvb8.ext.moe_experts_relu2
        x, idx = hidden_states.contiguous(), top_k_index.contiguous()
        if self.sharded:
            x = x.float()                                   # partial sums leave the kernels in fp32
            idx = idx - self.first_expert                   # other ranks' experts: outside [0, E), contribute zero
        out = fn(x, idx, top_k_weights.float(),
                 u["ids"], u["min_s"], u["tau_s"], u["nbits"], u["bit_off"], u["Q"], u["P"],
                 d["ids"], d["min_s"], d["tau_s"], d["nbits"], d["bit_off"], d["Q"], d["P"])
        if self.sharded:
            if self.reduce is not None:
                r = self.reduce(out)
                out = out if r is None else r
            out = out.to(hidden_states.dtype)
        return out
