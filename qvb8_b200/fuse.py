"""Same-input fusion for QVB8: sibling linears that read the same activation (q/k/v, gate/up) run as ONE launch.

The reference does this for its entropy-coded format (formats/qvb8r/fuse.py:1-60: the members' data is concatenated
into one virtual tensor, every kernel path runs unchanged on it, the output is split back per member).  A QVB8 pack
concatenates even more simply, because its rows are independent: the bit-packed rows are laid back to back, the
per-row vectors are concatenated, row bit offsets are shifted by the bits that precede them, and escape positions
by the rows that precede them.  Each row's sum is computed exactly as in the separate launch, so the fused output is
bit-identical to the members' outputs side by side.
"""
from __future__ import annotations

import torch

from . import packs
from .synth import QVB8Pack


def concat_packs(members: list[QVB8Pack]) -> tuple[QVB8Pack, list[int]]:
    """One pack holding the rows of `members` in order.  Returns (pack, row split points for torch.tensor_split)."""
    if not members:
        raise ValueError("concat_packs: no members")
    P = members[0].P
    dev = members[0].device
    for m in members:
        if m.P != P:
            raise ValueError("concat_packs: members must share P (they read the same activation)")
        if m.device != dev:
            raise ValueError("concat_packs: members must live on one device")
        if m.restore != members[0].restore:
            raise ValueError("concat_packs: members must share the restore code")
    pad = packs.PAYLOAD_PAD
    ids, bit_off, e_idx, e_val, e_idx16, e_val16 = [], [], [], [], [], []
    bits = 0
    rows = 0
    for m in members:
        payload = m.ids[:m.ids.numel() - pad]
        if (bits % 8) or int(m.bit_off[0].item()) != 0:
            raise ValueError("concat_packs: member payloads must be byte-aligned and start at bit 0")
        ids.append(payload)
        bit_off.append(m.bit_off + bits)
        e_idx.append(m.esc_idx + rows * P)
        e_val.append(m.esc_vals)
        e_idx16.append(m.esc_idx_bf16 + rows * P)
        e_val16.append(m.esc_vals_bf16)
        bits += payload.numel() * 8
        rows += m.Q
    ids.append(torch.zeros(pad, dtype=torch.uint8, device=dev))
    hist: dict = {}
    for m in members:
        for b, n in m.stats.get("nbits_hist", {}).items():
            hist[b] = hist.get(b, 0) + n
    same_table = all(m.esc_idx_bf16 is m.esc_idx for m in members)
    esc_idx, esc_vals = torch.cat(e_idx), torch.cat(e_val)
    fused = QVB8Pack(
        Q=rows, P=P, tau=max(m.tau for m in members), restore=members[0].restore, ids=torch.cat(ids),
        min_s=torch.cat([m.min_s for m in members]), tau_s=torch.cat([m.tau_s for m in members]),
        nbits=torch.cat([m.nbits for m in members]), bit_off=torch.cat(bit_off), esc_idx=esc_idx, esc_vals=esc_vals,
        esc_idx_bf16=esc_idx if same_table else torch.cat(e_idx16),
        esc_vals_bf16=esc_vals if same_table else torch.cat(e_val16),
        max_err=max(m.max_err for m in members), stats={"nbits_hist": hist, "members": [m.Q for m in members]})
    splits, acc = [], 0
    for m in members[:-1]:
        acc += m.Q
        splits.append(acc)
    return fused, splits


# (group name, member names) of a decoder layer whose members are fed the same tensor
SAME_INPUT_GROUPS = (("qkv", ("q", "k", "v")), ("gate_up", ("gate", "up")))
