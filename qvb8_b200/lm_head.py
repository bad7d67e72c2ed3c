"""Greedy decoding head over a packed lm_head: the next token of every sequence without materialising the logits
anywhere but on the rank that computed them.

The lm_head is the largest linear of a decoder (vocabulary x d_model).  The reference runs it like any other packed
linear and takes ``torch.argmax`` of the logits (run/run_inference.py); with the vocabulary split over ranks that would
mean gathering V floats per token.  Here a rank holds the output rows [v0, v1) of the head (a row shard of the pack:
``QVBandLinearV8.row_subset`` / ``fuse.row_shard``), computes its slice of the logits with the streaming kernel, reduces
it to ONE (value, token) pair per sequence on the device (``qvb8_argmax_rows``: largest value, lowest index among equals)
and the ranks exchange those pairs -- 16 bytes per sequence and rank -- and pick the winner by the same rule, so every
rank ends up with the same tokens, and with the tokens a single device would have chosen.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import lib as _lib


def pick_best(values: torch.Tensor, indices: torch.Tensor):
    """The winners among candidate pairs: values (R, M) and their token indices (R, M) -> (M,) values, (M,) indices.
    Larger value wins; among equal values the lower token index (what one argmax over the whole vocabulary returns)."""
    best = values.max(dim=0).values
    tied = values == best.unsqueeze(0)
    sentinel = torch.iinfo(indices.dtype).max
    tokens = torch.where(tied, indices, torch.full_like(indices, sentinel)).min(dim=0).values
    return best, tokens


class GreedyHead(nn.Module):
    """``forward(hidden) -> token ids``.

    linear: the head, or this rank's rows [first_row, first_row + linear.out_features) of it; group: the ranks that
    hold the other rows (None: a single device).  The logits are fp32; a bias of the head is part of them."""

    def __init__(self, linear: nn.Module, first_row: int = 0, group=None):
        super().__init__()
        self.linear = linear
        self.first_row = int(first_row)
        self.group = group

    def local_best(self, hidden: torch.Tensor):
        """This rank's candidates: (values (M,), token ids (M,)) over its rows."""
        x = hidden.reshape(-1, hidden.shape[-1])
        logits = self.linear(x).float().contiguous()
        return _lib.argmax_rows(logits, self.first_row)

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        val, tok = self.local_best(hidden)
        if self.group is not None:
            import torch.distributed as dist
            world = dist.get_world_size(self.group)
            if world > 1:
                vals = torch.empty(world * val.numel(), dtype=val.dtype, device=val.device)
                toks = torch.empty(world * tok.numel(), dtype=tok.dtype, device=tok.device)
                dist.all_gather_into_tensor(vals, val.contiguous(), group=self.group)
                dist.all_gather_into_tensor(toks, tok.contiguous(), group=self.group)
                val, tok = pick_best(vals.view(world, -1), toks.view(world, -1))
        return tok.reshape(hidden.shape[:-1])
