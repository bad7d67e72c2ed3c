"""``QVBandEmbeddingV8``: an ``nn.Embedding`` replacement whose table lives in device memory only as a QVB8 pack.

Mirrors the reference module of the same name (formats/qvb8/embedding.py:21-160): the same buffers and constructor
keywords, ``forward`` = decode the requested rows + write their escapes over + cast, ``weight`` = the whole table.
The reference decodes with torch ops and walks the escapes in a Python loop per looked-up row (:124-150); here one
kernel (``qvb8_embed_rows``) gathers the rows, restores them with the reference's arithmetic (``min_s + id * tau_s``:
a multiplication and an addition in fp32, then one cast) and applies the escapes, so the values are bit-identical.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import lib as _lib

FP32_METADATA = ("min_s", "tau_s", "esc_vals")


class QVBandEmbeddingV8(nn.Module):
    def __init__(self, *, min_s, nbits, bit_off, ids, Q, P, tau_s, esc_idx, esc_vals, out_dtype=torch.bfloat16):
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(Q), int(P)
        self._out_dtype = out_dtype
        if esc_idx.numel() > 1 and not bool((esc_idx[1:] >= esc_idx[:-1]).all()):
            o = torch.argsort(esc_idx, stable=True)          # the kernel finds a row's escapes by binary search
            esc_idx, esc_vals = esc_idx[o].contiguous(), esc_vals[o].contiguous()
        for name, t in (("tau_s", tau_s), ("min_s", min_s), ("nbits", nbits), ("bit_off", bit_off), ("ids", ids),
                        ("esc_idx", esc_idx), ("esc_vals", esc_vals)):
            self.register_buffer(name, t, persistent=False)

    @classmethod
    def from_pack(cls, pk, out_dtype=torch.bfloat16) -> "QVBandEmbeddingV8":
        """From a :class:`qvb8_b200.synth.QVB8Pack` (or any object with the same fields)."""
        return cls(min_s=pk.min_s, nbits=pk.nbits, bit_off=pk.bit_off, ids=pk.ids, Q=pk.Q, P=pk.P, tau_s=pk.tau_s,
                   esc_idx=pk.esc_idx, esc_vals=pk.esc_vals, out_dtype=out_dtype)

    def _apply(self, fn, recurse=True):
        """model.to(torch.bfloat16) must not round min_s / tau_s / esc_vals (embedding.py:24-27)."""
        keep = {n: self._buffers[n] for n in FP32_METADATA if self._buffers.get(n) is not None}
        for n in keep:
            self._buffers[n] = None
        try:
            out = super()._apply(fn, recurse)
        finally:
            dev = self._buffers["ids"].device
            for n, b in keep.items():
                self._buffers[n] = b.to(dev)
        return out

    def extra_repr(self):
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}, dtype={self._out_dtype}"

    def _pack(self):
        return _lib.pack_struct(self.ids, self.min_s, self.tau_s, self.nbits, self.bit_off, self.embedding_dim,
                                self.esc_idx, self.esc_vals)

    def _rows(self, rows: torch.Tensor, dtype) -> torch.Tensor:
        st, keep = self._pack()
        return _lib.embed_rows(st, keep, rows, dtype)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        dev_in = input.device
        flat = input.reshape(-1).to(device=self.ids.device, dtype=torch.int64).contiguous()
        if flat.numel() and not torch.cuda.is_current_stream_capturing():
            lo, hi = int(flat.min()), int(flat.max())       # torch's embedding refuses such indices too
            if lo < 0 or hi >= self.num_embeddings:
                raise IndexError(f"QVBandEmbeddingV8: index out of range [0, {self.num_embeddings})")
        out = self._rows(flat, self._out_dtype)
        return out.reshape(*input.shape, self.embedding_dim).to(dev_in)

    @property
    def weight(self) -> torch.Tensor:
        """Dense (Q, P) table, for callers that need all of it (tied lm_head, audits)."""
        return self._rows(torch.arange(self.num_embeddings, device=self.ids.device), self._out_dtype)


class QVBandEmbeddingV8R(nn.Module):
    """``nn.Embedding`` over an entropy-coded (.qvb8r) table.  The reference module of this name decodes the looked-up
    rows on the host so that the table never occupies a small card's memory (formats/qvb8r/module.py:340-391); here
    the table (about 5 bits per weight) stays in device memory and ``qvb8r_embed_rows`` decodes the rows there, with
    the reference's arithmetic, so the values are bit-identical."""

    def __init__(self, d: dict, out_dtype=torch.bfloat16, device="cuda", path: str | None = None):
        super().__init__()
        from .ext_qvb8r import EmbeddingTable
        self.num_embeddings, self.embedding_dim = int(d["Q"]), int(d["P"])
        self._out_dtype, self.device, self.path = out_dtype, torch.device(device), path
        self.table = EmbeddingTable.from_parsed(d, self.device)

    @classmethod
    def from_packfile(cls, path: str, *, out_dtype=torch.bfloat16, tau: float | None = None, device: str = "cuda",
                      blob: bytes | None = None) -> "QVBandEmbeddingV8R":
        from . import packs
        if blob is None:
            with open(path, "rb") as fh:
                blob = fh.read()
        return cls(packs.read_qvb8r(blob, str(path)), out_dtype=out_dtype, device=device, path=path)

    def extra_repr(self):
        return f"{self.num_embeddings}, {self.embedding_dim}, rows decoded on the device"

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        flat = input.reshape(-1).to(device=self.device, dtype=torch.int64)
        if flat.numel() and not torch.cuda.is_current_stream_capturing():
            if int(flat.min()) < 0 or int(flat.max()) >= self.num_embeddings:
                raise IndexError(f"QVBandEmbeddingV8R: index out of range [0, {self.num_embeddings})")
        return self.table.lookup(flat).to(self._out_dtype).reshape(*input.shape, self.embedding_dim)

    @property
    def weight(self) -> torch.Tensor:
        rows = torch.arange(self.num_embeddings, device=self.device)
        return self.table.lookup(rows).to(self._out_dtype)
