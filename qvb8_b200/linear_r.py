"""``QVBandLinearV8R``: an ``nn.Linear`` replacement whose weight lives in device memory only as an entropy-coded
QVB8R pack.

Mirrors the reference module of the same name (formats/qvb8r/module.py:57-325): buffers built from a parsed
``.qvb8r`` dict, ``from_packfile``, ``forward`` dispatch by the row count M of the flattened input, ``dense``.

    M = 1        ``gemv``   fp32 band value x fp32 activation
    M = 2..8     ``multi``  the same for several rows (a bf16 activation is read as it is: exact in fp32)
    M = 9..16    ``tc``     band value rounded once to fp16 x saturated-fp16 activation
    M = 17..48   equal passes of <= 16 rows through ``tc`` (module.py:303-312)
    M  > 48      the weight is restored chunk by chunk (whole blocks, <= CHUNK_BYTES of fp16 each) in sorted row order,
                 escapes written over, rows put back in output order, one fp16 GEMM with fp32 accumulation per chunk

After every kernel product the escape pass adds ``sum_e x[m, c_e] * delta_e`` per output in stored order
(module.py:212-214); for the ``tc`` path the differences are taken against the fp16-rounded band value (:121-124).
One escape table (the file's) is kept; the reference's split fp16 / bf16 tables and its disk-resident mode are loader
features outside the product path.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn

from . import packs, rans
from .ext_qvb8r import TILES_PER_BLOCK, core_tensors, ext

FP32_METADATA = ("min_s", "tau_s", "esc_val", "esc_delta", "esc_delta16", "chunk_evals")
TC_MAX = 16
TC_SPLIT_MAX = 48


class QVBandLinearV8R(nn.Module):
    CHUNK_BYTES = 512 << 20       # decoded fp16 weight per GEMM in the many-rows path (module.py:63)

    def __init__(self, d: dict, bias=None, device="cuda", path: str | None = None):
        super().__init__()
        self.path = path
        Q, P = int(d["Q"]), int(d["P"])
        self.out_features, self.in_features, self.T = Q, P, int(d["T"])
        dev = torch.device(device)
        names = ("words", "off", "states", "tiles", "blocks8", "tab", "perm", "min_s", "tau_s", "drow")
        for name, t in zip(names, core_tensors(d, dev)):
            self.register_buffer(name, t, persistent=False)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(dev)
        # escapes grouped by output row (CSR, sorted by row then column): one thread per (m, q) sums its group in this
        # fixed order
        ei = np.asarray(d["esc_idx"], np.int64)
        ev = np.asarray(d["esc_val"], np.float32)
        ed = np.asarray(d["esc_delta"], np.float32)
        o = np.argsort(ei, kind="stable")
        ei, ev, ed = ei[o], ev[o], ed[o]
        uq, cnt = np.unique(ei // P, return_counts=True)
        band = ev - ed
        for name, a, dt in (("esc_uq", uq, np.int64), ("esc_ptr", np.concatenate([[0], np.cumsum(cnt)]), np.int64),
                            ("esc_c", ei % P, np.int64), ("esc_delta", ed, np.float32),
                            ("esc_delta16", ev - band.astype(np.float16).astype(np.float32), np.float32),
                            ("esc_flat", ei, np.int64), ("esc_val", ev, np.float32)):
            self.register_buffer(name, t(a, dt), persistent=False)
        self.bias = None if bias is None else nn.Parameter(bias.detach().to(dev), requires_grad=False)

        # many rows: chunks of whole blocks and the escapes inside each.  Per chunk: first block, blocks, first sorted
        # row, rows, [o0, o1) into chunk_orows, [e0, e1) into chunk_eflat / chunk_evals  (module.py:127-161)
        tiles = np.asarray(d["tiles"], np.int64).reshape(-1, 3)
        blocks = rans.blocks_for(tiles, TILES_PER_BLOCK)
        perm = np.asarray(d["perm"], np.int64)
        inv = np.empty(Q, np.int64)
        inv[perm] = np.arange(Q)
        rows_per_block = [int(tiles[t0:t0 + n, 2].sum()) for _, t0, n in blocks]
        first_row = [int(tiles[t0, 1]) for _, t0, n in blocks]
        budget = max(1, self.CHUNK_BYTES // (2 * P))
        spans, orows, b, o0 = [], [], 0, 0
        while b < len(blocks):
            e, rows = b, 0
            while e < len(blocks) and (e == b or rows + rows_per_block[e] <= budget):
                rows += rows_per_block[e]
                e += 1
            base = first_row[b]
            orows.append(perm[base:base + rows])
            spans.append((b, e - b, base, rows, o0, o0 + rows))
            o0 += rows
            b = e
        sp = inv[ei // P] if ei.size else np.zeros(0, np.int64)
        flat, vals, self.chunks, e0 = [], [], [], 0
        for span in spans:
            base, rows = span[2], span[3]
            sel = np.nonzero((sp >= base) & (sp < base + rows))[0]
            flat.append((sp[sel] - base) * P + ei[sel] % P)
            vals.append(ev[sel])
            self.chunks.append(span + (e0, e0 + len(sel)))
            e0 += len(sel)
        cat = lambda xs, dt: np.concatenate(xs).astype(dt) if xs else np.zeros(0, dt)
        self.register_buffer("chunk_orows", t(cat(orows, np.int64), np.int64), persistent=False)
        self.register_buffer("chunk_eflat", t(cat(flat, np.int64), np.int64), persistent=False)
        self.register_buffer("chunk_evals", t(cat(vals, np.float32), np.float32), persistent=False)

    @classmethod
    def from_packfile(cls, path: str, *, bias=None, tau: float | None = None, device: str = "cuda",
                      blob: bytes | None = None) -> "QVBandLinearV8R":
        """`tau` is accepted for call-site compatibility and ignored: each file carries its own certified tau."""
        if blob is None:
            with open(path, "rb") as f:
                blob = f.read()
        return cls(packs.read_qvb8r(blob, str(path)), bias=bias, device=device, path=path)

    def _apply(self, fn, recurse=True):
        """module.to(...) / .half() / .bfloat16(): the fp32 metadata only ever changes DEVICE (module.py:188-202)."""
        keep = {n: self._buffers[n] for n in FP32_METADATA if self._buffers.get(n) is not None}
        for n in keep:
            self._buffers[n] = None
        try:
            out = super()._apply(fn, recurse)
        finally:
            dev = self._buffers["words"].device
            for n, b in keep.items():
                self._buffers[n] = b.to(dev)
        return out

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"

    # ---- kernel paths -------------------------------------------------------------------------------------
    def _core(self):
        return (self.words, self.off, self.states, self.tiles, self.blocks8, self.tab, self.perm, self.min_s,
                self.tau_s, self.drow)

    def _escapes(self, xf, y, delta):
        y = y.contiguous()
        ext.fix_escapes(xf, self.esc_uq, self.esc_ptr, self.esc_c, delta, y)
        return y

    def _gemv(self, x2):
        xf = x2.float().contiguous()
        return self._escapes(xf, ext.gemv(xf.view(-1), *self._core()).view(1, -1), self.esc_delta)

    def _multi(self, x2):
        xf = x2.float().contiguous()
        xk = x2.contiguous() if x2.dtype == torch.bfloat16 else xf
        return self._escapes(xf, ext.multi(xk, *self._core()), self.esc_delta)

    def _tc(self, x2):
        xf = x2.float().contiguous()
        xh = xf.clamp(-65504, 65504).half().contiguous()
        return self._escapes(xf, ext.tc(xh, *self._core(), self.T), self.esc_delta16)

    def _chunked(self, x2):
        xh = x2.half()
        xh = xh.clamp(-65504, 65504) if xh is x2 else xh.clamp_(-65504, 65504)
        y = torch.empty(x2.shape[0], self.out_features, device=x2.device, dtype=torch.float32)
        for b0, nb, base, rows, o0, o1, e0, e1 in self.chunks:
            W = ext.decode(*self._core(), self.in_features, 0, b0, nb, base, rows)
            if e1 > e0:
                W.view(-1)[self.chunk_eflat[e0:e1]] = self.chunk_evals[e0:e1].half()
            if len(self.chunks) == 1:                   # rows back in output order: the GEMM writes y directly
                Wo = torch.empty_like(W).index_copy_(0, self.chunk_orows[o0:o1], W)
                return torch.mm(xh, Wo.t(), out_dtype=torch.float32)
            y[:, self.chunk_orows[o0:o1]] = torch.mm(xh, W.t(), out_dtype=torch.float32)
        return y

    def _path(self, M: int):
        return self._gemv if M == 1 else self._multi if M <= 8 else self._tc if M <= TC_MAX else self._chunked

    def forward(self, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if x2.device != self.words.device:
            x2 = x2.to(self.words.device)
        out_dtype = x.dtype
        if x2.dtype == torch.float32 and torch.is_autocast_enabled(x2.device.type):
            ad = torch.get_autocast_dtype(x2.device.type)
            if ad in (torch.bfloat16, torch.float16):
                x2, out_dtype = x2.to(ad), ad
        M = x2.shape[0]
        if M == 0:
            return x2.new_empty(*shp[:-1], self.out_features, dtype=out_dtype)
        if TC_MAX < M <= TC_SPLIT_MAX:                   # equal tensor-core passes of <= 16 rows
            n = -(-M // TC_MAX)
            step = -(-M // n)
            y = torch.cat([self._path(min(M - i, step))(x2[i:i + step]) for i in range(0, M, step)])
        else:
            y = self._path(M)(x2)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.to(out_dtype).reshape(*shp[:-1], self.out_features)

    def dense(self, dtype=torch.bfloat16):
        """The exact weight (Q, P) in `dtype`, escapes applied: for audits, never on the product path."""
        code = {torch.float16: 0, torch.bfloat16: 1}.get(dtype, 2)
        W = ext.decode(*self._core(), self.in_features, code, 0, self.blocks8.shape[0], -1, 0)
        if self.esc_flat.numel():
            W.view(-1)[self.esc_flat] = self.esc_val.to(W.dtype)
        return W.to(dtype)
