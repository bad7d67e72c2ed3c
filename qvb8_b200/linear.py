"""``QVBandLinearV8``: an ``nn.Linear`` replacement whose weight lives in device memory only as a QVB8 pack.

Mirrors the reference module of the same name (formats/qvb8/module.py:59-464): same constructor keywords, buffers,
``from_packfile``, ``row_subset``, ``escapes`` and ``forward`` contract -- y = x @ W^T (+ bias), W restored inside the
kernel on every call and never cached dense.  Dispatch by row count M of the flattened input:

    M <= 48      one fused decode-in-matmul launch (fp32 band value x saturated-fp16 activation, fp32 result)
    M  > 48      restore once to fp16 (bf16 when the pack is bf16-certified, ``bf16_gemm`` is on and x is bf16)
                 and run one tensor-core GEMM

The reference splits 49..96 rows into two <=48-row passes before falling back to the dense route
(module.py:381-390); the same is done here.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import lib as _lib
from . import packs

FP32_METADATA = ("min_s", "tau_s", "esc_vals", "esc_vals_bf16")
SMALL_M_MAX = 48
SMALL_M_SPLIT_MAX = 2 * SMALL_M_MAX


class QVBandLinearV8(nn.Module):
    bf16_gemm = False             # opt-in per module (enable_bf16_gemm): bf16 callers with many rows use a bf16 GEMM
    bf16_certified = False        # the pack certifies |w - bf16(band)| <= tau (header restore code 3)
    fp16_table_missing = False    # fp16+bf16 pack loaded without escape_tables.json: fp16 calls are refused

    def __init__(self, *, min_s, nbits, bit_off, ids, Q, P, tau_s, esc_idx, esc_vals, bias=None, esc_idx_bf16=None,
                 esc_vals_bf16=None):
        super().__init__()
        self.in_features, self.out_features = int(P), int(Q)

        def _sorted(ei, ev):
            if ei.numel() > 1 and not bool((ei[1:] >= ei[:-1]).all()):
                o = torch.argsort(ei, stable=True)
                ei, ev = ei[o].contiguous(), ev[o].contiguous()
            return ei, ev
        esc_idx, esc_vals = _sorted(esc_idx, esc_vals)       # the escape correction relies on ascending positions
        if esc_idx_bf16 is None:
            esc_idx_bf16, esc_vals_bf16 = esc_idx, esc_vals
        else:
            esc_idx_bf16, esc_vals_bf16 = _sorted(esc_idx_bf16, esc_vals_bf16)
        for name, t in (("tau_s", tau_s), ("min_s", min_s), ("nbits", nbits), ("bit_off", bit_off), ("ids", ids),
                        ("esc_idx", esc_idx), ("esc_vals", esc_vals), ("esc_idx_bf16", esc_idx_bf16),
                        ("esc_vals_bf16", esc_vals_bf16)):
            self.register_buffer(name, t, persistent=False)
        self.bias = None if bias is None else nn.Parameter(bias, requires_grad=False)
        self._where = "QVBandLinearV8"

    # ---- construction -----------------------------------------------------------------------------------
    @classmethod
    def from_packfile(cls, path: str | None, *, bias=None, tau: float | None = None, device: str = "cuda",
                      blob: bytes | None = None) -> "QVBandLinearV8":
        """`tau` is accepted for call-site compatibility and ignored: the pack carries its own."""
        if blob is None:
            with open(path, "rb") as fh:
                blob = fh.read()
        d = packs.read_qvb8(blob, path)
        return cls.from_parsed(d, bias=bias, device=device, where=str(path))

    @classmethod
    def from_parsed(cls, d: dict, *, bias=None, device="cuda", where: str = "QVBandLinearV8") -> "QVBandLinearV8":
        dev = torch.device(device)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(dev)
        same = d["esc_idx_bf16"] is d["esc_idx"]
        b = None
        if bias is not None:
            b = (bias.detach() if isinstance(bias, torch.Tensor) else torch.tensor(bias)).to(dev)
        mod = cls(min_s=t(d["min_s"], np.float32), nbits=t(d["nbits"], np.uint8), bit_off=t(d["bit_off"], np.int64),
                  ids=t(d["ids"], np.uint8), Q=d["Q"], P=d["P"], tau_s=t(d["tau_s"], np.float32),
                  esc_idx=t(d["esc_idx"], np.int64), esc_vals=t(d["esc_vals"], np.float32), bias=b,
                  esc_idx_bf16=None if same else t(d["esc_idx_bf16"], np.int64),
                  esc_vals_bf16=None if same else t(d["esc_vals_bf16"], np.float32))
        mod.bf16_certified = d.get("restore") == "fp16+bf16"
        mod.fp16_table_missing = bool(d.get("fp16_table_missing", False))
        mod._where = where
        return mod

    @classmethod
    def from_pack(cls, pk, *, bias=None) -> "QVBandLinearV8":
        """From an in-memory :class:`qvb8_b200.synth.QVB8Pack` (tensors are shared, not copied)."""
        same = pk.esc_idx_bf16 is pk.esc_idx
        mod = cls(min_s=pk.min_s, nbits=pk.nbits, bit_off=pk.bit_off, ids=pk.ids, Q=pk.Q, P=pk.P, tau_s=pk.tau_s,
                  esc_idx=pk.esc_idx, esc_vals=pk.esc_vals, bias=bias,
                  esc_idx_bf16=None if same else pk.esc_idx_bf16, esc_vals_bf16=None if same else pk.esc_vals_bf16)
        mod.bf16_certified = pk.restore == "fp16+bf16"
        return mod

    def row_subset(self, rows: torch.Tensor) -> "QVBandLinearV8":
        """A linear over output rows `rows` only, sharing this module's packed ids (rows of a pack are independent:
        only the four per-row vectors are sliced and the escapes renumbered)."""
        rows = rows.to(self.min_s.device).long()
        P = self.in_features
        remap = torch.full((self.out_features,), -1, dtype=torch.long, device=rows.device)
        remap[rows] = torch.arange(rows.numel(), device=rows.device)

        def sub(ei, ev):
            if not ei.numel():
                return ei, ev
            q = ei // P
            keep = remap[q] >= 0
            return remap[q[keep]] * P + ei[keep] % P, ev[keep]
        ei, ev = sub(self.esc_idx, self.esc_vals)
        same = self.esc_idx_bf16 is self.esc_idx
        eib, evb = (None, None) if same else sub(self.esc_idx_bf16, self.esc_vals_bf16)
        m = type(self)(min_s=self.min_s[rows], nbits=self.nbits[rows], bit_off=self.bit_off[rows], ids=self.ids,
                       Q=int(rows.numel()), P=P, tau_s=self.tau_s[rows], esc_idx=ei, esc_vals=ev, bias=None,
                       esc_idx_bf16=eib, esc_vals_bf16=evb)
        m.bf16_certified, m.fp16_table_missing = self.bf16_certified, self.fp16_table_missing
        return m

    def escapes(self, dtype=torch.float16):
        """(esc_idx, esc_vals) for a restore that rounds the weight to `dtype`: the bf16 table for bf16, else fp16."""
        if dtype == torch.bfloat16:
            return self.esc_idx_bf16, self.esc_vals_bf16
        if dtype == torch.float16 and self.fp16_table_missing:
            raise packs.EscapeTableError(f"{self._where}: fp16 run on an fp16+bf16 pack without "
                                         f"{packs.ESCAPE_TABLES_FILE}")
        return self.esc_idx, self.esc_vals

    def _apply(self, fn, recurse=True):
        # module.to(dtype) must never narrow the fp32 decode metadata: only the device follows
        keep = {n: self._buffers[n] for n in FP32_METADATA if self._buffers.get(n) is not None}
        for n in keep:
            self._buffers[n] = None
        try:
            out = super()._apply(fn, recurse)
        finally:
            ref = self._buffers.get("ids")
            for n, b in keep.items():
                self._buffers[n] = b.to(ref.device) if ref is not None else b
        self.__dict__.pop("_pack_cache", None)
        return out

    # ---- kernels ----------------------------------------------------------------------------------------
    def _pack(self, table: str = "fp16"):
        cache = self.__dict__.setdefault("_pack_cache", {})
        key = (table, self.ids.data_ptr())
        hit = cache.get(key)
        if hit is None:
            ei, ev = (self.esc_idx_bf16, self.esc_vals_bf16) if table == "bf16" else (self.esc_idx, self.esc_vals)
            st, keep = _lib.pack_struct(self.ids, self.min_s, self.tau_s, self.nbits, self.bit_off, self.in_features,
                                        ei, ev)
            plan = None
            if self.ids.is_cuda and self.in_features % 128 == 0 and self.ids.data_ptr() % 16 == 0 \
                    and not torch.cuda.is_current_stream_capturing():
                plan = _lib.build_plan(st, keep)       # once per weight (and escape table), like the reference's _mma_order
            hit = cache[key] = (st, keep, plan)
        return hit

    def dense(self, dtype=torch.float16) -> torch.Tensor:
        """(Q, P) restored weight rounded once to `dtype`, escapes of the matching table applied."""
        self.escapes(dtype)
        pk, keep, _ = self._pack("bf16" if dtype == torch.bfloat16 else "fp16")
        return _lib.decode(pk, keep, dtype)

    def reserve(self, max_rows: int = SMALL_M_MAX) -> None:
        """Pre-allocate the scratch the fused kernel needs for up to `max_rows` rows (before graph capture)."""
        self._pack("fp16")
        if self.bf16_certified:
            self._pack("bf16")
        for m in {1, 2, 4, 8, 16, min(max_rows, SMALL_M_MAX)}:
            if m <= max_rows:
                _lib.reserve_scratch(self.ids.device, m, self.out_features, self.in_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        orig = x.shape
        x2 = x.reshape(-1, orig[-1])
        if x2.device != self.min_s.device:
            x2 = x2.to(self.min_s.device)
        out_dtype = x.dtype
        if x2.dtype == torch.float32 and torch.is_autocast_enabled(x2.device.type):     # honour autocast like nn.Linear
            ad = torch.get_autocast_dtype(x2.device.type)
            if ad in (torch.bfloat16, torch.float16):
                x2, out_dtype = x2.to(ad), ad
        M = x2.shape[0]
        if M == 0:
            return x2.new_empty(*orig[:-1], self.out_features, dtype=out_dtype)
        if self.fp16_table_missing and x2.dtype == torch.float16:
            self.escapes(torch.float16)
        if x2.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x2 = x2.float()
        bf16_mode = bool(self.bf16_certified) and x2.dtype == torch.bfloat16
        if M <= SMALL_M_SPLIT_MAX:
            pk, keep, plan = self._pack("bf16" if bf16_mode else "fp16")
            if M <= SMALL_M_MAX:
                y = _lib.small_m(pk, keep, x2, x_mode=1 if bf16_mode else 0, plan=plan)
            else:
                step = -(-M // 2)
                y = torch.cat([_lib.small_m(pk, keep, x2[i:i + step], x_mode=1 if bf16_mode else 0, plan=plan)
                               for i in range(0, M, step)])
        elif bf16_mode and self.bf16_gemm:
            b = None if self.bias is None else self.bias.to(torch.bfloat16)
            return F.linear(x2, self.dense(torch.bfloat16), b).reshape(*orig[:-1], self.out_features)
        else:
            W = self.dense(torch.float16)
            xh = x2 if x2.dtype == torch.float16 else x2.float().clamp(-65504.0, 65504.0).to(torch.float16)
            if x2.dtype == torch.float16:
                b = None if self.bias is None else self.bias.to(torch.float16)
                return F.linear(xh, W, b).reshape(*orig[:-1], self.out_features)
            y = torch.mm(xh, W.t(), out_dtype=torch.float32)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.to(out_dtype).reshape(*orig[:-1], self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


def enable_bf16_gemm(model: nn.Module) -> tuple[int, int]:
    """Switch every bf16-certified packed linear of `model` to the bf16 GEMM for many-row bf16 inputs
    (reference module.py:506-524).  Returns (switched, packed linears)."""
    n = tot = 0
    for m in model.modules():
        if isinstance(m, QVBandLinearV8):
            tot += 1
            if m.bf16_certified:
                m.bf16_gemm = True
                n += 1
    return n, tot


def footprint_report(module: nn.Module) -> dict:
    """Resident bytes of the packed linears of `module` (ids / escapes / row metadata) and bytes per parameter
    (reference module.py:527-587)."""
    ids = esc = meta = n_esc = n_par = n_lin = 0
    for m in module.modules():
        if not isinstance(m, QVBandLinearV8):
            continue
        n_lin += 1
        n_par += m.out_features * m.in_features
        ids += m.ids.numel()
        tabs = [m.esc_idx, m.esc_vals]
        if m.esc_idx_bf16.data_ptr() != m.esc_idx.data_ptr():
            tabs += [m.esc_idx_bf16, m.esc_vals_bf16]
        for t in tabs:
            n_esc += t.numel() if t.dtype == torch.int64 else 0
            esc += t.numel() * t.element_size()
        meta += sum(t.numel() * t.element_size() for t in (m.min_s, m.tau_s, m.nbits, m.bit_off))
    total = ids + esc + meta
    return dict(linears=n_lin, params=n_par, escape_count=n_esc, ids_bytes=ids, escape_bytes=esc, meta_bytes=meta,
                total_bytes=total, bytes_per_param=total / n_par if n_par else 0.0,
                escape_ratio=n_esc / n_par if n_par else 0.0)
