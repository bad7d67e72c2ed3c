"""``QVBandLinearV8``: a linear layer whose weight exists on the device only as a QVB8 pack.

The class keeps the public surface of the reference module of the same name (formats/qvb8/module.py:59-464) --
``from_packfile``, ``forward``, ``row_subset``, ``escapes``, the buffer names ``ids / min_s / tau_s / nbits / bit_off /
esc_idx / esc_vals (+ _bf16)``, ``in_features / out_features / bias`` -- so code written against the reference module
keeps working; everything underneath is this library's: one :class:`DevicePack` per escape table holding the C-ABI
struct and the streaming kernel's plan, an explicit :func:`choose_route`, scratch reservation for graph capture, and a
prefill route.

Routes by the row count M of the flattened input (``choose_route``):

    ================  =====================================================================================
    M <= 48           one launch of the streaming kernel (``qvb8_small_m_ex``)
    49 <= M <= 96     two launches of it on halves of the rows (the reference does the same, module.py:381-390)
    M > 96            ``PREFILL_ROUTE``: "dense" = restore once to 16 bits + one library GEMM (the reference's
                      route); "fused" = the tcgen05 kernel that restores inside the product (``qvb8_prefill``)
    ================  =====================================================================================

Which escape table and activation mode a call uses follows the reference's contract (module.py:375-400, 455-457):
fewer than 8 rows always take the fp16 table with activations narrowed to saturated fp16; from 8 rows on, a
bf16-certified pack called with bf16 activations takes the bf16 table and keeps the activations' range (``x_mode`` 1).
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch
import torch.nn as nn

from . import lib as _lib
from . import packs

STREAM_ROWS = 48                   # rows one streaming launch takes
PREFILL_ROUTE = "dense"            # route for M > 2 * STREAM_ROWS: "dense" | "fused"
_FP32_FIELDS = ("min_s", "tau_s", "esc_vals", "esc_vals_bf16")


@dataclasses.dataclass(frozen=True)
class Route:
    kind: str                      # "stream" | "dense" | "fused"
    passes: int                    # launches of the streaming kernel
    table: str                     # escape table: "fp16" | "bf16"
    x_mode: int                    # 0 = activations narrowed to saturated fp16, 1 = their range is kept


def choose_route(M: int, x_dtype: torch.dtype, bf16_certified: bool, bf16_gemm: bool, P: int) -> Route:
    """The kernel route of one call (pure function of the call's shape and types, so tests can state it)."""
    wide = bool(bf16_certified) and x_dtype == torch.bfloat16
    if M <= 2 * STREAM_ROWS:
        keep_range = wide and M >= 8
        return Route("stream", 1 if M <= STREAM_ROWS else 2, "bf16" if keep_range else "fp16", int(keep_range))
    if wide and bf16_gemm:
        return Route("dense", 0, "bf16", 1)
    if PREFILL_ROUTE == "fused" and P % 64 == 0:
        return Route("fused", 0, "fp16", 0)
    return Route("dense", 0, "fp16", 0)


class DevicePack:
    """A pack's tensors with one escape table, as the C ABI wants them: the ``qvb8_pack`` struct, the tensors it points
    at (kept alive here) and -- when the layout allows the streaming kernel -- its plan, built on first use."""

    def __init__(self, ids, min_s, tau_s, nbits, bit_off, P: int, esc_idx, esc_vals):
        self.struct, self.keep = _lib.pack_struct(ids, min_s, tau_s, nbits, bit_off, int(P), esc_idx, esc_vals)
        self.device = ids.device
        self.streamable = ids.is_cuda and int(P) % 128 == 0 and ids.data_ptr() % 16 == 0
        self._plan = None

    @property
    def plan(self):
        if self._plan is None and self.streamable and not torch.cuda.is_current_stream_capturing():
            self._plan = _lib.build_plan(self.struct, self.keep)
        return self._plan

    def product(self, x2: torch.Tensor, x_mode: int) -> torch.Tensor:
        return _lib.small_m(self.struct, self.keep, x2, x_mode=x_mode, plan=self.plan)

    def restore(self, dtype: torch.dtype) -> torch.Tensor:
        return _lib.decode(self.struct, self.keep, dtype)

    def fused_prefill(self, x2: torch.Tensor) -> torch.Tensor:
        return _lib.prefill(self.struct, self.keep, x2, self.plan)


def _ascending(idx: torch.Tensor, vals: torch.Tensor):
    """Escape positions in ascending order (the kernels' escape pass walks them row by row)."""
    if idx.numel() > 1 and bool((idx[1:] < idx[:-1]).any()):
        order = torch.sort(idx, stable=True).indices
        return idx[order].contiguous(), vals[order].contiguous()
    return idx, vals


class QVBandLinearV8(nn.Module):
    """y = x @ W^T (+ bias), W restored inside the kernels on every call and never kept dense."""

    bf16_gemm = False             # set by enable_bf16_gemm: many-row bf16 calls restore to bf16 and run a bf16 GEMM
    bf16_certified = False        # the pack certifies |w - bf16(band)| <= tau too (restore code 3)
    fp16_table_missing = False    # a bf16-certified pack loaded without its fp16 escape table: fp16 calls are refused

    def __init__(self, *, min_s, nbits, bit_off, ids, Q, P, tau_s, esc_idx, esc_vals, bias=None, esc_idx_bf16=None,
                 esc_vals_bf16=None):
        super().__init__()
        self.in_features, self.out_features = int(P), int(Q)
        esc_idx, esc_vals = _ascending(esc_idx, esc_vals)
        shared_table = esc_idx_bf16 is None
        if shared_table:
            esc_idx_bf16, esc_vals_bf16 = esc_idx, esc_vals
        else:
            esc_idx_bf16, esc_vals_bf16 = _ascending(esc_idx_bf16, esc_vals_bf16)
        tensors = dict(ids=ids, nbits=nbits, bit_off=bit_off, esc_idx=esc_idx, esc_idx_bf16=esc_idx_bf16, min_s=min_s,
                       tau_s=tau_s, esc_vals=esc_vals, esc_vals_bf16=esc_vals_bf16)
        for name, t in tensors.items():
            self.register_buffer(name, t, persistent=False)
        self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None
        self._where = type(self).__name__
        self._packs: dict[str, DevicePack] = {}

    # ---- construction -----------------------------------------------------------------------------------
    @classmethod
    def from_parsed(cls, d: dict, *, bias=None, device="cuda", where: str | None = None) -> "QVBandLinearV8":
        """From the dict :func:`qvb8_b200.packs.read_qvb8` returns (bounds re-checked before anything is uploaded)."""
        packs.validate_pack(d, where or "parsed pack")
        dev = torch.device(device)

        def up(key, dt):
            return torch.from_numpy(np.ascontiguousarray(d[key], dtype=dt)).to(dev)
        two_tables = d["esc_idx_bf16"] is not d["esc_idx"]
        if bias is not None:
            bias = torch.as_tensor(bias).detach().to(dev)
        mod = cls(min_s=up("min_s", np.float32), nbits=up("nbits", np.uint8), bit_off=up("bit_off", np.int64),
                  ids=up("ids", np.uint8), Q=d["Q"], P=d["P"], tau_s=up("tau_s", np.float32),
                  esc_idx=up("esc_idx", np.int64), esc_vals=up("esc_vals", np.float32), bias=bias,
                  esc_idx_bf16=up("esc_idx_bf16", np.int64) if two_tables else None,
                  esc_vals_bf16=up("esc_vals_bf16", np.float32) if two_tables else None)
        mod.bf16_certified = d.get("restore") == "fp16+bf16"
        mod.fp16_table_missing = bool(d.get("fp16_table_missing", False))
        if where:
            mod._where = where
        return mod

    @classmethod
    def from_packfile(cls, path: str | None, *, bias=None, tau: float | None = None, device: str = "cuda",
                      blob: bytes | None = None) -> "QVBandLinearV8":
        """The loader's entry point (reference run/run_inference.py:784-819 calls it with these keywords).  `tau` is
        accepted and unused: the file states its own."""
        if blob is None:
            with open(path, "rb") as fh:
                blob = fh.read()
        return cls.from_parsed(packs.read_qvb8(blob, path), bias=bias, device=device, where=str(path) if path else None)

    @classmethod
    def from_pack(cls, pk, *, bias=None) -> "QVBandLinearV8":
        """From an in-memory :class:`qvb8_b200.synth.QVB8Pack`; its tensors are shared, not copied."""
        two_tables = pk.esc_idx_bf16 is not pk.esc_idx
        mod = cls(min_s=pk.min_s, nbits=pk.nbits, bit_off=pk.bit_off, ids=pk.ids, Q=pk.Q, P=pk.P, tau_s=pk.tau_s,
                  esc_idx=pk.esc_idx, esc_vals=pk.esc_vals, bias=bias,
                  esc_idx_bf16=pk.esc_idx_bf16 if two_tables else None,
                  esc_vals_bf16=pk.esc_vals_bf16 if two_tables else None)
        mod.bf16_certified = pk.restore == "fp16+bf16"
        return mod

    def row_subset(self, rows: torch.Tensor) -> "QVBandLinearV8":
        """A layer over the output rows `rows` (in that order) that shares this layer's packed ids: a row of a pack is
        self-contained (own origin, step, width and bit offset), so a subset is four gathers and a renumbering of the
        escapes -- no bytes of the payload are copied (the reference offers the same, module.py:126-160)."""
        dev = self.ids.device
        rows = rows.to(device=dev, dtype=torch.int64)
        P = self.in_features
        new_row_of = torch.full((self.out_features,), -1, dtype=torch.int64, device=dev)
        new_row_of[rows] = torch.arange(rows.numel(), dtype=torch.int64, device=dev)

        def renumber(idx, vals):
            if idx.numel() == 0:
                return idx, vals
            target = new_row_of[torch.div(idx, P, rounding_mode="floor")]
            kept = target >= 0
            return _ascending(target[kept] * P + torch.remainder(idx[kept], P), vals[kept])
        ei, ev = renumber(self.esc_idx, self.esc_vals)
        two_tables = self.esc_idx_bf16 is not self.esc_idx
        eib, evb = renumber(self.esc_idx_bf16, self.esc_vals_bf16) if two_tables else (None, None)
        sub = type(self)(min_s=self.min_s[rows], nbits=self.nbits[rows], bit_off=self.bit_off[rows], ids=self.ids,
                         Q=int(rows.numel()), P=P, tau_s=self.tau_s[rows], esc_idx=ei, esc_vals=ev,
                         esc_idx_bf16=eib, esc_vals_bf16=evb)
        sub.bf16_certified, sub.fp16_table_missing, sub.bf16_gemm = self.bf16_certified, self.fp16_table_missing, self.bf16_gemm
        return sub

    def escapes(self, dtype=torch.float16):
        """(positions, values) of the escape table that goes with a restore rounded to `dtype`."""
        if dtype == torch.bfloat16:
            return self.esc_idx_bf16, self.esc_vals_bf16
        if dtype == torch.float16 and self.fp16_table_missing:
            raise packs.EscapeTableError(f"{self._where}: this pack is certified for fp16 and bf16 and was loaded without "
                                         f"{packs.ESCAPE_TABLES_FILE}, which holds its fp16 escape table; fp16 runs need it")
        return self.esc_idx, self.esc_vals

    def _apply(self, fn, recurse=True):
        """``.to()`` / ``.half()`` / ``.bfloat16()``: the origins, steps and escape values are fp32 data of the format,
        not parameters of the model -- a dtype cast must not touch them; they follow the ids to a new device."""
        held = {n: self._buffers.pop(n) for n in _FP32_FIELDS}
        try:
            super()._apply(fn, recurse)
        finally:
            dev = self._buffers["ids"].device
            for n, t in held.items():
                self._buffers[n] = t if t.device == dev else t.to(dev)
            self._packs = {}
        return self

    # ---- kernels ----------------------------------------------------------------------------------------
    def device_pack(self, table: str = "fp16") -> DevicePack:
        """The :class:`DevicePack` of one escape table ("fp16" | "bf16"), made once per table and device."""
        dp = self._packs.get(table)
        if dp is None or dp.device != self.ids.device:
            idx, vals = (self.esc_idx_bf16, self.esc_vals_bf16) if table == "bf16" else (self.esc_idx, self.esc_vals)
            dp = self._packs[table] = DevicePack(self.ids, self.min_s, self.tau_s, self.nbits, self.bit_off,
                                                 self.in_features, idx, vals)
        return dp

    def dense(self, dtype=torch.float16) -> torch.Tensor:
        """(Q, P) weight rounded once to `dtype`, the matching escape table written over."""
        self.escapes(dtype)                                             # refuses an fp16 restore without its table
        return self.device_pack("bf16" if dtype == torch.bfloat16 else "fp16").restore(dtype)

    def reserve(self, max_rows: int = STREAM_ROWS) -> None:
        """Everything a later call would otherwise create on first use -- plans and the streaming kernel's scratch for
        up to `max_rows` rows -- so that calls can be captured into a CUDA graph."""
        for table in ("fp16", "bf16") if self.bf16_certified else ("fp16",):
            _ = self.device_pack(table).plan
        rows = sorted({1, 2, 4, 8, 16, 32, min(int(max_rows), STREAM_ROWS)})
        for m in rows:
            if m <= max_rows:
                _lib.reserve_scratch(self.ids.device, m, self.out_features, self.in_features)

    def route_for(self, M: int, x_dtype: torch.dtype) -> Route:
        return choose_route(M, x_dtype, self.bf16_certified, self.bf16_gemm, self.in_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).to(self.ids.device)
        result_dtype = x.dtype
        if x2.dtype == torch.float32 and torch.is_autocast_enabled(x2.device.type):
            cast_to = torch.get_autocast_dtype(x2.device.type)          # behave like nn.Linear under autocast
            if cast_to in (torch.float16, torch.bfloat16):
                x2, result_dtype = x2.to(cast_to), cast_to
        if x2.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x2 = x2.float()
        M = x2.shape[0]
        if M == 0:
            return torch.empty(*lead, self.out_features, dtype=result_dtype, device=x2.device)
        if x2.dtype == torch.float16:
            self.escapes(torch.float16)
        route = self.route_for(M, x2.dtype)
        if route.kind == "stream":
            dp = self.device_pack(route.table)
            if route.passes == 1:
                y = dp.product(x2, route.x_mode)
            else:
                half = (M + 1) // 2
                y = torch.cat([dp.product(x2[:half], route.x_mode), dp.product(x2[half:], route.x_mode)])
        elif route.kind == "fused":
            y = self.device_pack(route.table).fused_prefill(x2)
        elif route.table == "bf16":
            y = torch.mm(x2, self.dense(torch.bfloat16).t())
        else:
            xh = x2 if x2.dtype == torch.float16 else x2.float().clamp(-65504.0, 65504.0).to(torch.float16)
            y = torch.mm(xh, self.dense(torch.float16).t(), out_dtype=torch.float32)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.to(result_dtype).reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"restore={'fp16+bf16' if self.bf16_certified else 'fp16'}")


def enable_bf16_gemm(model: nn.Module) -> tuple[int, int]:
    """Turns the bf16 GEMM route on for every bf16-certified packed linear under `model` (what the reference's loader
    does after loading, module.py:506-524).  Returns (layers switched, packed layers seen)."""
    layers = [m for m in model.modules() if isinstance(m, QVBandLinearV8)]
    switched = 0
    for layer in layers:
        if layer.bf16_certified:
            layer.bf16_gemm = True
            switched += 1
    return switched, len(layers)


def footprint_report(module: nn.Module) -> dict:
    """Device bytes of the packed linears under `module`, by kind, and bytes per weight (the reference prints the same
    summary at load, module.py:527-587)."""
    tally = dict(linears=0, params=0, escape_count=0, ids_bytes=0, escape_bytes=0, meta_bytes=0)
    size = lambda t: t.numel() * t.element_size()
    for layer in module.modules():
        if not isinstance(layer, QVBandLinearV8):
            continue
        tally["linears"] += 1
        tally["params"] += layer.in_features * layer.out_features
        tally["ids_bytes"] += size(layer.ids)
        tally["meta_bytes"] += size(layer.min_s) + size(layer.tau_s) + size(layer.nbits) + size(layer.bit_off)
        tables = [(layer.esc_idx, layer.esc_vals)]
        if layer.esc_idx_bf16.data_ptr() != layer.esc_idx.data_ptr():
            tables.append((layer.esc_idx_bf16, layer.esc_vals_bf16))
        for idx, vals in tables:
            tally["escape_count"] += idx.numel()
            tally["escape_bytes"] += size(idx) + size(vals)
    total = tally["ids_bytes"] + tally["escape_bytes"] + tally["meta_bytes"]
    n = tally["params"]
    tally.update(total_bytes=total, bytes_per_param=total / n if n else 0.0,
                 escape_ratio=tally["escape_count"] / n if n else 0.0)
    return tally
