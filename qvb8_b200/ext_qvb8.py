"""Drop-in object for the reference's ``qvb8_cuda`` extension module.

The reference fetches its kernels through ``_load_ext()`` (formats/qvb8/module.py:20-36) and calls the attributes
listed at formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu:2673-2691.  :data:`ext` exposes the same names, argument
order, dtypes, return shapes and error type (``RuntimeError``), backed by the sm_100a kernels of this package.
:func:`install` rebinds the reference's loaders to it, so ``QVBandLinearV8``, ``QVBandExpertsV8`` and the
format registry run unchanged on top.

Numerics shared by every small-M entry point here: the weight is the un-narrowed fp32 band value
``fma(id, tau_s, min_s)`` (the contract of the reference's M <= 8 GEMV); X is narrowed to saturated fp16 first.
The reference's 9..48-row kernels round the weight once to fp16 (or bf16) instead; the results agree within the
1e-2 relative-Frobenius tolerance the parity tests state, and the un-narrowed value is at least as close to the
certified weight.
"""
from __future__ import annotations

import os

import torch

from . import lib as _lib

_SMALL_M_MAX = 48
# Many rows (M > 48): "dense" = restore once to fp16 and run a library GEMM, the reference's own route
# (qvb8_cuda.cu:1542-1671) and today the faster of the two for thousands of rows (1.10 ms against 1.74 ms on the
# 27B-class MLP projections at 2048 rows); "fused" = the tcgen05 kernel that restores the weights inside the product
# and never writes a dense copy.  The faster route is the default; QVB8_PREFILL=fused selects the other.
PREFILL_PATH = os.environ.get("QVB8_PREFILL", "dense")


def _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
    return _lib.pack_struct(ids, min_s, tau_s, row_nbits, row_bit_off, int(P), esc_idx, esc_vals)


def _small_m(ids, pk, keep, X, x_mode=0):
    """The streaming kernel needs the pack's plan (row ordering + regrouped escapes).  The reference keeps such
    per-weight metadata on the module (formats/qvb8/module.py:267-276); this extension object has no module to hold
    it, so it is cached on the `ids` tensor object the module owns, built on first use."""
    if int(pk.P) % 128 == 0 and ids.data_ptr() % 16 == 0 and not torch.cuda.is_current_stream_capturing():
        return _lib.small_m(pk, keep, X, x_mode=x_mode, plan=_lib.plan_on(ids, pk, keep))
    plans = getattr(ids, "_qvb8_plans", None)
    if plans:                                             # capturing: use a plan only if one already exists
        key = (pk.ids, pk.Q, pk.P, pk.n_esc, pk.esc_idx, pk.min_s, pk.bit_off)
        if key in plans:
            return _lib.small_m(pk, keep, X, x_mode=x_mode, plan=plans[key])
    return _lib.small_m(pk, keep, X, x_mode=x_mode)


def _existing_or_new_plan(ids, pk, keep):
    """The pack's plan; while a CUDA graph is being captured only one that already exists (building allocates and
    launches outside the capture's intent), else None."""
    if not torch.cuda.is_current_stream_capturing():
        return _lib.plan_on(ids, pk, keep)
    plans = getattr(ids, "_qvb8_plans", None) or {}
    return plans.get((pk.ids, pk.Q, pk.P, pk.n_esc, pk.esc_idx, pk.min_s, pk.bit_off))


def _as_2d(X: torch.Tensor, P: int) -> torch.Tensor:
    if X.dim() == 1:
        X = X.reshape(1, -1)
    if X.dim() != 2 or X.shape[1] != P:
        raise RuntimeError(f"qvb8: X must be (M, {P}), got {tuple(X.shape)}")
    if X.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        X = X.float()
    return X


def _sat_half(X: torch.Tensor) -> torch.Tensor:
    """Saturating narrowing to fp16 (reference qvb8_cuda.cu:761-841): +-65504 clamp, NaN kept."""
    if X.dtype == torch.float16:
        return X
    return X.float().clamp(-65504.0, 65504.0).to(torch.float16)


class Qvb8Ext:
    """Same attribute surface as the reference's ``qvb8_cuda`` pybind module."""

    # ---- dense restore ------------------------------------------------------------------------------------
    def decode(self, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """(Q, P) fp16 restore: fp16(fma(id, tau_s, min_s)), escapes written over (qvb8_cuda.cu:651-699)."""
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _lib.decode(pk, keep, torch.float16)

    def decode_bf16(self, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """(Q, P) bf16 restore, one rounding of the fp32 band value (qvb8_cuda.cu:1711-1727)."""
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _lib.decode(pk, keep, torch.bfloat16)

    def decode_f32(self, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """(Q, P) fp32 band values with exact escapes (no counterpart entry point in the reference: its fp32 value
        lives only inside the GEMV, qvb8_cuda.cu:346-353)."""
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _lib.decode(pk, keep, torch.float32)

    # ---- small M ------------------------------------------------------------------------------------------
    def gemv(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """M = 1: X fp16 of length P -> (1, Q) fp32 (qvb8_cuda.cu:1416-1512)."""
        if X.dtype != torch.float16:
            raise RuntimeError("X must be fp16")
        if X.numel() != P:
            raise RuntimeError("X length must equal P")
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _small_m(ids, pk, keep, X.reshape(1, -1))

    def gemv_multi(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """M = 1..8 -> (M, Q) fp32 (qvb8_cuda.cu:1059-1166)."""
        X = _as_2d(X, int(P))
        if not 1 <= X.shape[0] <= 8:
            raise RuntimeError(f"qvb8 GEMV-multi: M={X.shape[0]} is outside the range 1..8")
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _small_m(ids, pk, keep, X)

    def gemv_rb(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals, perm, tile_nb):
        """The reference's register-blocked sm_70 variant (qvb8_cuda.cu:1350-1413); same result as gemv_multi.
        perm / tile_nb are accepted and not needed: the pack's plan holds this library's own row ordering."""
        return self.gemv_multi(X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)

    def mma_multi(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals, perm, tile_nb,
                  bf16=False, esc_starts=None, general=-1):
        """QVB8 tensor-core multi-row product (M<=48) -> (M, Q) fp32; accepts the bf16 mode flag.

        (qvb8_cuda.cu:2566-2671.)  perm, tile_nb, esc_starts and general describe a row ordering the reference
        computes per module; this library keeps its own ordering in the pack's plan, so they are validated and unused.
        bf16=True keeps X's range (no fp16 clamp)."""
        X = _as_2d(X, int(P))
        M = X.shape[0]
        if not 1 <= M <= _SMALL_M_MAX:
            raise RuntimeError(f"qvb8 mma-multi: M={M} outside 1..48")
        if int(P) % 128 != 0 or ids.data_ptr() % 4 != 0:
            raise RuntimeError("qvb8 mma-multi: needs P%128==0 and 4-byte-aligned ids")
        Q = min_s.numel()
        if perm is not None and perm.numel() not in (0, Q):
            raise RuntimeError("qvb8 mma-multi: perm must be an int32 CUDA tensor of length Q (or empty)")
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        return _small_m(ids, pk, keep, X, x_mode=1 if bf16 else 0)

    # ---- any M --------------------------------------------------------------------------------------------
    def _forward(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals, out_half: bool):
        X = _as_2d(X, int(P))
        M = X.shape[0]
        pk, keep = _pack(ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals)
        if M <= _SMALL_M_MAX:
            y = _small_m(ids, pk, keep, X)
            return y.to(torch.float16) if (out_half and M > 8) else y
        if int(P) % 64 == 0 and PREFILL_PATH == "fused":
            # prefill: the ids are unpacked into tensor memory and contracted by tcgen05.mma, no dense copy of W
            plan = _existing_or_new_plan(ids, pk, keep)
            if plan is not None:
                y = _lib.prefill(pk, keep, X, plan)
                return y.to(torch.float16) if out_half else y
        # other shapes: restore once to fp16, then one library GEMM with fp32 accumulation (qvb8_cuda.cu:1542-1671)
        W = _lib.decode(pk, keep, torch.float16)
        Xh = _sat_half(X)
        if out_half:
            return torch.mm(Xh, W.t())
        return torch.mm(Xh, W.t(), out_dtype=torch.float32)

    def forward(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """Any M -> (M, Q) fp32 (qvb8_cuda.cu:1520-1683)."""
        return self._forward(X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals, False)

    def forward_half(self, X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals):
        """As forward, but the M > 8 result is fp16 (qvb8_cuda.cu:1685-1697)."""
        return self._forward(X, ids, min_s, row_nbits, row_bit_off, P, tau_s, esc_idx, esc_vals, True)


    # ---- mixture of experts ---------------------------------------------------------------------------------
    def moe_experts(self, X, idx, w, gu_ids, gu_min, gu_tau, gu_nb, gu_off, Qgu, Pgu,
                    dn_ids, dn_min, dn_tau, dn_nb, dn_off, Qdn, Pdn):
        """Gated-SiLU expert MLP over stacked packs -> (M, Qdn) in X.dtype (qvb8_cuda.cu:949-992)."""
        if X.dim() != 2 or X.shape[1] != Pgu:
            raise RuntimeError("moe: bad X")
        if Qgu % 2 != 0 or Qgu // 2 != Pdn:
            raise RuntimeError("moe: gate_up/down shapes disagree")
        if Pgu % 8 != 0 or Pdn % 8 != 0:
            raise RuntimeError("moe: P must be a multiple of 8")
        up = _lib.expert_stack_struct(gu_ids, gu_min, gu_tau, gu_nb, gu_off, Qgu, Pgu)
        dn = _lib.expert_stack_struct(dn_ids, dn_min, dn_tau, dn_nb, dn_off, Qdn, Pdn)
        return _lib.moe_experts(X, idx, w, up, dn, 0)

    def moe_experts_relu2(self, X, idx, w, up_ids, up_min, up_tau, up_nb, up_off, Qup, Pup,
                          dn_ids, dn_min, dn_tau, dn_nb, dn_off, Qdn, Pdn):
        """Non-gated expert MLP, H = relu(up(x))^2 -> (M, Qdn) in X.dtype (qvb8_cuda.cu:1002-1058)."""
        if X.dim() != 2 or X.shape[1] != Pup:
            raise RuntimeError("moe_relu2: bad X")
        if Qup != Pdn:
            raise RuntimeError("moe_relu2: up/down shapes disagree")
        if Pup % 8 != 0 or Pdn % 8 != 0:
            raise RuntimeError("moe_relu2: P must be a multiple of 8")
        up = _lib.expert_stack_struct(up_ids, up_min, up_tau, up_nb, up_off, Qup, Pup)
        dn = _lib.expert_stack_struct(dn_ids, dn_min, dn_tau, dn_nb, dn_off, Qdn, Pdn)
        return _lib.moe_experts(X, idx, w, up, dn, 1)


ext = Qvb8Ext()


def install() -> None:
    """Make the reference's QVB8 modules use this package's kernels: rebinds ``_load_ext`` in every reference module
    that imported it (formats/qvb8/module.py:20, backends_experts.py:13).  The reference package must be importable
    (it is not a dependency of this package)."""
    import importlib
    for name in ("qv_band.formats.qvb8.module", "qv_band.formats.qvb8.backends_experts"):
        mod = importlib.import_module(name)
        mod._load_ext = lambda: ext
