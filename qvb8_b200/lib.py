"""ctypes binding of ``libqvb8_b200.so`` (the C ABI declared in ``include/qvb8_b200.h``).

The library is the product: there is no fallback.  :func:`load` raises if it has not been built
(``python -m qvb8_b200.build``), and every wrapper raises ``RuntimeError`` with the library's own message on a
non-zero status.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqvb8_b200.so")

F16, BF16, F32 = 0, 1, 2
_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}

# every symbol include/qvb8_b200.h declares
EXPORTS = (
    "qvb8_last_error", "qvb8_version", "qvb8_decode", "qvb8_small_m_scratch_bytes", "qvb8_small_m",
    "qvb8_small_m_generic", "qvb8_plan_bytes", "qvb8_plan_build", "qvb8_small_m_ex", "qvb8_small_m_set_tuning",
    "qvb8_device_status", "qvb8_debug_trace", "qvb8_small_m_static_max_scratch", "qvb8_small_m_static",
    "qvb8_moe_scratch_bytes", "qvb8_moe_experts", "qvb8_moe_bad_index", "qvb8_moe_plan_bytes", "qvb8_moe_plan_build",
    "qvb8_moe_experts_planned", "qvb8_moe_streams", "qvb8_argmax_scratch_bytes", "qvb8_argmax_rows", "qvb8_small_m_group_describe",
    "qvb8r_ids", "qvb8r_decode", "qvb8r_small_m", "qvb8r_fix_escapes", "qvb8_prefill_scratch_bytes", "qvb8_prefill", "qvb8_prefill_set_tuning",
    "qvb8_embed_rows", "qvb8_peer_bytes", "qvb8_peer_alloc", "qvb8_peer_open", "qvb8_peer_close", "qvb8_peer_allreduce",
    "qvb8_peer_allreduce_ex", "qvb8_peer_allreduce_local", "qvb8_peer_allgather", "qvb8_peer_allgather_local", "qvb8_device_status_reset", "qvb8r_embed_rows",
    "qvb8_small_m_group_scratch_bytes", "qvb8_small_m_group",
)


class PackStruct(ctypes.Structure):
    """``struct qvb8_pack`` of the header."""
    _fields_ = [
        ("ids", ctypes.c_void_p), ("ids_bytes", ctypes.c_int64), ("min_s", ctypes.c_void_p),
        ("tau_s", ctypes.c_void_p), ("nbits", ctypes.c_void_p), ("bit_off", ctypes.c_void_p),
        ("Q", ctypes.c_int64), ("P", ctypes.c_int64), ("esc_idx", ctypes.c_void_p), ("esc_vals", ctypes.c_void_p),
        ("n_esc", ctypes.c_int64),
    ]


class JobStruct(ctypes.Structure):
    """``struct qvb8_job`` of the header."""
    _fields_ = [("w", ctypes.POINTER(PackStruct)), ("plan", ctypes.c_void_p), ("X", ctypes.c_void_p),
                ("Y", ctypes.c_void_p), ("x_dtype", ctypes.c_int), ("x_mode", ctypes.c_int)]


class ExpertStackStruct(ctypes.Structure):
    """``struct qvb8_expert_stack`` of the header."""
    _fields_ = [
        ("ids", ctypes.c_void_p), ("ids_bytes", ctypes.c_int64), ("min_s", ctypes.c_void_p),
        ("tau_s", ctypes.c_void_p), ("nbits", ctypes.c_void_p), ("bit_off", ctypes.c_void_p),
        ("Q", ctypes.c_int64), ("P", ctypes.c_int64),
    ]


class RPackStruct(ctypes.Structure):
    """``struct qvb8r_pack`` of the header."""
    _fields_ = [
        ("words", ctypes.c_void_p), ("tile_off", ctypes.c_void_p), ("states", ctypes.c_void_p),
        ("tiles", ctypes.c_void_p), ("n_tiles", ctypes.c_int64), ("blocks", ctypes.c_void_p),
        ("n_blocks", ctypes.c_int64), ("tab", ctypes.c_void_p), ("perm", ctypes.c_void_p), ("min_s", ctypes.c_void_p),
        ("tau_s", ctypes.c_void_p), ("drow", ctypes.c_void_p), ("Q", ctypes.c_int64), ("P", ctypes.c_int64),
    ]


_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build the CUDA kernel library first (python -m qvb8_b200.build). "
                    "There is no CPU or eager fallback for the QVB8 kernels.")
            lib = ctypes.CDLL(LIB_PATH)
            vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
            pk = ctypes.POINTER(PackStruct)
            lib.qvb8_last_error.restype = ctypes.c_char_p
            lib.qvb8_version.restype = ctypes.c_char_p
            lib.qvb8_decode.argtypes = [pk, ci, vp, vp]
            lib.qvb8_small_m_scratch_bytes.argtypes = [i64, i64, i64]
            lib.qvb8_small_m_scratch_bytes.restype = i64
            lib.qvb8_small_m.argtypes = [pk, vp, ci, ci, i64, vp, vp, i64, vp]
            lib.qvb8_small_m_generic.argtypes = [pk, vp, ci, ci, i64, vp, vp]
            lib.qvb8_small_m_static.argtypes = [pk, vp, vp, ci, ci, i64, vp, ci, vp]
            lib.qvb8_small_m_static_max_scratch.argtypes = []
            lib.qvb8_small_m_static_max_scratch.restype = i64
            lib.qvb8_plan_bytes.argtypes = [i64, i64]
            lib.qvb8_plan_bytes.restype = i64
            lib.qvb8_plan_build.argtypes = [pk, vp, i64, vp]
            lib.qvb8_small_m_ex.argtypes = [pk, vp, vp, ci, ci, i64, vp, vp, i64, ci, vp]
            lib.qvb8_small_m_set_tuning.argtypes = [ci, ci, ci, ci, ci]
            jb = ctypes.POINTER(JobStruct)
            lib.qvb8_small_m_group_scratch_bytes.argtypes = [jb, ci, i64]
            lib.qvb8_small_m_group_scratch_bytes.restype = i64
            lib.qvb8_small_m_group.argtypes = [jb, ci, i64, vp, i64, ci, vp]
            pi = ctypes.POINTER(ctypes.c_int)
            lib.qvb8_small_m_group_describe.argtypes = [jb, ci, i64, pi, pi, pi]
            lib.qvb8_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
            lib.qvb8_debug_trace.argtypes = [ctypes.POINTER(ctypes.c_uint64)]
            lib.qvb8_small_m_set_tuning.restype = None
            lib.qvb8_prefill_scratch_bytes.argtypes = [i64, i64, i64]
            lib.qvb8_prefill_scratch_bytes.restype = i64
            lib.qvb8_prefill.argtypes = [pk, vp, vp, ci, i64, vp, vp, i64, vp]
            lib.qvb8_embed_rows.argtypes = [pk, vp, i64, ci, vp, vp]
            lib.qvb8_peer_bytes.argtypes = [ci, i64]
            lib.qvb8_peer_bytes.restype = i64
            lib.qvb8_peer_alloc.argtypes = [i64, ctypes.POINTER(vp), ctypes.c_char_p]
            lib.qvb8_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
            lib.qvb8_peer_close.argtypes = [vp, ci]
            lib.qvb8_peer_allreduce.argtypes = [ctypes.POINTER(vp), ci, ci, i64, vp, vp, vp, i64, ci, vp]
            lib.qvb8_peer_allreduce_ex.argtypes = [ctypes.POINTER(vp), ci, ci, i64, vp, vp, vp, i64, ci, ctypes.c_uint64, vp]
            lib.qvb8_peer_allreduce_local.argtypes = [ctypes.POINTER(vp), ci, i64, ctypes.POINTER(vp), ctypes.POINTER(vp),
                                                      ctypes.POINTER(vp), i64, ctypes.c_uint64, vp]
            lib.qvb8_peer_allgather.argtypes = lib.qvb8_peer_allreduce_ex.argtypes
            lib.qvb8_peer_allgather_local.argtypes = lib.qvb8_peer_allreduce_local.argtypes
            lib.qvb8_device_status_reset.argtypes = []
            lib.qvb8_prefill_set_tuning.argtypes = [ci]
            lib.qvb8_prefill_set_tuning.restype = None
            es = ctypes.POINTER(ExpertStackStruct)
            rp = ctypes.POINTER(RPackStruct)
            lib.qvb8r_ids.argtypes = [rp, vp, vp]
            lib.qvb8r_decode.argtypes = [rp, ci, vp, i64, i64, i64, vp]
            lib.qvb8r_small_m.argtypes = [rp, vp, ci, i64, ci, vp, vp]
            lib.qvb8r_fix_escapes.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
            lib.qvb8r_embed_rows.argtypes = [rp, vp, i64, vp, vp, vp, vp, vp, vp, vp]
            lib.qvb8_moe_scratch_bytes.argtypes = [i64, i64, i64, i64, i64, i64, ci]
            lib.qvb8_moe_scratch_bytes.restype = i64
            lib.qvb8_moe_experts.argtypes = [vp, ci, i64, vp, vp, i64, i64, es, es, ci, vp, vp, i64, vp]
            lib.qvb8_moe_streams.argtypes = [i64, i64, i64, es, es]
            lib.qvb8_argmax_scratch_bytes.argtypes = [i64]
            lib.qvb8_argmax_scratch_bytes.restype = i64
            lib.qvb8_argmax_rows.argtypes = [vp, i64, i64, i64, i64, vp, vp, vp, i64, vp]
            lib.qvb8_moe_plan_bytes.argtypes = [i64, i64]
            lib.qvb8_moe_plan_bytes.restype = i64
            lib.qvb8_moe_plan_build.argtypes = [es, i64, vp, i64, vp]
            lib.qvb8_moe_experts_planned.argtypes = [vp, ci, i64, vp, vp, i64, i64, es, es, vp, vp, ci, vp, vp, i64, vp]
            lib.qvb8_moe_bad_index.argtypes = [vp, i64, i64, i64, i64, i64, i64, ci, ctypes.POINTER(ctypes.c_int)]
            _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (status {rc}): {load().qvb8_last_error().decode()}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise RuntimeError(f"qvb8_b200: dtype {dt} is not float16 / bfloat16 / float32") from None


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _cuda(t: torch.Tensor, name: str, dtype: torch.dtype) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"qvb8_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"qvb8_b200: {name} must be {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def pack_struct(ids, min_s, tau_s, nbits, bit_off, P: int, esc_idx, esc_vals):
    """Validated ``qvb8_pack`` for tensors on one CUDA device.  Returns (struct, keepalive list)."""
    ids = _cuda(ids, "ids", torch.uint8)
    min_s = _cuda(min_s, "min_s", torch.float32)
    tau_s = _cuda(tau_s, "tau_s", torch.float32)
    nbits = _cuda(nbits, "row_nbits", torch.uint8)
    bit_off = _cuda(bit_off, "row_bit_off", torch.int64)
    Q = min_s.numel()
    if tau_s.numel() != Q or nbits.numel() != Q or bit_off.numel() != Q:
        raise RuntimeError("qvb8_b200: min_s / tau_s / row_nbits / row_bit_off must all have Q entries")
    n_esc = esc_idx.numel() if esc_idx is not None else 0
    keep = [ids, min_s, tau_s, nbits, bit_off]
    ei = ev = None
    if n_esc:
        ei = _cuda(esc_idx, "esc_idx", torch.int64)
        ev = _cuda(esc_vals, "esc_vals", torch.float32)
        if ev.numel() != n_esc:
            raise RuntimeError("qvb8_b200: esc_idx and esc_vals differ in length")
        keep += [ei, ev]
    dev = ids.device
    for t in keep:
        if t.device != dev:
            raise RuntimeError("qvb8_b200: all pack tensors must live on one device")
    s = PackStruct(ids.data_ptr(), ids.numel(), min_s.data_ptr(), tau_s.data_ptr(), nbits.data_ptr(),
                   bit_off.data_ptr(), Q, int(P), ei.data_ptr() if n_esc else None, ev.data_ptr() if n_esc else None,
                   n_esc)
    return s, keep


# ---------------------------------------------------------------------------------------------------------------
# scratch (split-K partial sums + tickets), one zero-initialised buffer per (device, stream)

_scratch: dict = {}


def scratch_for(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """A zero-initialised scratch buffer of at least `nbytes` for the current stream of `device`.  Kernels leave it
    reusable; buffers are keyed by stream because two calls sharing one buffer must not overlap on the device."""
    if nbytes <= 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr(device))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def reserve_scratch(device: torch.device, M: int, Q: int, P: int) -> None:
    """Allocate the scratch a later small-M call of these sizes needs (call before capturing a CUDA graph)."""
    scratch_for(device, int(load().qvb8_small_m_scratch_bytes(M, Q, P)))


# ---------------------------------------------------------------------------------------------------------------
# thin wrappers

def decode(pack, keep, out_dtype: torch.dtype) -> torch.Tensor:
    dev = keep[0].device
    out = torch.empty((pack.Q, pack.P), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        check(load().qvb8_decode(ctypes.byref(pack), dtype_code(out_dtype), out.data_ptr(), stream_ptr(dev)),
              "qvb8_decode")
    return out


def embed_rows(pack, keep, rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """(n, P) restored rows `rows` (int64, on the pack's device) of a pack used as an embedding table."""
    dev = keep[0].device
    if rows.dtype != torch.int64 or rows.device != dev or not rows.is_contiguous() or rows.dim() != 1:
        raise RuntimeError("qvb8_b200: embed_rows takes a contiguous 1-D int64 tensor on the pack's device")
    out = torch.empty((rows.numel(), pack.P), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        check(load().qvb8_embed_rows(ctypes.byref(pack), rows.data_ptr(), rows.numel(), dtype_code(out_dtype),
                                     out.data_ptr(), stream_ptr(dev)), "qvb8_embed_rows")
    return out


FLAG_PDL = 1


def device_status(device=None) -> int:
    """Error word of `device` (0 = no kernel of this library ever gave up on a wait).  Synchronises."""
    v = ctypes.c_int(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        check(load().qvb8_device_status(ctypes.byref(v)), "qvb8_device_status")
    return int(v.value)


def build_plan(pack, keep) -> torch.Tensor:
    """Device buffer with the pack's plan (rows sorted by width into tile descriptors + escapes regrouped by row)."""
    dev = keep[0].device
    lib = load()
    nbytes = int(lib.qvb8_plan_bytes(pack.Q, pack.n_esc))
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(lib.qvb8_plan_build(ctypes.byref(pack), buf.data_ptr(), nbytes, stream_ptr(dev)), "qvb8_plan_build")
    return buf


def plan_on(ids: torch.Tensor, pack, keep) -> torch.Tensor:
    """The plan of a pack, cached on the `ids` tensor OBJECT (so it lives and dies with the weight and can never be
    matched to another weight that later reuses the address); rebuilt if the pack's geometry or escape table differ."""
    key = (pack.ids, pack.Q, pack.P, pack.n_esc, pack.esc_idx, pack.min_s, pack.bit_off)
    cache = ids.__dict__.setdefault("_qvb8_plans", {}) if hasattr(ids, "__dict__") else None
    if cache is None:
        return build_plan(pack, keep)
    plan = cache.get(key)
    if plan is None:
        if len(cache) > 8:
            cache.clear()
        plan = cache[key] = build_plan(pack, keep)
    return plan


def small_m(pack, keep, X: torch.Tensor, x_mode: int = 0, generic: bool = False, out: torch.Tensor | None = None,
            plan: torch.Tensor | None = None, flags: int = 0):
    """(M, Q) fp32 = X (M, P) @ W^T through the fused kernel (M <= 48).  `plan` from build_plan / plan_on selects the
    streaming kernel; without it the layout-agnostic kernel runs."""
    dev = keep[0].device
    if not X.is_cuda or X.device != dev:
        raise RuntimeError("qvb8_b200: X must be a CUDA tensor on the pack's device")
    if X.dim() != 2 or X.shape[1] != pack.P:
        raise RuntimeError(f"qvb8_b200: X must be (M, {pack.P}), got {tuple(X.shape)}")
    X = X if X.is_contiguous() else X.contiguous()
    M = X.shape[0]
    Y = out if out is not None else torch.empty((M, pack.Q), dtype=torch.float32, device=dev)
    lib = load()
    with torch.cuda.device(dev):
        if generic:
            rc = lib.qvb8_small_m_generic(ctypes.byref(pack), X.data_ptr(), dtype_code(X.dtype), x_mode, M,
                                          Y.data_ptr(), stream_ptr(dev))
        else:
            nbytes = int(lib.qvb8_small_m_scratch_bytes(M, pack.Q, pack.P))
            sc = scratch_for(dev, nbytes)
            rc = lib.qvb8_small_m_ex(ctypes.byref(pack), plan.data_ptr() if plan is not None else None, X.data_ptr(),
                                     dtype_code(X.dtype), x_mode, M, Y.data_ptr(),
                                     sc.data_ptr() if sc is not None else None, sc.numel() if sc is not None else 0,
                                     flags, stream_ptr(dev))
    check(rc, "qvb8_small_m")
    return Y


class JobList:
    """A list of independent products prepared once for :func:`small_m_group`: (pack struct, keepalive, plan, X, Y) per
    job, all with the same row count M.  The ctypes array and everything it points at is kept alive here."""

    def __init__(self, items, x_mode: int = 0):
        if not items:
            raise RuntimeError("qvb8_b200: an empty job list")
        self.items = list(items)
        self.M = int(self.items[0][3].shape[0])
        self.device = self.items[0][1][0].device
        self.array = (JobStruct * len(self.items))()
        for k, (st, keep, plan, X, Y) in enumerate(self.items):
            if X.dim() != 2 or X.shape != (self.M, st.P) or not X.is_contiguous() or X.device != self.device:
                raise RuntimeError(f"qvb8_b200: job {k}: X must be a contiguous ({self.M}, {st.P}) tensor on the packs' device")
            if Y.dtype != torch.float32 or Y.shape != (self.M, st.Q) or not Y.is_contiguous() or Y.device != self.device:
                raise RuntimeError(f"qvb8_b200: job {k}: Y must be a contiguous fp32 ({self.M}, {st.Q}) tensor")
            if plan is None:
                raise RuntimeError(f"qvb8_b200: job {k} has no plan")
            self.array[k] = JobStruct(ctypes.pointer(st), plan.data_ptr(), X.data_ptr(), Y.data_ptr(), dtype_code(X.dtype),
                                      int(x_mode))
        self.scratch_bytes = int(load().qvb8_small_m_group_scratch_bytes(self.array, len(self.items), self.M))


def small_m_group(jobs: JobList, flags: int = 0) -> None:
    """Runs the jobs of a :class:`JobList` (outputs land in the Y tensors it was built with) on the current stream."""
    dev = jobs.device
    sc = scratch_for(dev, jobs.scratch_bytes)
    with torch.cuda.device(dev):
        check(load().qvb8_small_m_group(jobs.array, len(jobs.items), jobs.M, sc.data_ptr() if sc is not None else None,
                                        sc.numel() if sc is not None else 0, int(flags), stream_ptr(dev)),
              "qvb8_small_m_group")


def prefill(pack, keep, X: torch.Tensor, plan: torch.Tensor | None = None) -> torch.Tensor:
    """(M, Q) fp32 = X (M, P) @ W^T through the tcgen05 prefill kernel (any M; meant for M in the hundreds and up)."""
    dev = keep[0].device
    if not X.is_cuda or X.device != dev or X.dim() != 2 or X.shape[1] != pack.P:
        raise RuntimeError(f"qvb8_b200: X must be a CUDA (M, {pack.P}) tensor on the pack's device")
    X = X if X.is_contiguous() else X.contiguous()
    M = X.shape[0]
    lib = load()
    if plan is None:
        plan = build_plan(pack, keep)
    nbytes = int(lib.qvb8_prefill_scratch_bytes(M, pack.Q, pack.P))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    Y = torch.empty((M, pack.Q), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.qvb8_prefill(ctypes.byref(pack), plan.data_ptr(), X.data_ptr(),
                               dtype_code(X.dtype), M, Y.data_ptr(), scratch.data_ptr(), nbytes, stream_ptr(dev)),
              "qvb8_prefill")
    return Y


def argmax_rows(Y: torch.Tensor, index_base: int = 0):
    """(values fp32 (M,), indices int64 (M,)) of the largest logit per row of Y (M, V) fp32 and the lowest column that
    holds it (+ index_base), on Y's device and current stream."""
    if not Y.is_cuda or Y.dtype != torch.float32 or Y.dim() != 2 or Y.stride(1) != 1:
        raise RuntimeError("qvb8_b200: argmax_rows takes a CUDA fp32 matrix with contiguous rows (there is no CPU path)")
    M, V = Y.shape
    L = load()
    dev = Y.device
    val = torch.empty(M, dtype=torch.float32, device=dev)
    idx = torch.empty(M, dtype=torch.int64, device=dev)
    nbytes = int(L.qvb8_argmax_scratch_bytes(M))
    scratch = torch.empty(max(8, nbytes), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(L.qvb8_argmax_rows(Y.data_ptr(), M, V, Y.stride(0) if M > 1 else V, int(index_base), val.data_ptr(),
                                 idx.data_ptr(), scratch.data_ptr(), nbytes, stream_ptr(dev)), "qvb8_argmax_rows")
    return val, idx


# ---------------------------------------------------------------------------------------------------------------
# mixture of experts

def expert_stack_struct(ids, min_s, tau_s, nbits, bit_off, Q: int, P: int):
    """Validated ``qvb8_expert_stack`` for stacked expert tensors on one CUDA device.  Returns (struct, keepalive)."""
    ids = _cuda(ids, "stacked ids", torch.uint8)
    min_s = _cuda(min_s, "stacked min_s", torch.float32)
    tau_s = _cuda(tau_s, "stacked tau_s", torch.float32)
    nbits = _cuda(nbits, "stacked nbits", torch.uint8)
    bit_off = _cuda(bit_off, "stacked bit_off", torch.int64)
    n = min_s.numel()
    if n == 0 or n % int(Q) or tau_s.numel() != n or nbits.numel() != n or bit_off.numel() != n:
        raise RuntimeError("qvb8_b200: stacked expert metadata must all have E * Q entries")
    s = ExpertStackStruct(ids.data_ptr(), ids.numel(), min_s.data_ptr(), tau_s.data_ptr(), nbits.data_ptr(),
                          bit_off.data_ptr(), int(Q), int(P))
    return s, [ids, min_s, tau_s, nbits, bit_off], n // int(Q)


def moe_plan_on(stack) -> torch.Tensor | None:
    """The per-expert plans of a stack (struct, keepalive, E), cached on its `ids` tensor object like a pack's plan.
    None while a stream capture is in progress and no plan exists yet (the caller then takes the plan-less route)."""
    st, keep, E = stack
    ids = keep[0]
    key = ("moe", st.ids, st.Q, st.P, E, st.bit_off, st.min_s)
    cache = ids.__dict__.setdefault("_qvb8_plans", {}) if hasattr(ids, "__dict__") else {}
    plan = cache.get(key)
    if plan is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        L = load()
        nbytes = int(L.qvb8_moe_plan_bytes(E, st.Q))
        plan = torch.empty(nbytes, dtype=torch.uint8, device=ids.device)
        with torch.cuda.device(ids.device):
            check(L.qvb8_moe_plan_build(ctypes.byref(st), E, plan.data_ptr(), nbytes, stream_ptr(ids.device)),
                  "qvb8_moe_plan_build")
        if len(cache) > 8:
            cache.clear()
        cache[key] = plan
    return plan


MOE_STREAM_TOKENS = 8        # up to this many tokens the expert layer runs on the streaming kernel (needs plans)


def moe_experts(X: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, up, dn, act: int) -> torch.Tensor:
    """(M, Qdn) in X.dtype.  `up` / `dn` = (struct, keepalive, E) from expert_stack_struct; act 0 gated SiLU, 1 relu^2."""
    ust, ukeep, E = up
    dst, dkeep, E2 = dn
    if E != E2:
        raise RuntimeError("moe: up and down stacks hold different numbers of experts")
    dev = ukeep[0].device
    if not X.is_cuda or X.device != dev or X.dim() != 2 or X.shape[1] != ust.P:
        raise RuntimeError("moe: bad X")
    if idx.dtype != torch.int64 or w.dtype != torch.float32:
        raise RuntimeError("moe: idx must be int64 and w float32")
    if X.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        X = X.float()
    X, idx, w = X.contiguous(), idx.to(dev).contiguous(), w.to(dev).contiguous()
    M, topk = idx.shape
    if M != X.shape[0] or tuple(w.shape) != (M, topk):
        raise RuntimeError("moe: idx / w must be (M, topk)")
    lib = load()
    nbytes = int(lib.qvb8_moe_scratch_bytes(M, topk, E, ust.P, ust.Q, dst.Q, act))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)       # stream-ordered: torch's allocator
    out = torch.empty((M, dst.Q), dtype=X.dtype, device=dev)
    uplan = dplan = None
    if M <= MOE_STREAM_TOKENS and ust.P % 128 == 0 and dst.P % 128 == 0:
        uplan, dplan = moe_plan_on(up), moe_plan_on(dn)
    with torch.cuda.device(dev):
        check(lib.qvb8_moe_experts_planned(X.data_ptr(), dtype_code(X.dtype), M, idx.data_ptr(), w.data_ptr(), topk, E,
                                           ctypes.byref(ust), ctypes.byref(dst),
                                           uplan.data_ptr() if uplan is not None and dplan is not None else None,
                                           dplan.data_ptr() if uplan is not None and dplan is not None else None,
                                           act, out.data_ptr(), scratch.data_ptr(), nbytes, stream_ptr(dev)),
              "qvb8_moe_experts")
    return out
