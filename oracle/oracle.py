"""numpy front end of the C oracle (test infrastructure; see the package docstring).

Every function takes and returns numpy arrays.  The C library is built on first
use with ``make`` (gcc) into ``oracle/_build``; a prebuilt copy is used as is.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libqvb8_oracle.so")
_lib = None

__all__ = [
    "build", "num_threads", "unpack_ids", "restore_f32", "decode_16", "matmul_f32w", "f32_to_f16_bits",
    "f32_to_bf16_bits", "sat_half", "rans_decode_ids", "rans_restore_f32", "slot_tables", "qvb8_dense",
    "qvb8r_dense", "moe_experts",
]


def build(force: bool = False) -> str:
    """Compile qvb8_oracle.c if the library is missing or older than the source."""
    src = os.path.join(_HERE, "qvb8_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_LIB_PATH))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(_load().qvb8o_num_threads())


def unpack_ids(buf, nbits, bit_off, Q: int, P: int) -> np.ndarray:
    """(Q, P) uint16 ids of a QVB8 payload (decode.py:346-365)."""
    buf, nbits, bit_off = _c(buf, np.uint8), _c(nbits, np.uint8), _c(bit_off, np.int64)
    out = np.empty((Q, P), np.uint16)
    _load().qvb8o_unpack_ids(_p(buf), _p(nbits), _p(bit_off), ctypes.c_int64(Q), ctypes.c_int64(P), _p(out))
    return out


def restore_f32(ids, min_s, tau_s, esc_idx=None, esc_vals=None) -> np.ndarray:
    """fp32 band values fma(id, tau_s, min_s) with escapes written over (decode.py:196-212)."""
    ids = _c(ids, np.uint16)
    Q, P = ids.shape
    min_s, tau_s = _c(min_s, np.float32), _c(tau_s, np.float32)
    ei = _c(esc_idx if esc_idx is not None else [], np.int64)
    ev = _c(esc_vals if esc_vals is not None else [], np.float32)
    out = np.empty((Q, P), np.float32)
    _load().qvb8o_restore_f32(_p(ids), _p(min_s), _p(tau_s), ctypes.c_int64(Q), ctypes.c_int64(P), _p(ei), _p(ev),
                              ctypes.c_int64(ei.size), _p(out))
    return out


def decode_16(buf, nbits, bit_off, min_s, tau_s, Q: int, P: int, esc_idx, esc_vals, kind: str) -> np.ndarray:
    """Dense (Q, P) restore rounded once to fp16 (kind='f16') or bf16 (kind='bf16'); returns the raw 16-bit
    patterns as uint16 (qvb8_cuda.cu:592-699, 1711-1727)."""
    buf, nbits, bit_off = _c(buf, np.uint8), _c(nbits, np.uint8), _c(bit_off, np.int64)
    min_s, tau_s = _c(min_s, np.float32), _c(tau_s, np.float32)
    ei, ev = _c(esc_idx, np.int64), _c(esc_vals, np.float32)
    out = np.empty((Q, P), np.uint16)
    _load().qvb8o_decode_16(_p(buf), _p(nbits), _p(bit_off), _p(min_s), _p(tau_s), ctypes.c_int64(Q),
                            ctypes.c_int64(P), _p(ei), _p(ev), ctypes.c_int64(ei.size),
                            ctypes.c_int(1 if kind == "bf16" else 0), _p(out))
    return out


def matmul_f32w(X, W, narrow_x: bool = True) -> np.ndarray:
    """(M, Q) float64 product of X (M, P) with fp32 weights W (Q, P); X narrowed to saturated fp16 first when
    narrow_x (the QVB8 GEMV contract, qvb8_cuda.cu:1082-1102)."""
    X, W = _c(X, np.float32), _c(W, np.float32)
    M, P = X.shape
    Q = W.shape[0]
    out = np.empty((M, Q), np.float64)
    _load().qvb8o_matmul_f32w(_p(X), ctypes.c_int64(M), _p(W), ctypes.c_int64(Q), ctypes.c_int64(P),
                              ctypes.c_int(1 if narrow_x else 0), _p(out))
    return out


def f32_to_f16_bits(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    _load().qvb8o_f32_to_f16(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def f32_to_bf16_bits(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    _load().qvb8o_f32_to_bf16(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def sat_half(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.float32)
    _load().qvb8o_sat_half(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def slot_tables(freq) -> np.ndarray:
    """(K, N) frequencies (each row sums to 4096) -> (K, 4096) packed slot entries
    ``symbol | offset_in_symbol << 11 | (freq - 1) << 22`` (qvb8r/codec.py:11-20)."""
    F = np.asarray(freq, np.int64)
    K, N = F.shape
    tab = np.zeros((K, 4096), np.uint32)
    for k in range(K):
        assert int(F[k].sum()) == 4096, "frequencies of a class must sum to 4096"
        sym = np.repeat(np.arange(N, dtype=np.int64), F[k])
        start = np.cumsum(F[k]) - F[k]
        d = np.arange(4096, dtype=np.int64) - start[sym]
        tab[k] = (sym | (d << 11) | ((F[k][sym] - 1) << 22)).astype(np.uint32)
    return tab


def rans_decode_ids(words, tile_off, states, tiles, tab, perm, drow, Q: int, P: int) -> np.ndarray:
    """(Q, P) int16 ids of a .qvb8r tensor in original row order (qvb8r_cpu.cpp:13-58)."""
    words = _c(words, np.uint32)
    tile_off, tiles = _c(tile_off, np.int64), _c(tiles, np.int64)
    states, tab = _c(states, np.uint64), _c(tab, np.uint32)
    perm, drow = _c(perm, np.int32), _c(drow, np.int32)
    out = np.zeros((Q, P), np.int16)
    rc = _load().qvb8ro_decode_ids(_p(words), ctypes.c_int64(words.size), _p(tile_off), _p(states), _p(tiles),
                                   ctypes.c_int64(tiles.shape[0]), _p(tab), _p(perm), _p(drow), ctypes.c_int64(P),
                                   _p(out))
    if rc != 0:
        raise ValueError("rANS stream ran past the end of the word array")
    return out


def rans_restore_f32(ids, min_s, tau_s) -> np.ndarray:
    ids = _c(ids, np.int16)
    Q, P = ids.shape
    out = np.empty((Q, P), np.float32)
    _load().qvb8ro_restore_f32(_p(ids), _p(_c(min_s, np.float32)), _p(_c(tau_s, np.float32)), ctypes.c_int64(Q),
                               ctypes.c_int64(P), _p(out))
    return out


# ---------------------------------------------------------------------------------------------------------------
# whole-pack conveniences (dicts as produced by the package's pack readers)

def qvb8_dense(pk: dict, table: str = "fp16") -> np.ndarray:
    """fp32 restored weights of a parsed QVB8 pack dict, escapes of the chosen table written over."""
    ids = unpack_ids(pk["ids"], pk["nbits"], pk["bit_off"], pk["Q"], pk["P"])
    ei, ev = (pk["esc_idx_bf16"], pk["esc_vals_bf16"]) if table == "bf16" else (pk["esc_idx"], pk["esc_vals"])
    return restore_f32(ids, pk["min_s"], pk["tau_s"], ei, ev)


def qvb8r_dense(d: dict) -> np.ndarray:
    """fp32 restored weights of a parsed .qvb8r dict (escapes written over with their exact value)."""
    tab = slot_tables(d["freq"])
    ids = rans_decode_ids(d["words"], d["tile_off"], d["states"], d["tiles"], tab, d["perm"],
                          np.asarray(d["drow"], np.int32), int(d["Q"]), int(d["P"]))
    W = rans_restore_f32(ids, d["min_s"], d["tau_s"])
    if len(d["esc_idx"]):
        W.reshape(-1)[np.asarray(d["esc_idx"], np.int64)] = np.asarray(d["esc_val"], np.float32)
    return W


def moe_experts(X, idx, w, up_dense, dn_dense, act: str = "silu") -> np.ndarray:
    """Expert MLP the grouped kernels compute (reference qvb8_cuda.cu:949-992 gated SiLU; :1002-1058 relu^2):
    out[t] = sum_j w[t, j] * W_dn[e] @ act(W_up[e] @ x_t), e = idx[t, j], x narrowed to saturated fp16 first, the
    hidden activations kept in full precision.  up_dense / dn_dense: per-expert restored fp32 weights (E, Q, P).
    Accumulates in float64; returns float64 (M, Qdn)."""
    X = np.asarray(X, dtype=np.float32)
    xs = sat_half(X).astype(np.float64)
    idx = np.asarray(idx)
    w = np.asarray(w, dtype=np.float32).astype(np.float64)
    M, topk = idx.shape
    out = np.zeros((M, dn_dense.shape[1]), dtype=np.float64)
    for t in range(M):
        for j in range(topk):
            e = int(idx[t, j])
            y = up_dense[e].astype(np.float64) @ xs[t]
            if act == "silu":
                half = y.shape[0] // 2
                g, u = y[:half], y[half:]
                h = (g / (1.0 + np.exp(-g))) * u
            else:
                h = np.maximum(y, 0.0) ** 2
            # the kernels keep h in fp32
            h = h.astype(np.float32).astype(np.float64)
            out[t] += w[t, j] * (dn_dense[e].astype(np.float64) @ h)
    return out
