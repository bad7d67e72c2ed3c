"""Drop-in object for the reference's ``qvb8r_cuda`` extension module (entropy-coded QVB8).

The reference fetches it through ``_load_ext()`` (formats/qvb8r/module.py:25-33) and calls the entry points registered
at formats/qvb8r/backends/cuda_qvb8r/qvb8r_cuda.cu:446-456 with the ten "core" tensors
``(words i32, off i64, states i64, tiles i64, blocks i32, tab i32, perm i32, min_s f32, tau_s f32, drow i32)``
(:322-335).  :data:`ext` exposes the same names, argument order, dtypes and return shapes on the sm_100a kernels of
this package; :func:`core_tensors` builds the ten tensors from a parsed ``.qvb8r`` dict the way the reference's
loader does (container.py:84-89 runtime_tables, :74-82 blocks_for).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import lib as _lib
from . import rans

TILES_PER_BLOCK = 8


def core_tensors(d: dict, device) -> tuple:
    """The ten core tensors of a parsed .qvb8r dict (numpy arrays) on `device`."""
    dev = torch.device(device)
    words = np.concatenate([np.asarray(d["words"], np.uint32), np.zeros(rans.PAD_WORDS, np.uint32)])
    tiles = np.asarray(d["tiles"], np.int64).reshape(-1, 3)
    blocks = rans.blocks_for(tiles, TILES_PER_BLOCK)
    tab = rans.slot_tables(np.asarray(d["freq"]))
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt) if a.dtype.itemsize == np.dtype(dt).itemsize
                                       else np.ascontiguousarray(a, dtype=dt)).to(dev)
    return (t(words, np.int32), t(np.asarray(d["tile_off"], np.int64), np.int64),
            t(np.asarray(d["states"], np.uint64).reshape(-1), np.int64), t(tiles, np.int64), t(blocks, np.int32),
            t(tab, np.int32), t(np.asarray(d["perm"], np.int32), np.int32), t(np.asarray(d["min_s"], np.float32), np.float32),
            t(np.asarray(d["tau_s"], np.float32), np.float32), t(np.asarray(d["drow"], np.int32), np.int32))


def _struct(P, words, off, states, tiles, blocks, tab, perm, mn, ts, drow):
    want = (torch.int32, torch.int64, torch.int64, torch.int64, torch.int32, torch.int32, torch.int32, torch.float32,
            torch.float32, torch.int32)
    core = (words, off, states, tiles, blocks, tab, perm, mn, ts, drow)
    dev = words.device
    for a, dt in zip(core, want):
        if not a.is_cuda or a.device != dev or a.dtype != dt or not a.is_contiguous():
            raise RuntimeError("qvb8r: core tensor dtypes")
    st = _lib.RPackStruct(words.data_ptr(), off.data_ptr(), states.data_ptr(), tiles.data_ptr(), tiles.numel() // 3,
                          blocks.data_ptr(), blocks.numel() // 3, tab.data_ptr(), perm.data_ptr(), mn.data_ptr(),
                          ts.data_ptr(), drow.data_ptr(), mn.numel(), int(P))
    return st, dev


class Qvb8rExt:
    """Same attribute surface as the reference's ``qvb8r_cuda`` pybind module (GPU entry points)."""

    def ids(self, P, *core):
        """Every id, (Q, P) int16 in original row order (qvb8r_cuda.cu:351-363)."""
        if int(P) % 128:
            raise RuntimeError("qvb8r ids: P % 128 == 0")
        st, dev = _struct(P, *core)
        out = torch.empty((st.Q, int(P)), dtype=torch.int16, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().qvb8r_ids(ctypes.byref(st), out.data_ptr(), _lib.stream_ptr(dev)), "qvb8r_ids")
        return out

    def _mm(self, X, core, round_w):
        st, dev = _struct(X.shape[1], *core)
        M = X.shape[0]
        Y = torch.empty((M, st.Q), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().qvb8r_small_m(ctypes.byref(st), X.data_ptr(), _lib.dtype_code(X.dtype), M, round_w,
                                                 Y.data_ptr(), _lib.stream_ptr(dev)), "qvb8r_small_m")
        return Y

    def gemv(self, X, *core):
        """M = 1: X fp32 of length P -> (Q) fp32 (qvb8r_cuda.cu:337-349)."""
        if not X.is_cuda or X.dtype != torch.float32 or not X.is_contiguous() or X.numel() % 128:
            raise RuntimeError("qvb8r gemv: X must be contiguous fp32 CUDA, P % 128 == 0")
        return self._mm(X.reshape(1, -1), core, 0).reshape(-1)

    def multi(self, X, *core):
        """M = 1..8, X fp32 or bf16 -> (M, Q) fp32 (qvb8r_cuda.cu:365-392)."""
        if not X.is_cuda or X.dtype not in (torch.float32, torch.bfloat16) or X.dim() != 2:
            raise RuntimeError("qvb8r multi: X must be (M, P) fp32 or bf16 CUDA")
        if not 1 <= X.shape[0] <= 8 or X.shape[1] % 128:
            raise RuntimeError("qvb8r multi: M must be 1..8 and P % 128 == 0")
        return self._mm(X.contiguous(), core, 0)

    def tc(self, X, *core_and_T):
        """M = 1..16, X fp16, band value rounded to fp16 -> (M, Q) fp32 (qvb8r_cuda.cu:394-407).  The trailing
        tile-height argument T of the reference is accepted and not needed."""
        *core, _T = core_and_T
        if not X.is_cuda or X.dtype != torch.float16 or not X.is_contiguous() or X.dim() != 2:
            raise RuntimeError("qvb8r tc: X must be contiguous (M, P) fp16 CUDA")
        if not 1 <= X.shape[0] <= 16 or X.shape[1] % 128:
            raise RuntimeError("qvb8r tc: M must be 1..16 and P % 128 == 0")
        return self._mm(X, core, 1)

    def decode(self, *args):
        """decode(*core, P, out_dtype in {0 fp16, 1 bf16, 2 fp32}, b0, nb, row_base, nrows) (qvb8r_cuda.cu:409-432)."""
        *core, P, out_dtype, b0, nb, row_base, nrows = args
        if int(P) % 128:
            raise RuntimeError("qvb8r decode: P % 128 == 0")
        st, dev = _struct(P, *core)
        if b0 < 0 or nb < 0 or b0 + nb > st.n_blocks:
            raise RuntimeError("qvb8r decode: block range out of bounds")
        rows = st.Q if row_base < 0 else int(nrows)
        dt = (torch.float16, torch.bfloat16, torch.float32)[int(out_dtype)]
        W = torch.empty((rows, int(P)), dtype=dt, device=dev)
        if nb == 0:
            return W
        with torch.cuda.device(dev):
            _lib.check(_lib.load().qvb8r_decode(ctypes.byref(st), _lib.dtype_code(dt), W.data_ptr(), int(b0), int(nb),
                                                int(row_base), _lib.stream_ptr(dev)), "qvb8r_decode")
        return W

    def fix_escapes(self, X, uq, ptr, ec, ed, Y):
        """In place: Y[m, uq[u]] += sum_e X[m, ec[e]] * ed[e] (qvb8r_cuda.cu:434-444)."""
        if X.dtype != torch.float32 or Y.dtype != torch.float32 or not X.is_contiguous() or not Y.is_contiguous():
            raise RuntimeError("qvb8r fix_escapes: X and Y must be contiguous fp32")
        U = uq.numel()
        if U == 0:
            return
        dev = Y.device
        with torch.cuda.device(dev):
            _lib.check(_lib.load().qvb8r_fix_escapes(X.data_ptr(), uq.data_ptr(), ptr.data_ptr(), ec.data_ptr(),
                                                     ed.data_ptr(), Y.data_ptr(), U, X.shape[0], X.shape[1], Y.shape[1],
                                                     _lib.stream_ptr(dev)), "qvb8r_fix_escapes")


    # ---- the reference extension's host-side entry points (qvb8r_cuda.cu:453-455) ------------------------------
    def embed_rows(self, rows, words, off, states, tiles, tab, inv_perm, row_tile, mn, ts, drow, esc_ptr, esc_col,
                   esc_val, P):
        """(n, P) fp32 rows of an entropy-coded embedding table, escapes written over (qvb8r_cpu.cpp:13-58).  The
        reference hands HOST tensors here and decodes on the host, because its target cards cannot hold the table; on
        a B200 the table is uploaded once (cached on the `words` tensor object) and the rows are decoded by
        ``qvb8r_embed_rows`` on the device.  The result comes back on the host, as the caller expects."""
        if int(P) % 128:
            raise RuntimeError("qvb8r embed_rows: P % 128 == 0")
        table = words.__dict__.get("_qvb8r_device_table") if hasattr(words, "__dict__") else None
        if table is None:
            table = EmbeddingTable(words, off, states, tiles, tab, inv_perm, row_tile, mn, ts, drow, esc_ptr, esc_col,
                                   esc_val, int(P), torch.device("cuda", torch.cuda.current_device()))
            if hasattr(words, "__dict__"):
                words.__dict__["_qvb8r_device_table"] = table
        Q = table.Q
        rows = rows.reshape(-1).to(torch.int64)
        if rows.numel() and (int(rows.min()) < 0 or int(rows.max()) >= Q):
            raise RuntimeError("qvb8r embed_rows: row id out of range")
        return table.lookup(rows.to(table.device)).cpu()

    def encode(self, sym, tiles, F, C):
        """rANS-code (R, P) int16 symbols in sorted row order -> [words i32, tile_off i64, states i64]
        (qvb8r_cpu.cpp:60-110).  A writer's tool, run once per tensor on the host."""
        if sym.dtype != torch.int16 or sym.dim() != 2 or sym.shape[1] % 128 or not sym.is_contiguous():
            raise RuntimeError("qvb8r encode: sym must be contiguous (R, P) int16, P % 128 == 0")
        if tiles.dtype != torch.int64 or F.dtype != torch.int64 or C.dtype != torch.int64:
            raise RuntimeError("qvb8r encode: int64 tables")
        t = tiles.cpu().numpy().reshape(-1, 3)
        states, words, tile_off = rans.encode_symbols(sym.cpu().numpy(), t[:, 0], t[:, 2], F.cpu().numpy())
        return [torch.from_numpy(words.view(np.int32).copy()), torch.from_numpy(tile_off.astype(np.int64)),
                torch.from_numpy(states.view(np.int64).copy())]

    def row_hist(self, sym, N):
        """(R, N) int32 histogram of every row's int16 symbols in [0, N) (qvb8r_cpu.cpp:112-121)."""
        if sym.dtype != torch.int16 or sym.dim() != 2 or not sym.is_contiguous():
            raise RuntimeError("qvb8r row_hist: (R, P) int16")
        s = sym.cpu().numpy().astype(np.int64)
        if s.size and (s.min() < 0 or s.max() >= int(N)):
            raise RuntimeError("qvb8r row_hist: symbol outside [0, N)")
        R = s.shape[0]
        flat = (np.arange(R, dtype=np.int64)[:, None] * int(N) + s).ravel()
        return torch.from_numpy(np.bincount(flat, minlength=R * int(N)).reshape(R, int(N)).astype(np.int32))


class EmbeddingTable:
    """An entropy-coded embedding table resident on one device + the row lookup kernel."""

    def __init__(self, words, off, states, tiles, tab, inv_perm, row_tile, mn, ts, drow, esc_ptr, esc_col, esc_val, P: int,
                 device):
        dev = torch.device(device)
        up = lambda t, dt: t.to(device=dev, dtype=dt).contiguous()
        self.device, self.P, self.Q = dev, int(P), int(mn.numel())
        tiles_d = up(tiles, torch.int64)
        blocks = torch.from_numpy(rans.blocks_for(tiles.cpu().numpy().reshape(-1, 3), TILES_PER_BLOCK)).to(dev)
        perm = torch.empty(self.Q, dtype=torch.int32)
        perm[inv_perm.cpu().long()] = torch.arange(self.Q, dtype=torch.int32)
        self.core = (up(words, torch.int32), up(off, torch.int64), up(states, torch.int64), tiles_d, blocks.contiguous(),
                     up(tab, torch.int32), perm.to(dev), up(mn, torch.float32), up(ts, torch.float32), up(drow, torch.int32))
        self.inv_perm, self.row_tile = up(inv_perm, torch.int32), up(row_tile, torch.int32)
        self.esc_ptr, self.esc_col, self.esc_val = up(esc_ptr, torch.int64), up(esc_col, torch.int32), up(esc_val, torch.float32)

    def lookup(self, rows: torch.Tensor) -> torch.Tensor:
        """(n, P) fp32 on the table's device; `rows` int64 on that device."""
        st, dev = _struct(self.P, *self.core)
        rows = rows.contiguous()
        out = torch.empty((rows.numel(), self.P), dtype=torch.float32, device=dev)
        if rows.numel():
            null = lambda t: t.data_ptr() if t.numel() else None
            with torch.cuda.device(dev):
                _lib.check(_lib.load().qvb8r_embed_rows(ctypes.byref(st), rows.data_ptr(), rows.numel(),
                                                        self.inv_perm.data_ptr(), self.row_tile.data_ptr(),
                                                        self.esc_ptr.data_ptr(), null(self.esc_col), null(self.esc_val),
                                                        out.data_ptr(), _lib.stream_ptr(dev)), "qvb8r_embed_rows")
        return out

    @classmethod
    def from_parsed(cls, d: dict, device) -> "EmbeddingTable":
        """From a parsed .qvb8r dict (packs.read_qvb8r): builds the per-row tables a lookup needs."""
        Q, P = int(d["Q"]), int(d["P"])
        tiles = np.asarray(d["tiles"], np.int64).reshape(-1, 3)
        inv = np.empty(Q, np.int32)
        inv[np.asarray(d["perm"], np.int64)] = np.arange(Q, dtype=np.int32)
        row_tile = np.repeat(np.arange(len(tiles), dtype=np.int32), tiles[:, 2])
        pos = np.asarray(d["esc_idx"], np.int64)
        order = np.argsort(pos, kind="stable")
        ptr = np.concatenate([[0], np.cumsum(np.bincount(pos // P, minlength=Q))]).astype(np.int64)
        T = torch.from_numpy
        words = np.concatenate([np.asarray(d["words"], np.uint32), np.zeros(rans.PAD_WORDS, np.uint32)])
        return cls(T(words.view(np.int32)), T(np.asarray(d["tile_off"]).astype(np.int64)),
                   T(np.ascontiguousarray(np.asarray(d["states"], np.uint64).reshape(-1)).view(np.int64)), T(tiles),
                   T(rans.slot_tables(np.asarray(d["freq"])).view(np.int32)), T(inv), T(row_tile),
                   T(np.asarray(d["min_s"], np.float32)), T(np.asarray(d["tau_s"], np.float32)),
                   T(np.asarray(d["drow"]).astype(np.int32)), T(ptr), T((pos % P)[order].astype(np.int32)),
                   T(np.asarray(d["esc_val"], np.float32)[order]), P, device)


ext = Qvb8rExt()


def escape_csr(d: dict, device):
    """(uq, ptr, ec, ed): the outputs that have escapes, their ranges, the escapes' columns and stored differences --
    what the reference module builds at load for fix_escapes (formats/qvb8r/module.py:100-124)."""
    P = int(d["P"])
    ei = np.asarray(d["esc_idx"], np.int64)
    rows, cols = ei // P, ei % P
    uq, start = np.unique(rows, return_index=True)
    ptr = np.concatenate([start, [ei.size]]).astype(np.int64)
    dev = torch.device(device)
    return (torch.from_numpy(uq.astype(np.int64)).to(dev), torch.from_numpy(ptr).to(dev),
            torch.from_numpy(cols.astype(np.int64)).to(dev), torch.from_numpy(np.asarray(d["esc_delta"], np.float32)).to(dev))


def install() -> None:
    """Rebind the reference's qvb8r loader to this package's kernels (the reference package must be importable)."""
    import importlib
    mod = importlib.import_module("qv_band.formats.qvb8r.module")
    mod._load_ext = lambda: ext
