"""QVB8 pack files: byte layouts, readers and writers.

Two on-disk containers hold a QVB8 tensor (per-row virtual-band ids, LSB-first bit-packed, rows back to back):

``QVBD`` (the current container; reference formats/qvb8/pack_container.py:8-22, 48-106)
    32-byte header ``<4sBIIffBBB8x`` = magic ``QVBD``, version 1, Q, P, tau f32, max_err f32, source code,
    calc_method (0 = formula), restore code (0 = fp16, 3 = fp16+bf16); then ``min_s f32[Q]``, ``tau_s f32[Q]``,
    ``nbits u8[Q]``, the bit payload (+8 zero bytes), ``n_esc u64, n8 u64``, the fp32-pool escapes
    (``idx i64[n32]`` + values: bf16 bits as ``u16`` for a 16-bit source, ``u32`` fp32 bits for an fp32 source),
    the FP8-pool escapes (``idx i64[n8]`` + E4M3 codes ``u8[n8]``) and ``s8 f32[Q]`` (per-row FP8 scale).
    Row bit offsets are NOT stored: row q starts at ``sum(nbits[:q]) * P``.

legacy ``QVB8`` v11 blob (reference formats/qvb8/decode.py:30-43, 53-86, 384-430)
    64-byte header ``<IIIIdQIQ20x`` = magic 0x38425651, Q, P, version 11, tau f64, n_esc, esc_mode, n_fp8; then
    ``min_s``, ``tau_s``, ``nbits u8[Q]``, ``bit_off u64[Q]``, escapes (mode 0: ``idx i64`` + ``f32``; mode 1: fp32
    pool, FP8 pool, ``s8 f32[Q]``), then the bit payload to the end of the blob.

Both decode to the same in-memory dict (see :func:`read_qvb8`), which is what the device-side loader uploads.
"""
from __future__ import annotations

import json
import os
import struct
import zlib

import numpy as np

QVBD_MAGIC = b"QVBD"
QVBD_HEADER = "<4sBIIffBBB8x"
QVBD_HEADER_BYTES = 32
LEGACY_MAGIC = 0x38425651
LEGACY_HEADER = "<IIIIdQIQ20x"
LEGACY_HEADER_V10 = "<IIIIdQIB27x"
LEGACY_HEADER_BYTES = 64
MAX_CERTIFIED_NBITS = 14          # decode.py:76-86: wider rows cannot be certified in fp32
PAYLOAD_PAD = 8                   # zero bytes after the bit payload (decode.py:303-306)
SOURCE_CODES = {"bf16": 0, "fp8_block": 1, "q4_block": 2, "fp32": 3}
SOURCE_NAMES = {v: k for k, v in SOURCE_CODES.items()}
RESTORE_NAMES = {0: "fp16", 3: "fp16+bf16"}
RESTORE_CODES = {v: k for k, v in RESTORE_NAMES.items()}
ESCAPE_TABLES_FILE = "escape_tables.json"


class PackFormatError(ValueError):
    """A pack blob that cannot be read (bad magic, version, truncated, unsupported layout)."""


# ---------------------------------------------------------------------------------------------------------------
# bit payload

def row_bit_offsets(nbits: np.ndarray, P: int) -> np.ndarray:
    """Absolute bit offset of every row's first id (exclusive prefix sum of nbits * P)."""
    bits = np.asarray(nbits, np.int64) * int(P)
    off = np.zeros(len(bits), np.int64)
    if len(bits) > 1:
        np.cumsum(bits[:-1], out=off[1:])
    return off


def payload_bytes(nbits: np.ndarray, P: int) -> int:
    return (int(np.asarray(nbits, np.int64).sum()) * int(P) + 7) // 8


def pack_ids(ids: np.ndarray, nbits: np.ndarray) -> np.ndarray:
    """Bit-pack (Q, P) ids at each row's own width, LSB-first, rows back to back, + PAYLOAD_PAD zero bytes.

    Host-side writer for small tensors (tests, fixtures); the bulk generator packs on the device.
    """
    ids = np.asarray(ids)
    Q, P = ids.shape
    nb = np.asarray(nbits, np.int64)
    off = row_bit_offsets(nb, P)
    total = payload_bytes(nb, P)
    bits = np.zeros(total * 8 + 64, np.uint8)
    for q in range(Q):
        w = int(nb[q])
        row = ids[q].astype(np.uint32)
        if int(row.max(initial=0)) >> w:
            raise PackFormatError(f"row {q}: an id does not fit {w} bits")
        b = ((row[:, None] >> np.arange(w, dtype=np.uint32)[None, :]) & 1).astype(np.uint8)
        bits[off[q]:off[q] + w * P] = b.reshape(-1)
    buf = np.packbits(bits[:total * 8], bitorder="little")
    return np.concatenate([buf, np.zeros(PAYLOAD_PAD, np.uint8)])


# ---------------------------------------------------------------------------------------------------------------
# FP8 escape pool (reference decode.py:104-161)

def e4m3_table() -> np.ndarray:
    """The 256 float32 values of the E4M3FN bit patterns (0x7F / 0xFF are NaN)."""
    code = np.arange(256)
    sign = np.where(code & 0x80, -1.0, 1.0)
    e, m = (code >> 3) & 0xF, code & 0x7
    sub = sign * m * 2.0 ** -9
    nor = sign * (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7.0)
    v = np.where(e == 0, sub, nor)
    v = np.where((e == 15) & (m == 7), np.nan, v)
    return v.astype(np.float32)


def merge_escape_pools(e32_idx, e32_vals, e8_idx, e8_codes, s8, P: int):
    """One escape list, ascending by flat index.  An FP8 escape's value is fp16(lut[code] * s8[row])."""
    if len(e8_idx) == 0:
        return np.asarray(e32_idx, np.int64), np.asarray(e32_vals, np.float32)
    with np.errstate(over="ignore"):
        v8 = (e4m3_table()[e8_codes] * s8[e8_idx // P]).astype(np.float16).astype(np.float32)
    idx = np.concatenate([e32_idx, e8_idx]).astype(np.int64)
    val = np.concatenate([e32_vals, v8]).astype(np.float32)
    o = np.argsort(idx, kind="stable")
    return idx[o], val[o]


# ---------------------------------------------------------------------------------------------------------------
# escape_tables.json (reference formats/qvb8/escape_split.py:14-54)

class EscapeTableError(RuntimeError):
    pass


def fp16_escape_mask(pack_path: str | None, esc_idx: np.ndarray):
    """Keep-mask selecting the fp16 escape table out of the pack's full list, from the folder's escape_tables.json
    (version 2).  None when there is no file or no entry for this pack."""
    if not pack_path:
        return None
    f = os.path.join(os.path.dirname(os.path.abspath(pack_path)), ESCAPE_TABLES_FILE)
    if not os.path.exists(f):
        return None
    with open(f) as fh:
        data = json.load(fh)
    if data.get("version") != 2:
        raise EscapeTableError(f"{f}: version {data.get('version')}, this reader knows 2")
    e = data.get("tensors", {}).get(os.path.basename(pack_path))
    if e is None or e.get("restore") != "fp16+bf16":
        return None
    kind = "fp16" if "fp16" in e else "bf16_only"
    lst = np.asarray(e[kind], np.int64)
    if int(e["n_bf16"]) != len(esc_idx):
        raise EscapeTableError(f"{pack_path}: {ESCAPE_TABLES_FILE} says {e['n_bf16']} escapes, the pack has "
                               f"{len(esc_idx)}")
    hit = np.isin(esc_idx, lst)
    if int(hit.sum()) != len(lst):
        raise EscapeTableError(f"{pack_path}: {ESCAPE_TABLES_FILE} lists positions that are not escapes of this pack")
    keep = hit if kind == "fp16" else ~hit
    if int(keep.sum()) != int(e["n_fp16"]):
        raise EscapeTableError(f"{pack_path}: fp16 table size mismatch")
    return keep


def write_escape_tables(folder: str, entries: dict) -> None:
    """entries: pack basename -> (full esc_idx, fp16 keep-mask)."""
    tensors = {}
    for name, (idx, keep) in entries.items():
        idx = np.asarray(idx, np.int64)
        fp16, bonly = idx[keep], idx[~keep]
        rec = {"restore": "fp16+bf16", "n_bf16": int(len(idx)), "n_fp16": int(keep.sum())}
        if len(fp16) <= len(bonly):
            rec["fp16"] = fp16.tolist()
        else:
            rec["bf16_only"] = bonly.tolist()
        tensors[name] = rec
    with open(os.path.join(folder, ESCAPE_TABLES_FILE), "w") as fh:
        json.dump({"version": 2, "tensors": tensors}, fh)


# ---------------------------------------------------------------------------------------------------------------
# readers

def validate_pack(d: dict, where: str = "pack") -> dict:
    """Bounds of a parsed pack, checked on the host before anything is uploaded: the kernels trust these fields, so a
    cut-short or damaged file must be refused here and never become an out-of-range read on the device.  Row widths
    1..14, every row's bit range (plus the 8 pad bytes the readers may touch) inside the payload, escape positions
    ascending and inside the weight."""
    Q, P = int(d["Q"]), int(d["P"])
    nbits = np.asarray(d["nbits"], np.int64)
    bit_off = np.asarray(d["bit_off"], np.int64)
    if Q < 0 or P <= 0 or nbits.shape != (Q,) or bit_off.shape != (Q,) or len(d["min_s"]) != Q or len(d["tau_s"]) != Q:
        raise PackFormatError(f"{where}: per-row arrays do not have Q = {Q} entries")
    if Q:
        if nbits.min() < 1 or nbits.max() > MAX_CERTIFIED_NBITS:
            raise PackFormatError(f"{where}: row width outside 1..{MAX_CERTIFIED_NBITS} bits")
        if bit_off.min() < 0:
            raise PackFormatError(f"{where}: negative row offset")
        last_byte = int(((bit_off + nbits * P + 7) >> 3).max())
        if last_byte + PAYLOAD_PAD > len(d["ids"]):
            raise PackFormatError(f"{where}: a row ends at byte {last_byte} (+{PAYLOAD_PAD} pad bytes) but the payload "
                                  f"holds {len(d['ids'])} bytes (cut-short or damaged file)")
    for key in ("esc_idx", "esc_idx_bf16"):
        ei = np.asarray(d.get(key, ()), np.int64)
        vals = d.get("esc_vals" if key == "esc_idx" else "esc_vals_bf16", ())
        if ei.size != len(vals):
            raise PackFormatError(f"{where}: {key} and its values differ in length")
        if ei.size and (ei.min() < 0 or ei.max() >= Q * P or np.any(np.diff(ei) < 0)):
            raise PackFormatError(f"{where}: {key} is not an ascending list of positions inside the weight")
    return d


def _need(blob, cur, n, what):
    if cur + n > len(blob):
        raise PackFormatError(f"truncated pack: {what} needs {n} bytes at {cur}, blob has {len(blob)}")


def read_qvbd(blob: bytes, path: str | None = None) -> dict:
    if len(blob) < QVBD_HEADER_BYTES:
        raise PackFormatError("truncated QVBD header")
    magic, ver, Q, P, tau, max_err, src, calc, restore = struct.unpack(QVBD_HEADER, blob[:QVBD_HEADER_BYTES])
    if magic != QVBD_MAGIC:
        raise PackFormatError(f"not a QVBD blob (magic {magic!r})")
    if ver != 1:
        raise PackFormatError(f"QVBD version {ver}, this reader knows 1")
    if calc != 0:
        raise PackFormatError("QVBD table packs (calc_method=1) are a pre-unification layout: re-pack")
    if restore not in RESTORE_NAMES:
        raise PackFormatError(f"QVBD restore code {restore} is not fp16 (0) or fp16+bf16 (3)")
    source = SOURCE_NAMES.get(src)
    if source is None:
        raise PackFormatError(f"QVBD source code {src} unknown")
    cur = QVBD_HEADER_BYTES
    _need(blob, cur, 9 * Q, "row metadata")
    min_s = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
    tau_s = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
    nbits = np.frombuffer(blob, np.uint8, Q, cur).copy(); cur += Q
    if Q and (nbits.min() < 1 or nbits.max() > MAX_CERTIFIED_NBITS):
        raise PackFormatError(f"row width outside 1..{MAX_CERTIFIED_NBITS} bits")
    nbytes = payload_bytes(nbits, P) + PAYLOAD_PAD
    _need(blob, cur, nbytes + 16, "bit payload")
    ids = np.frombuffer(blob, np.uint8, nbytes, cur).copy(); cur += nbytes
    n_esc, n8 = struct.unpack_from("<QQ", blob, cur); cur += 16
    n32 = n_esc - n8
    if n32 < 0:
        raise PackFormatError(f"{n8} FP8 escapes of {n_esc} total")
    w32 = 4 if source == "fp32" else 2
    _need(blob, cur, (8 + w32) * n32 + 9 * n8 + 4 * Q, "escape pools")
    e32_idx = np.frombuffer(blob, "<i8", n32, cur).copy(); cur += 8 * n32
    raw = np.frombuffer(blob, "<u4" if w32 == 4 else "<u2", n32, cur).copy(); cur += w32 * n32
    e32_vals = raw.view(np.float32) if w32 == 4 else (raw.astype(np.uint32) << 16).view(np.float32)
    e8_idx = np.frombuffer(blob, "<i8", n8, cur).copy(); cur += 8 * n8
    e8_codes = np.frombuffer(blob, np.uint8, n8, cur).copy(); cur += n8
    s8 = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
    esc_idx, esc_vals = merge_escape_pools(e32_idx, e32_vals, e8_idx, e8_codes, s8, P)
    out = dict(container="QVBD", Q=int(Q), P=int(P), tau=float(tau), max_err=float(max_err), source=source,
               restore=RESTORE_NAMES[restore], min_s=min_s, tau_s=tau_s, nbits=nbits,
               bit_off=row_bit_offsets(nbits, P), ids=ids)
    # The blob's list is the bf16 table (every escape).  The fp16 table is the subset named by escape_tables.json;
    # for an fp16-only pack the two are the same list.
    out["esc_idx_bf16"], out["esc_vals_bf16"] = esc_idx, esc_vals
    out["fp16_table_missing"] = False
    if out["restore"] == "fp16+bf16":
        keep = fp16_escape_mask(path, esc_idx)
        if keep is None:
            out["esc_idx"], out["esc_vals"] = esc_idx, esc_vals
            out["fp16_table_missing"] = True
        else:
            out["esc_idx"], out["esc_vals"] = esc_idx[keep], esc_vals[keep]
    else:
        out["esc_idx"], out["esc_vals"] = esc_idx, esc_vals
    return validate_pack(out, path or "QVBD blob")


def read_qvb8_legacy(blob: bytes) -> dict:
    if len(blob) < LEGACY_HEADER_BYTES:
        raise PackFormatError("truncated QVB8 header")
    magic, Q, P, version = struct.unpack_from("<IIII", blob, 0)
    if magic != LEGACY_MAGIC:
        raise PackFormatError(f"not a QVB8 blob (magic {magic:#x})")
    if version not in (9, 10, 11):
        raise PackFormatError(f"QVB8 version {version}, this reader knows 9, 10, 11")
    fmt = LEGACY_HEADER_V10 if version == 10 else LEGACY_HEADER
    _, Q, P, _, tau, n_esc, esc_mode, n_fp8 = struct.unpack(fmt, blob[:LEGACY_HEADER_BYTES])
    cur = LEGACY_HEADER_BYTES
    _need(blob, cur, 17 * Q, "row metadata")
    min_s = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
    tau_s = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
    nbits = np.frombuffer(blob, np.uint8, Q, cur).copy(); cur += Q
    bit_off = np.frombuffer(blob, "<u8", Q, cur).astype(np.int64); cur += 8 * Q
    if version == 9 or esc_mode == 0:
        _need(blob, cur, 12 * n_esc, "escapes")
        esc_idx = np.frombuffer(blob, "<i8", n_esc, cur).copy(); cur += 8 * n_esc
        esc_vals = np.frombuffer(blob, "<f4", n_esc, cur).copy(); cur += 4 * n_esc
    else:
        if n_fp8 > n_esc:
            raise PackFormatError(f"{n_fp8} FP8 escapes of {n_esc} total")
        n32 = n_esc - n_fp8
        _need(blob, cur, 12 * n32 + 9 * n_fp8 + 4 * Q, "escape pools")
        e32_idx = np.frombuffer(blob, "<i8", n32, cur).copy(); cur += 8 * n32
        e32_vals = np.frombuffer(blob, "<f4", n32, cur).copy(); cur += 4 * n32
        e8_idx = np.frombuffer(blob, "<i8", n_fp8, cur).copy(); cur += 8 * n_fp8
        e8_codes = np.frombuffer(blob, np.uint8, n_fp8, cur).copy(); cur += n_fp8
        s8 = np.frombuffer(blob, "<f4", Q, cur).copy(); cur += 4 * Q
        esc_idx, esc_vals = merge_escape_pools(e32_idx, e32_vals, e8_idx, e8_codes, s8, P)
    ids = np.frombuffer(blob, np.uint8, offset=cur).copy()
    return validate_pack(dict(container="QVB8", Q=int(Q), P=int(P), tau=float(tau), max_err=float("nan"), source="bf16",
                restore="fp16", min_s=min_s, tau_s=tau_s, nbits=nbits, bit_off=bit_off, ids=ids,
                esc_idx=esc_idx, esc_vals=esc_vals, esc_idx_bf16=esc_idx, esc_vals_bf16=esc_vals,
                fp16_table_missing=False), "QVB8 blob")


def read_qvb8(blob: bytes, path: str | None = None) -> dict:
    """Parse either container into one dict:

    Q, P, tau, restore ('fp16' | 'fp16+bf16'), min_s f32[Q], tau_s f32[Q], nbits u8[Q], bit_off i64[Q],
    ids u8[payload + 8], esc_idx i64 / esc_vals f32 (the fp16 table, sorted by flat index q*P+c),
    esc_idx_bf16 / esc_vals_bf16 (the bf16 table = every escape), fp16_table_missing.
    """
    if blob[:4] == QVBD_MAGIC:
        return read_qvbd(blob, path)
    return read_qvb8_legacy(blob)


def read_qvb8_shape(blob: bytes) -> tuple[int, int]:
    if blob[:4] == QVBD_MAGIC:
        _, _, Q, P = struct.unpack_from("<4sBII", blob, 0)
        return int(Q), int(P)
    magic, Q, P = struct.unpack_from("<III", blob, 0)
    if magic != LEGACY_MAGIC:
        raise PackFormatError("not a QVB8 blob")
    return int(Q), int(P)


# ---------------------------------------------------------------------------------------------------------------
# writers (the reference ships readers only; these emit bytes its readers parse)

def write_qvbd(*, Q, P, tau, max_err, min_s, tau_s, nbits, ids, esc_idx, esc_vals, source="bf16",
               restore="fp16", fp8_idx=None, fp8_codes=None, fp8_scale=None) -> bytes:
    """`ids` is the bit payload INCLUDING its 8 pad bytes; esc_idx / esc_vals are the escapes kept at full width
    (values must be exactly representable in the source type: they are stored as bf16 bits for a 16-bit source).
    fp8_idx / fp8_codes / fp8_scale: the escapes kept as E4M3 codes with a per-row scale f32[Q] (the second pool of
    the container, pack_container.py:14-20); a reader merges both pools into one list."""
    nbits = np.asarray(nbits, np.uint8)
    ids = np.asarray(ids, np.uint8)
    if len(ids) != payload_bytes(nbits, P) + PAYLOAD_PAD:
        raise PackFormatError("payload length does not match nbits")
    esc_idx = np.asarray(esc_idx, np.int64)
    esc_vals = np.asarray(esc_vals, np.float32)
    if source == "fp32":
        raw = esc_vals.view(np.uint32).astype("<u4").tobytes()
    else:
        bits = esc_vals.view(np.uint32)
        if np.any(bits & 0xFFFF):
            raise PackFormatError("an escape value is not bf16-representable but the source is 16-bit")
        raw = (bits >> 16).astype("<u2").tobytes()
    hdr = struct.pack(QVBD_HEADER, QVBD_MAGIC, 1, int(Q), int(P), float(tau), float(max_err), SOURCE_CODES[source], 0,
                      RESTORE_CODES[restore])
    n8 = 0 if fp8_idx is None else len(fp8_idx)
    if n8:
        fp8_idx, fp8_codes = np.asarray(fp8_idx, np.int64), np.asarray(fp8_codes, np.uint8)
        s8 = np.asarray(fp8_scale, np.float32)
        if len(fp8_codes) != n8 or s8.shape != (int(Q),):
            raise PackFormatError("FP8 pool: one code per index and one scale per row")
        pool8 = fp8_idx.astype("<i8").tobytes() + fp8_codes.tobytes()
    else:
        pool8, s8 = b"", np.zeros(int(Q), np.float32)
    return b"".join([
        hdr, np.asarray(min_s, "<f4").tobytes(), np.asarray(tau_s, "<f4").tobytes(), nbits.tobytes(), ids.tobytes(),
        struct.pack("<QQ", len(esc_idx) + n8, n8), esc_idx.astype("<i8").tobytes(), raw, pool8,
        s8.astype("<f4").tobytes()])


def write_qvb8_legacy(*, Q, P, tau, min_s, tau_s, nbits, bit_off, ids, esc_idx, esc_vals) -> bytes:
    hdr = struct.pack(LEGACY_HEADER, LEGACY_MAGIC, int(Q), int(P), 11, float(tau), len(esc_idx), 0, 0)
    return b"".join([
        hdr, np.asarray(min_s, "<f4").tobytes(), np.asarray(tau_s, "<f4").tobytes(),
        np.asarray(nbits, np.uint8).tobytes(), np.asarray(bit_off, "<u8").tobytes(),
        np.asarray(esc_idx, "<i8").tobytes(), np.asarray(esc_vals, "<f4").tobytes(), np.asarray(ids, np.uint8).tobytes()])


def pack_filename(tensor_name: str, fmt: str) -> str:
    """File name of a tensor inside a pack directory (reference common/formats.py:45-48)."""
    import re
    return re.sub(r"[^A-Za-z0-9]", "_", tensor_name) + "." + fmt


# ---------------------------------------------------------------------------------------------------------------
# .qvb8r (reference formats/qvb8r/container.py:1-12, 30-89)

QVBR_MAGIC, QVBR_VERSION, QVBR_PB = b"QVBR", 2, 12
QVBR_PAD_WORDS = 2048      # zero words appended at load: the stream readers fetch ahead of their cursor


QVBR_ARRAYS = (("perm", np.int32), ("freq", np.uint16), ("tiles", np.int32), ("tile_off", np.uint32),
               ("states", np.uint64), ("words", np.uint32), ("drow", np.int16), ("min_s", np.float32),
               ("tau_s", np.float32), ("esc_idx", np.int64), ("esc_val", np.float32), ("esc_delta", np.float32))
_QVBR_ALIGN = 64


def _align64(n: int) -> int:
    return -(-n // _QVBR_ALIGN) * _QVBR_ALIGN


def _qvbr_directory(meta: dict, arrays: dict) -> tuple[bytes, dict]:
    """The JSON header of a .qvb8r file and the byte offset of every array.  The directory sits inside the JSON whose
    own length moves the offsets, so the text is regenerated until its length no longer changes (it can only grow by
    a digit or two, so this settles in two or three rounds)."""
    where: dict = {}
    text_len = -1
    while True:
        cursor = _align64(12 + max(text_len, 0))
        for name, a in arrays.items():
            where[name] = cursor
            cursor = _align64(cursor + a.nbytes)
        head = dict(meta, arrays={n: [where[n], a.dtype.str, list(a.shape)] for n, a in arrays.items()})
        text = json.dumps(head).encode()
        if len(text) == text_len:
            return text, where
        text_len = len(text)


def write_qvb8r(enc: dict, *, Q, P, min_s, tau_s, esc_idx, esc_val, esc_delta, cert: dict) -> bytes:
    """The bytes of a .qvb8r file (layout: reference formats/qvb8r/container.py:1-12): ``QVBR`` | u32 version 2 |
    u32 header length | JSON header (Q, P, T, K, N, PB, cert, arrays: name -> [offset, dtype, shape]) | zero pad to
    64 | the arrays, each starting on a multiple of 64 | zero pad to 64 | u32 crc32 of every byte before it.
    enc: perm, freq, tiles, tile_off, states, words, drow, T, K, N (see :mod:`qvb8_b200.rans`)."""
    given = dict(enc, min_s=min_s, tau_s=tau_s, esc_idx=esc_idx, esc_val=esc_val, esc_delta=esc_delta)
    arrays = {name: np.ascontiguousarray(given[name], dtype=dt) for name, dt in QVBR_ARRAYS}
    meta = dict(Q=int(Q), P=int(P), T=int(enc["T"]), K=int(enc["K"]), N=int(enc["N"]), PB=QVBR_PB, cert=cert)
    text, where = _qvbr_directory(meta, arrays)
    end = _align64(max([12 + len(text)] + [where[n] + a.nbytes for n, a in arrays.items()]))
    out = np.zeros(end + 4, np.uint8)
    out[:4] = np.frombuffer(QVBR_MAGIC, np.uint8)
    out[4:12] = np.frombuffer(struct.pack("<II", QVBR_VERSION, len(text)), np.uint8)
    out[12:12 + len(text)] = np.frombuffer(text, np.uint8)
    for name, a in arrays.items():
        out[where[name]:where[name] + a.nbytes] = np.frombuffer(a.tobytes(), np.uint8)
    out[end:] = np.frombuffer(struct.pack("<I", zlib.crc32(out[:end].tobytes()) & 0xFFFFFFFF), np.uint8)
    return out.tobytes()


def read_qvb8r(blob: bytes, where: str = "<blob>") -> dict:
    """Header fields + arrays (copies) of a .qvb8r file; PackFormatError on anything that is not a sound version-2
    file: wrong magic or version, checksum, model constants, an array outside the file or of the wrong type / shape."""
    n = len(blob)
    if n < 16 or bytes(blob[:4]) != QVBR_MAGIC:
        raise PackFormatError(f"{where}: no QVBR magic at the start")
    version, text_len = struct.unpack_from("<II", blob, 4)
    if version != QVBR_VERSION:
        raise PackFormatError(f"{where}: file version {version}; only version {QVBR_VERSION} "
                              "(centred rows, 64-bit states, 32-bit words) can be read")
    stored = struct.unpack_from("<I", blob, n - 4)[0]
    if stored != zlib.crc32(memoryview(blob)[:n - 4]) & 0xFFFFFFFF:
        raise PackFormatError(f"{where}: checksum does not match the contents (cut short or damaged)")
    if 12 + text_len > n - 4:
        raise PackFormatError(f"{where}: header length {text_len} runs past the file")
    try:
        head = json.loads(bytes(blob[12:12 + text_len]))
        listing = head["arrays"]
        Q, P = int(head["Q"]), int(head["P"])
    except (ValueError, KeyError, TypeError) as ex:
        raise PackFormatError(f"{where}: unreadable header ({ex})") from None
    if head.get("PB") != QVBR_PB:
        raise PackFormatError(f"{where}: probability precision {head.get('PB')} bits, the decoders are built for {QVBR_PB}")
    out = {k: v for k, v in head.items()}
    for name, want in QVBR_ARRAYS:
        if name not in listing:
            raise PackFormatError(f"{where}: array {name} is missing")
        off, dt, shape = listing[name]
        dt = np.dtype(dt)
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if dt != np.dtype(want) or off < 0 or off + count * dt.itemsize > n - 4:
            raise PackFormatError(f"{where}: array {name} has the wrong type or lies outside the file")
        out[name] = np.frombuffer(blob, dt, count, off).reshape(shape).copy()
    nt = out["tiles"].shape[0] if out["tiles"].ndim == 2 else -1
    ok = (out["perm"].shape == (Q,) and out["drow"].shape == (Q,) and out["min_s"].shape == (Q,)
          and out["tau_s"].shape == (Q,) and out["tiles"].ndim == 2 and out["tiles"].shape[1:] == (3,)
          and out["tile_off"].shape == (nt + 1,) and out["states"].shape == (nt, 32) and out["freq"].ndim == 2
          and out["esc_idx"].shape == out["esc_val"].shape == out["esc_delta"].shape)
    if not ok:
        raise PackFormatError(f"{where}: array shapes do not fit Q = {Q}")
    if nt and (int(out["tile_off"][-1]) > out["words"].size or np.any(np.diff(out["tile_off"].astype(np.int64)) < 0)):
        raise PackFormatError(f"{where}: tile offsets do not fit the word stream")
    return out
