"""Seeded synthetic QVB8 packs.

The reference ships pack *readers* only, and no sample packs.  This module writes packs in the reference's layout
from seeded random weights so the kernels, the tests and the benchmark have inputs of the shapes and value
distributions the benchmark configurations name.  It is written with torch ops only, so the same code runs on the
host (small test tensors, byte-identical fixtures) and on the GPU (multi-gigabyte benchmark stacks in seconds).

Encoding of one row (reference formats/qvb8/decode.py:14-28, formats/qvb8/module.py:92-94):

    id    = floor((w - row_min) / tau_s)        min_s = row_min + tau_s / 2
    value = fma(id, tau_s, min_s)               nbits = ceil(log2(number of buckets)), at least 1

``tau_s`` is chosen per row as 2 * (tau - half an fp16 ulp at the row's largest in-band magnitude) so that the value
ROUNDED to fp16 still lies within tau of the source weight.  Every element is then checked against the certificate
``|fp16(value) - w| <= tau`` and ``|value - w| <= tau``; an element that fails, lies outside the band, or exceeds
``tau * 2**10`` in magnitude (decode.py:88-91) is escaped: its exact value is stored with its flat position.
For ``restore='fp16+bf16'`` a second, larger escape table additionally holds the positions where
``|bf16(value) - w| > tau`` (formats/qvb8/escape_split.py:14-34).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import packs

FP16_MANTISSA_BITS = 10


def synth_weight(Q: int, P: int, seed: int, device="cpu", std: float = 0.02, outlier_frac: float = 1e-3,
                 outlier_sigma: float = 10.0) -> torch.Tensor:
    """(Q, P) bf16 weights ~ N(0, std) with `outlier_frac` of the entries replaced by +-outlier_sigma*std."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    w = torch.randn(Q, P, generator=g, device=device, dtype=torch.float32) * std
    if outlier_frac > 0:
        u = torch.rand(Q, P, generator=g, device=device, dtype=torch.float32)
        out = u < outlier_frac
        sign = torch.where(u < outlier_frac / 2, -1.0, 1.0)
        w = torch.where(out, sign * (outlier_sigma * std), w)
    return w.to(torch.bfloat16)


def synth_activation(M: int, P: int, seed: int = 7, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return torch.randn(M, P, generator=g, device=device, dtype=torch.float32).to(dtype)


@dataclass
class QVB8Pack:
    """A QVB8 tensor as the kernels read it (all tensors on one device).

    ids       u8[payload + 8]   bit-packed ids, LSB-first, rows back to back, 8 zero pad bytes
    min_s     f32[Q]            row origin (centre of bucket 0)
    tau_s     f32[Q]            row bucket step
    nbits     u8[Q]             row id width
    bit_off   i64[Q]            first bit of each row in `ids`
    esc_idx   i64[E]            flat positions q*P+c of the escapes, ascending  (fp16 table)
    esc_vals  f32[E]            their exact values
    esc_idx_bf16 / esc_vals_bf16   the bf16 table (a superset; the same tensors for an fp16-only pack)
    """
    Q: int
    P: int
    tau: float
    restore: str
    ids: torch.Tensor
    min_s: torch.Tensor
    tau_s: torch.Tensor
    nbits: torch.Tensor
    bit_off: torch.Tensor
    esc_idx: torch.Tensor
    esc_vals: torch.Tensor
    esc_idx_bf16: torch.Tensor
    esc_vals_bf16: torch.Tensor
    max_err: float = float("nan")
    stats: dict = field(default_factory=dict)

    @property
    def device(self):
        return self.ids.device

    def to(self, device) -> "QVB8Pack":
        kw = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in self.__dict__.items()}
        return QVB8Pack(**kw)

    def weight_bytes(self) -> int:
        """Algorithmic bytes one small-M pass must read: payload + 17 B/row metadata + 12 B/escape (fp16 table)."""
        payload = (int(self.nbits.to(torch.int64).sum().item()) * self.P + 7) // 8
        return payload + 17 * self.Q + 12 * int(self.esc_idx.numel())

    def to_blob(self, container: str = "QVBD") -> bytes:
        """Serialise (host side).  The QVBD blob stores the full (bf16-table) escape list."""
        c = lambda t: t.detach().cpu().numpy()
        if container == "QVBD":
            return packs.write_qvbd(Q=self.Q, P=self.P, tau=self.tau, max_err=self.max_err, min_s=c(self.min_s),
                                    tau_s=c(self.tau_s), nbits=c(self.nbits), ids=c(self.ids),
                                    esc_idx=c(self.esc_idx_bf16), esc_vals=c(self.esc_vals_bf16), source="bf16",
                                    restore=self.restore)
        return packs.write_qvb8_legacy(Q=self.Q, P=self.P, tau=self.tau, min_s=c(self.min_s), tau_s=c(self.tau_s),
                                       nbits=c(self.nbits), bit_off=c(self.bit_off), ids=c(self.ids),
                                       esc_idx=c(self.esc_idx), esc_vals=c(self.esc_vals))

    @staticmethod
    def from_parsed(d: dict, device="cpu") -> "QVB8Pack":
        """From the dict :func:`qvb8_b200.packs.read_qvb8` returns."""
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(device)
        ei, ev = t(d["esc_idx"], np.int64), t(d["esc_vals"], np.float32)
        same = d["esc_idx_bf16"] is d["esc_idx"]
        eib, evb = (ei, ev) if same else (t(d["esc_idx_bf16"], np.int64), t(d["esc_vals_bf16"], np.float32))
        return QVB8Pack(Q=d["Q"], P=d["P"], tau=d["tau"], restore=d["restore"], ids=t(d["ids"], np.uint8),
                        min_s=t(d["min_s"], np.float32), tau_s=t(d["tau_s"], np.float32), nbits=t(d["nbits"], np.uint8),
                        bit_off=t(d["bit_off"], np.int64), esc_idx=ei, esc_vals=ev, esc_idx_bf16=eib,
                        esc_vals_bf16=evb, max_err=d.get("max_err", float("nan")))


def band_value(ids: torch.Tensor, tau_s: torch.Tensor, min_s: torch.Tensor) -> torch.Tensor:
    """fma(id, tau_s, min_s) rounded once to fp32.  The product of a <= 14-bit id and an fp32 step and its sum with an
    fp32 origin of similar magnitude are exact in float64, so one narrowing gives the fused result bit for bit."""
    return (ids.to(torch.float64) * tau_s.to(torch.float64)[:, None] + min_s.to(torch.float64)[:, None]).to(torch.float32)


def pack_payload(ids: torch.Tensor, nbits: torch.Tensor, rows_per_chunk: int = 2048) -> tuple[torch.Tensor, torch.Tensor]:
    """Bit-pack (Q, P) integer ids at per-row widths -> (u8[payload + 8], bit_off i64[Q]).  Needs byte-aligned rows
    (nbits * P % 8 == 0 for every row), which holds whenever P % 8 == 0."""
    Q, P = ids.shape
    dev = ids.device
    nb64 = nbits.to(torch.int64)
    row_bits = nb64 * P
    if bool((row_bits % 8 != 0).any()):
        raise ValueError("pack_payload needs byte-aligned rows (use packs.pack_ids on the host for odd P)")
    bit_off = torch.cumsum(row_bits, 0) - row_bits
    total = int(row_bits.sum().item()) // 8
    buf = torch.zeros(total + packs.PAYLOAD_PAD, dtype=torch.uint8, device=dev)
    byte_off = bit_off // 8
    for nb in torch.unique(nb64).tolist():
        rows_all = (nb64 == nb).nonzero().view(-1)
        rb = nb * P // 8
        b = torch.arange(rb, device=dev, dtype=torch.int64)
        f0 = (8 * b) // nb                       # first field touching byte b
        sh = 8 * b - f0 * nb
        K = 8 // nb + 2                          # fields that can touch one byte
        for r0 in range(0, rows_all.numel(), rows_per_chunk):
            rows = rows_all[r0:r0 + rows_per_chunk]
            x = ids[rows].to(torch.int64)
            acc = torch.zeros(rows.numel(), rb, dtype=torch.int64, device=dev)
            for k in range(K):
                f = f0 + k
                ok = f < P
                acc += torch.where(ok[None, :], x[:, f.clamp(max=P - 1)], torch.zeros((), dtype=torch.int64, device=dev)) << (k * nb)
            by = ((acc >> sh[None, :]) & 0xFF).to(torch.uint8)
            dst = byte_off[rows][:, None] + b[None, :]
            buf[dst.reshape(-1)] = by.reshape(-1)
    return buf, bit_off


def encode_qvb8(W: torch.Tensor, tau: float = 1e-3, policy: str = "escape_outliers", restore: str = "fp16",
                outlier_k: float = 6.0, keep_ids: bool = False) -> QVB8Pack:
    """Encode (Q, P) bf16 (or bf16-representable fp32) weights into a QVB8 pack on W's device.

    policy  'escape_outliers'  elements further than outlier_k row standard deviations from the row mean are
                               escaped, the band covers the rest (typical rows: 6-7 bits at tau=1e-3)
            'inband'           the band covers every element that may legally be banded (outliers widen the row)
    """
    if W.dim() != 2:
        raise ValueError("encode_qvb8: W must be (Q, P)")
    if restore not in packs.RESTORE_CODES:
        raise ValueError(f"restore {restore!r}")
    Q, P = W.shape
    dev = W.device
    w = W.to(torch.float32)
    if not torch.equal(w.to(torch.bfloat16).to(torch.float32), w):
        raise ValueError("encode_qvb8: weights must be bf16-representable (the pack stores escapes as bf16 bits)")
    legal = w.abs() <= tau * 2.0 ** FP16_MANTISSA_BITS
    if policy == "escape_outliers":
        mu = w.mean(1, keepdim=True)
        sd = w.std(1, keepdim=True).clamp_min(1e-12)
        inband = legal & ((w - mu).abs() <= outlier_k * sd)
    elif policy == "inband":
        inband = legal
    else:
        raise ValueError(f"policy {policy!r}")
    big = torch.finfo(torch.float32).max
    row_min = torch.where(inband, w, torch.full_like(w, big)).amin(1)
    row_max = torch.where(inband, w, torch.full_like(w, -big)).amax(1)
    empty = row_min > row_max                                 # a row with nothing in band: one bucket at 0
    row_min = torch.where(empty, torch.zeros_like(row_min), row_min)
    row_max = torch.where(empty, torch.zeros_like(row_max), row_max)
    amax = torch.maximum(row_min.abs(), row_max.abs()).clamp_min(2.0 ** -14)
    half_ulp16 = torch.exp2(torch.floor(torch.log2(amax)) - (FP16_MANTISSA_BITS + 1))
    tau_s = (2.0 * (tau - half_ulp16.to(torch.float64)) * (1.0 - 2.0 ** -18)).to(torch.float32)
    if bool((tau_s <= 0).any()):
        raise ValueError("encode_qvb8: tau is below half an fp16 ulp of a row's peak; the row cannot be certified")
    span = (row_max.to(torch.float64) - row_min.to(torch.float64)) / tau_s.to(torch.float64)
    nbuckets = torch.floor(span).to(torch.int64) + 1
    nbits = torch.ceil(torch.log2(nbuckets.to(torch.float64))).to(torch.int64).clamp_min(1)
    nbits = torch.where((1 << nbits) < nbuckets, nbits + 1, nbits)       # guard the float log2
    if int(nbits.max().item()) > packs.MAX_CERTIFIED_NBITS:
        raise ValueError(f"encode_qvb8: a row needs {int(nbits.max())} bits (> {packs.MAX_CERTIFIED_NBITS}); not certifiable")
    top = (1 << nbits) - 1
    ids = torch.floor((w.to(torch.float64) - row_min.to(torch.float64)[:, None]) / tau_s.to(torch.float64)[:, None])
    ids = torch.minimum(ids.clamp_min(0).to(torch.int64), top[:, None]).to(torch.int32)
    min_s = (row_min.to(torch.float64) + tau_s.to(torch.float64) / 2).to(torch.float32)
    band = band_value(ids, tau_s, min_s)
    w64 = w.to(torch.float64)
    err32 = (band.to(torch.float64) - w64).abs()
    err16 = (band.to(torch.float16).to(torch.float64) - w64).abs()
    ok16 = inband & (err16 <= tau) & (err32 <= tau)
    esc16 = ~ok16
    max_err = float(torch.where(ok16, err16, torch.zeros_like(err16)).max().item()) if w.numel() else 0.0
    flat16 = esc16.reshape(-1).nonzero().view(-1)
    wf = w.reshape(-1)
    if restore == "fp16+bf16":
        errb = (band.to(torch.bfloat16).to(torch.float64) - w64).abs()
        escb = esc16 | (errb > tau)
        flatb = escb.reshape(-1).nonzero().view(-1)
        eib, evb = flatb, wf[flatb].contiguous()
        max_err = max(max_err, float(torch.where(~escb, errb, torch.zeros_like(errb)).max().item()))
    buf, bit_off = pack_payload(ids, nbits) if P % 8 == 0 else _pack_payload_host(ids, nbits, dev)
    ei, ev = flat16, wf[flat16].contiguous()
    if restore != "fp16+bf16":
        eib, evb = ei, ev
    nb8 = nbits.to(torch.uint8)
    hist = torch.bincount(nbits, minlength=packs.MAX_CERTIFIED_NBITS + 1).tolist()
    return QVB8Pack(Q=Q, P=P, tau=float(tau), restore=restore, ids=buf, min_s=min_s, tau_s=tau_s, nbits=nb8,
                    bit_off=bit_off, esc_idx=ei, esc_vals=ev, esc_idx_bf16=eib, esc_vals_bf16=evb, max_err=max_err,
                    stats=dict(nbits_hist={b: n for b, n in enumerate(hist) if n}, n_esc=int(ei.numel()),
                               n_esc_bf16=int(eib.numel()), policy=policy, **({"ids": ids} if keep_ids else {})))


def _pack_payload_host(ids, nbits, dev):
    buf = packs.pack_ids(ids.cpu().numpy(), nbits.cpu().numpy())
    off = packs.row_bit_offsets(nbits.cpu().numpy(), ids.shape[1])
    return torch.from_numpy(buf).to(dev), torch.from_numpy(off).to(dev)


def synth_pack(Q: int, P: int, seed: int, tau: float = 1e-3, device="cpu", policy: str = "escape_outliers",
               restore: str = "fp16", return_weight: bool = False):
    """Seeded weights -> pack.  Returns the pack (and the bf16 source weights when return_weight)."""
    W = synth_weight(Q, P, seed, device=device)
    pk = encode_qvb8(W, tau=tau, policy=policy, restore=restore)
    return (pk, W) if return_weight else pk


def reference_dense(pk: QVB8Pack, dtype=torch.float32, table: str | None = None) -> torch.Tensor:
    """Dense (Q, P) restore computed with torch ops on the pack's device: band value rounded once to `dtype`, escapes
    of the matching table written over.  Used for size-independent checks at sizes the CPU oracle cannot reach; it
    needs the unpacked ids, so it re-derives them from the payload with integer ops."""
    Q, P = pk.Q, pk.P
    dev = pk.device
    c = torch.arange(P, device=dev, dtype=torch.int64)
    out = torch.empty(Q, P, dtype=dtype, device=dev)
    nb64 = pk.nbits.to(torch.int64)
    idsb = pk.ids.to(torch.int64)
    step = max(1, (1 << 24) // max(P, 1))
    for r0 in range(0, Q, step):
        r1 = min(Q, r0 + step)
        bit = pk.bit_off[r0:r1, None] + c[None, :] * nb64[r0:r1, None]
        by = bit >> 3
        word = idsb[by] | (idsb[by + 1] << 8) | (idsb[by + 2] << 16) | (idsb[by + 3] << 24)
        idv = (word >> (bit & 7)) & ((1 << nb64[r0:r1, None]) - 1)
        out[r0:r1] = band_value(idv, pk.tau_s[r0:r1], pk.min_s[r0:r1]).to(dtype)
    if table is None:
        table = "bf16" if dtype == torch.bfloat16 else "fp16"
    ei, ev = (pk.esc_idx_bf16, pk.esc_vals_bf16) if table == "bf16" else (pk.esc_idx, pk.esc_vals)
    if ei.numel():
        out.view(-1)[ei] = ev.to(dtype)
    return out


def encode_qvb8r(W: torch.Tensor, tau: float = 2e-3, K: int = 2, T: int | None = None,
                 policy: str = "escape_outliers") -> dict:
    """Encode (Q, P) weights into the arrays of a ``.qvb8r`` file (numpy, host): the QVB8 band of every row, its ids
    entropy-coded by :mod:`qvb8_b200.rans`, the escapes with their exact value and the stored difference
    ``exact - band`` the escape pass adds.  T (rows per tile) defaults to ceil(Q / 4096)."""
    from . import rans
    pk = encode_qvb8(W, tau=tau, policy=policy, keep_ids=True)
    ids = pk.stats.pop("ids").cpu().numpy().astype(np.int64)
    Q, P = ids.shape
    enc = rans.encode_ids(ids, K=K, T=T if T is not None else max(1, -(-Q // 4096)))
    ei = pk.esc_idx.cpu().numpy()
    ev = pk.esc_vals.cpu().numpy()
    rows = ei // P
    # fma(id, tau_s, min_s) of the escaped positions: exact in float64, one narrowing (see band_value)
    band = (ids.reshape(-1)[ei].astype(np.float64) * pk.tau_s.cpu().numpy().astype(np.float64)[rows]
            + pk.min_s.cpu().numpy().astype(np.float64)[rows]).astype(np.float32)
    enc.update(Q=Q, P=P, min_s=pk.min_s.cpu().numpy(), tau_s=pk.tau_s.cpu().numpy(), esc_idx=ei, esc_val=ev,
               esc_delta=(ev.astype(np.float32) - band).astype(np.float32),
               tau=float(tau), max_err=pk.max_err)
    return enc
