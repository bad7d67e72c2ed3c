"""Helpers shared by the tests: hand-made packs with arbitrary row widths, upload, comparisons."""
from __future__ import annotations

import numpy as np
import torch

from qvb8_b200 import packs, synth


def random_pack(Q, P, widths, seed, esc_frac=0.0, device="cpu") -> synth.QVB8Pack:
    """A pack with random ids: row widths drawn from `widths`, random origins/steps, `esc_frac` of the elements
    escaped with random exact values.  Not certified against any source weight -- it exercises the decoders."""
    rng = np.random.default_rng(seed)
    nbits = rng.choice(np.asarray(widths), size=Q).astype(np.int64)
    ids = (rng.integers(0, 1 << 30, size=(Q, P)) & ((1 << nbits)[:, None] - 1)).astype(np.int64)
    tau_s = (rng.uniform(1e-3, 3e-3, Q)).astype(np.float32)
    min_s = (-(2.0 ** (nbits - 1)) * tau_s * rng.uniform(0.8, 1.2, Q)).astype(np.float32)
    buf = packs.pack_ids(ids, nbits)
    bit_off = packs.row_bit_offsets(nbits, P)
    n_esc = int(round(esc_frac * Q * P))
    esc_idx = np.sort(rng.choice(Q * P, size=n_esc, replace=False)).astype(np.int64) if n_esc else np.zeros(0, np.int64)
    esc_vals = torch.from_numpy(rng.standard_normal(n_esc).astype(np.float32) * 0.3).to(torch.bfloat16).float().numpy()
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(device)
    ei, ev = t(esc_idx, np.int64), t(esc_vals, np.float32)
    return synth.QVB8Pack(Q=Q, P=P, tau=1e-3, restore="fp16", ids=t(buf, np.uint8), min_s=t(min_s, np.float32),
                          tau_s=t(tau_s, np.float32), nbits=t(nbits, np.uint8), bit_off=t(bit_off, np.int64),
                          esc_idx=ei, esc_vals=ev, esc_idx_bf16=ei, esc_vals_bf16=ev)


def pack_np(pk: synth.QVB8Pack) -> dict:
    """The numpy dict form the oracle takes."""
    c = lambda t: t.detach().cpu().numpy()
    return dict(Q=pk.Q, P=pk.P, ids=c(pk.ids), nbits=c(pk.nbits), bit_off=c(pk.bit_off), min_s=c(pk.min_s),
                tau_s=c(pk.tau_s), esc_idx=c(pk.esc_idx), esc_vals=c(pk.esc_vals), esc_idx_bf16=c(pk.esc_idx_bf16),
                esc_vals_bf16=c(pk.esc_vals_bf16))


def ext_args(pk: synth.QVB8Pack, table="fp16"):
    """Positional arguments (after X) of the reference-style entry points."""
    ei, ev = (pk.esc_idx_bf16, pk.esc_vals_bf16) if table == "bf16" else (pk.esc_idx, pk.esc_vals)
    return (pk.ids, pk.min_s, pk.nbits, pk.bit_off, pk.P, pk.tau_s, ei, ev)


def rel_fro(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)
