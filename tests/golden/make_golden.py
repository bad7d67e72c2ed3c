"""Generates the golden fixtures of this folder by running the REFERENCE's own decoders.

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

The reference ships no tests or known-answer vectors for the QVB8 path, so the pins are produced here: seeded packs
are written in the reference's byte layout, parsed and restored by the reference's Python decoder
(qv_band.formats.qvb8.pack_container.unpack_formula / decode.unpack_tensor, decode.unpack_bits_rows,
decode.reconstruct), and the results are stored next to the pack bytes.  The test-suite then checks the CPU oracle
and the CUDA kernels against these files without needing the reference.

Each case is one ``.npz``:
    blob        the pack file bytes (uint8)
    ids         (Q, P) uint16  ids as the reference unpacks them
    w32         (Q, P) float32 reference reconstruct(...) with the pack's full escape list
    w16_bits    (Q, P) uint16  w32 narrowed by numpy to float16 (bit pattern)
    wbf_bits    (Q, P) uint16  w32 narrowed by torch to bfloat16 (bit pattern)
    source_bits (Q, P) uint16  the bf16 weights the pack was made from (bit pattern)

One more file, ``escpool_32x256.npz``, pins the two escape pools and the escape-table selection: a bf16-certified pack
whose escapes are split between the full-width pool and the FP8 (E4M3 code + row scale) pool, read by the reference's
``unpack_formula`` together with an ``escape_tables.json`` that the reference's ``fp16_list_for`` / ``select_fp16``
interpret (formats/qvb8/decode.py:104-161, escape_split.py:14-54):
    blob, tables_json   the pack bytes and the JSON text (uint8)
    esc_idx / esc_vals              the merged list the reference returns (ascending)
    esc_idx_fp16 / esc_vals_fp16    the reference's fp16 table
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from qvb8_b200 import synth  # noqa: E402

CASES = [
    # name, Q, P, seed, tau, policy, restore, container
    ("qvbd_48x256_escout", 48, 256, 11, 1e-3, "escape_outliers", "fp16", "QVBD"),
    ("qvbd_40x384_inband", 40, 384, 12, 1e-3, "inband", "fp16", "QVBD"),
    ("qvbd_33x128_tau5e3", 33, 128, 13, 5e-3, "escape_outliers", "fp16", "QVBD"),
    ("qvbd_24x256_bf16cert", 24, 256, 14, 2e-3, "escape_outliers", "fp16+bf16", "QVBD"),
    ("legacy_32x256", 32, 256, 15, 1e-3, "escape_outliers", "fp16", "QVB8"),
    ("qvbd_20x136_oddP", 20, 136, 16, 1e-3, "escape_outliers", "fp16", "QVBD"),
]


def main() -> None:
    from qv_band.formats.qvb8 import decode as D
    from qv_band.formats.qvb8 import pack_container as PC

    for name, Q, P, seed, tau, policy, restore, container in CASES:
        pk, W = synth.synth_pack(Q, P, seed, tau=tau, policy=policy, restore=restore, return_weight=True)
        blob = pk.to_blob(container)
        if container == "QVBD":
            d = PC.unpack_formula(blob)
            ids = d["codes"]
            w32 = D.reconstruct(d["min_s"], d["tau_s"], ids, d["esc_idx"], d["esc_vals"])
            assert abs(d["max_err"] - pk.max_err) < 1e-9
        else:
            (min_s, tau_s, nbits, bit_off, buf, q_, p_, _tau, esc_idx, esc_vals) = D.unpack_tensor(blob)
            ids = D.unpack_bits_rows(buf, nbits, bit_off, q_, p_)
            w32 = D.reconstruct(min_s, tau_s, ids, esc_idx, esc_vals)
        src = W.float().numpy()
        # the pack certifies: fp16(restore) within tau of the source at every element, escapes included
        assert np.abs(w32.astype(np.float16).astype(np.float64) - src.astype(np.float64)).max() <= tau
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            blob=np.frombuffer(blob, np.uint8),
            ids=ids.astype(np.uint16),
            w32=w32.astype(np.float32),
            w16_bits=w32.astype(np.float16).view(np.uint16),
            wbf_bits=torch.from_numpy(w32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16),
            source_bits=W.view(torch.int16).numpy().view(np.uint16),
        )
        print(f"{name}: Q={Q} P={P} nbits={pk.stats['nbits_hist']} escapes={pk.stats['n_esc']}/{pk.stats['n_esc_bf16']}"
              f" max_err={pk.max_err:.3e} blob={len(blob)} B")


def escape_pool_case() -> None:
    import tempfile
    from qv_band.formats.qvb8 import escape_split as ES
    from qv_band.formats.qvb8 import pack_container as PC
    from qvb8_b200 import packs

    Q, P = 32, 256
    pk = synth.synth_pack(Q, P, 31, tau=2e-3, policy="escape_outliers", restore="fp16+bf16")
    c = lambda t: t.detach().cpu().numpy()
    ei, ev = c(pk.esc_idx_bf16), c(pk.esc_vals_bf16)
    rng = np.random.default_rng(31)
    to8 = rng.random(ei.size) < 0.5                          # these go to the FP8 pool
    lut = packs.e4m3_table()
    s8 = np.ones(Q, np.float32)
    rows8 = ei[to8] // P
    for q in np.unique(rows8):
        s8[q] = np.abs(ev[to8][rows8 == q]).max() / 448.0
    grid = lut[:127]                                         # finite positive codes
    mag = np.abs(ev[to8]) / s8[rows8]
    codes = np.abs(mag[:, None] - grid[None, :]).argmin(1).astype(np.uint8) | np.where(ev[to8] < 0, 0x80, 0).astype(np.uint8)
    blob = packs.write_qvbd(Q=Q, P=P, tau=pk.tau, max_err=pk.max_err, min_s=c(pk.min_s), tau_s=c(pk.tau_s),
                            nbits=c(pk.nbits), ids=c(pk.ids), esc_idx=ei[~to8], esc_vals=ev[~to8], source="bf16",
                            restore="fp16+bf16", fp8_idx=ei[to8], fp8_codes=codes, fp8_scale=s8)
    keep = rng.random(ei.size) < 0.3                         # the fp16 table: a subset of all escapes
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "layer_w.qvb8")
        with open(path, "wb") as fh:
            fh.write(blob)
        packs.write_escape_tables(tmp, {"layer_w.qvb8": (ei, keep)})
        tables = open(os.path.join(tmp, packs.ESCAPE_TABLES_FILE), "rb").read()
        lst = ES.fp16_list_for(path)
        d = PC.unpack_formula(blob, fp16_list=lst, where=path)
    assert d["esc_idx"].size == ei.size and d["esc_idx_fp16"].size == int(keep.sum())
    np.savez_compressed(os.path.join(HERE, "escpool_32x256.npz"), blob=np.frombuffer(blob, np.uint8),
                        tables_json=np.frombuffer(tables, np.uint8), esc_idx=d["esc_idx"], esc_vals=d["esc_vals"],
                        esc_idx_fp16=d["esc_idx_fp16"], esc_vals_fp16=d["esc_vals_fp16"])
    print(f"escpool_32x256: {ei.size} escapes, {int(to8.sum())} in the FP8 pool, fp16 table {int(keep.sum())}")


if __name__ == "__main__":
    main()
    escape_pool_case()
