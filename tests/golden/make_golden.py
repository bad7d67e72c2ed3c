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


if __name__ == "__main__":
    main()
