"""Generates the QVB8R golden fixtures of this folder with the REFERENCE's own code.

    python oracle/build_ref.py qvb8r_cuda            # once: compiles the reference's qvb8r extension into oracle/_ref
    PYTHONPATH=<reference>/src python tests/golden/make_golden_qvb8r.py

Every byte and number stored here comes out of reference code: the symbols of a seeded tensor are entropy-coded by the
reference's C++ ``encode`` (qvb8r_cpu.cpp:60-110), written by ``container.write`` (formats/qvb8r/container.py:30-49),
read back by ``container.read`` (:52-71), turned into runtime tables by ``runtime_tables`` / ``blocks_for`` /
``codec.slot_tables`` (:74-89, codec.py:11-20) and decoded by the reference's C++ ``embed_rows``
(qvb8r_cpu.cpp:13-58).  Only the coding MODEL (row order, classes, frequency tables, centring, tile height) is this
repository's: the reference release has no writer, and its reader accepts any model.

Each case is one ``.npz``:
    blob        the .qvb8r file bytes (uint8), as container.write produced them
    ids         (Q, P) int16   every id in ORIGINAL row order: embed_rows with min_s = 0, tau_s = 1 (ids below 2048 are
                               exact in fp32) and the file's drow
    sym         (Q, P) int16   the same with drow = 0: the raw symbols
    tab         (K, 4096) u32  codec.slot_tables(freq)
    blocks8, blocks16          container.blocks_for(tiles, 8 / 16)
    embed_f32   (Q, P) f32     embed_rows with the file's min_s / tau_s / drow and escapes: the reference's embedding
                               values (mul then add, qvb8r_cpu.cpp:44), escapes written over
    cert_json                  the certification record passed to container.write (so the file can be re-made)
"""
from __future__ import annotations

import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)

from qvb8_b200 import rans, synth  # noqa: E402
from oracle import build_ref  # noqa: E402

CASES = [
    # name, Q, P, seed, tau, K, T
    ("qvb8r_40x256_k2_t4", 40, 256, 21, 2e-3, 2, 4),
    ("qvb8r_72x384_k3_t8", 72, 384, 22, 2e-3, 3, 8),
    ("qvb8r_33x128_k1_t16", 33, 128, 23, 1e-3, 1, 16),
    ("qvb8r_96x512_k4_t2", 96, 512, 24, 5e-3, 4, 2),
]


def embed_all(refext, d, tab, tiles, words, off, *, min_s, tau_s, drow, escapes: bool):
    """reference embed_rows over every row, tensors built as QVBandEmbeddingV8R.__init__ does (module.py:345-372)"""
    Q, P = int(d["Q"]), int(d["P"])
    inv = np.empty(Q, np.int32)
    inv[d["perm"]] = np.arange(Q, dtype=np.int32)
    row_tile = np.empty(Q, np.int32)
    for t, (_, r0, nr) in enumerate(tiles):
        row_tile[r0:r0 + nr] = t
    ei = d["esc_idx"].astype(np.int64) if escapes else np.zeros(0, np.int64)
    ev = np.asarray(d["esc_val"], np.float32) if escapes else np.zeros(0, np.float32)
    er = ei // P
    o = np.argsort(er, kind="stable")
    ptr = np.zeros(Q + 1, np.int64)
    np.add.at(ptr, er + 1, 1)
    ptr = np.cumsum(ptr)
    C = lambda a: torch.from_numpy(np.array(a, copy=True, order="C"))
    rows = torch.arange(Q, dtype=torch.int64)
    out = refext.embed_rows(rows, C(words.view(np.int32)), C(off), C(d["states"].view(np.int64)), C(tiles),
                            C(tab.view(np.int32)), C(inv), C(row_tile), C(min_s.astype(np.float32)),
                            C(tau_s.astype(np.float32)), C(drow.astype(np.int32)), C(ptr),
                            C((ei % P)[o].astype(np.int32)), C(ev[o]), P)
    return out.numpy()


def main() -> None:
    from qv_band.formats.qvb8r import container as QF
    from qv_band.formats.qvb8r.codec import slot_tables

    refext = build_ref.load("qvb8r_cuda")
    if refext is None:
        raise SystemExit("oracle/_ref/qvb8r_cuda.so is missing: run oracle/build_ref.py first")
    for name, Q, P, seed, tau, K, T in CASES:
        W = synth.synth_weight(Q, P, seed)
        pk = synth.encode_qvb8(W, tau=tau, policy="escape_outliers", keep_ids=True)
        ids = pk.stats.pop("ids").cpu().numpy().astype(np.int64)
        m = rans.model_for(ids, K=K, T=T)
        sym = m.pop("sym")
        F = m["freq"].astype(np.int64)
        Cum = np.cumsum(F, 1) - F
        words, off, states = refext.encode(torch.from_numpy(np.ascontiguousarray(sym[m["perm"]].astype(np.int16))),
                                           torch.from_numpy(m["tiles"].astype(np.int64)), torch.from_numpy(F),
                                           torch.from_numpy(np.ascontiguousarray(Cum)))
        enc = dict(m, words=words.numpy().view(np.uint32), tile_off=off.numpy().astype(np.uint32),
                   states=states.numpy().view(np.uint64))
        ei = pk.esc_idx.numpy()
        ev = pk.esc_vals.numpy()
        min_s, tau_s = pk.min_s.numpy(), pk.tau_s.numpy()
        band = (ids.reshape(-1)[ei].astype(np.float64) * tau_s.astype(np.float64)[ei // P]
                + min_s.astype(np.float64)[ei // P]).astype(np.float32)
        cert = dict(tau=float(tau), max_err=float(pk.max_err), restore="fp16")
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, name + ".qvb8r")
            QF.write(path, enc, Q, P, min_s, tau_s, ei, ev, (ev - band).astype(np.float32), cert)
            blob = open(path, "rb").read()
        d = QF.read(blob=blob)
        tab, tiles, wpad, toff = QF.runtime_tables(d)
        assert np.array_equal(tab, slot_tables(d["freq"]))
        zero, one = np.zeros(Q, np.float32), np.ones(Q, np.float32)
        symo = embed_all(refext, d, tab, tiles, wpad, toff, min_s=zero, tau_s=one, drow=np.zeros(Q, np.int32), escapes=False)
        idso = embed_all(refext, d, tab, tiles, wpad, toff, min_s=zero, tau_s=one, drow=d["drow"], escapes=False)
        emb = embed_all(refext, d, tab, tiles, wpad, toff, min_s=d["min_s"], tau_s=d["tau_s"], drow=d["drow"], escapes=True)
        assert np.array_equal(idso.astype(np.int64), ids), "the reference decoder did not return the coded ids"
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), blob=np.frombuffer(blob, np.uint8), ids=idso.astype(np.int16),
            sym=symo.astype(np.int16), tab=tab.astype(np.uint32), blocks8=QF.blocks_for(tiles, 8),
            blocks16=QF.blocks_for(tiles, 16), embed_f32=emb.astype(np.float32),
            cert_json=np.frombuffer(json.dumps(cert).encode(), np.uint8))
        print(f"{name}: Q={Q} P={P} K={K} T={T} tiles={len(tiles)} words={d['words'].size} "
              f"bits/weight={d['words'].size * 32 / (Q * P):.2f} escapes={ei.size} file={len(blob)} B")


if __name__ == "__main__":
    main()
