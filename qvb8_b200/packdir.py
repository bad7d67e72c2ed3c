"""Pack directory: one file per tensor plus ``manifest.json``, the layout the reference's loaders walk.

Reference: the manifest keys its code reads are ``format`` (``qvb8`` / ``qvband`` / ``qvb8r``), ``tau``,
``tensors{name: {pack, Q, P, bytes, restore}}`` (+ ``max_err`` per the README), ``failed``, ``hf_model``
(run/run_inference.py:554-568, 581-589; run/placement.py:92-107); a tensor's file is
``re.sub('[^A-Za-z0-9]', '_', name) + '.' + format`` (common/formats.py:45-48); the slices of a stacked expert tensor
are keyed ``<base>#expert<e:03d>`` (common/expert_key.py:18).  This module writes and reads that layout and builds the
modules of this package from it; everything here is load-time host code.
"""
from __future__ import annotations

import json
import os

import torch

from . import packs

EXPERT_KEY_SEP = "#expert"
FORMATS = ("qvb8", "qvband", "qvb8r")


def expert_key(base: str, e: int) -> str:
    """Manifest key of expert `e` of a stacked expert tensor."""
    return f"{base}{EXPERT_KEY_SEP}{int(e):03d}"


def split_expert_key(name: str):
    """(base, e) of an expert key, (name, None) for any other tensor."""
    if EXPERT_KEY_SEP in name:
        base, _, e = name.rpartition(EXPERT_KEY_SEP)
        if e.isdigit():
            return base, int(e)
    return name, None


def write_pack_dir(folder: str, tensors: dict, *, fmt: str = "qvb8", tau: float, hf_model: str | None = None,
                   failed: list | None = None) -> dict:
    """tensors: name -> :class:`qvb8_b200.synth.QVB8Pack` (fmt qvb8 / qvband) or a parsed ``.qvb8r`` dict (fmt qvb8r).
    Writes one file per tensor and the manifest; returns the manifest."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown pack format {fmt!r}")
    os.makedirs(folder, exist_ok=True)
    entries = {}
    for name, t in tensors.items():
        fname = packs.pack_filename(name, fmt)
        if fmt == "qvb8r":
            blob = packs.write_qvb8r(t, Q=t["Q"], P=t["P"], min_s=t["min_s"], tau_s=t["tau_s"], esc_idx=t["esc_idx"],
                                     esc_val=t["esc_val"], esc_delta=t["esc_delta"],
                                     cert=dict(tau=t.get("tau", tau), max_err=t.get("max_err", 0.0)))
            Q, P, restore, max_err = int(t["Q"]), int(t["P"]), "fp16", float(t.get("max_err", 0.0))
        else:
            blob = t.to_blob("QVBD")
            Q, P, restore, max_err = int(t.Q), int(t.P), t.restore, float(t.max_err)
        with open(os.path.join(folder, fname), "wb") as f:
            f.write(blob)
        entries[name] = {"pack": fname, "Q": Q, "P": P, "bytes": len(blob), "restore": restore, "max_err": max_err}
    manifest = {"format": fmt, "tau": float(tau), "tensors": entries, "failed": list(failed or [])}
    if hf_model:
        manifest["hf_model"] = hf_model
    with open(os.path.join(folder, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    return manifest


def read_manifest(folder: str) -> dict:
    """The manifest of a pack directory, checked for the keys the loaders rely on."""
    path = os.path.join(folder, "manifest.json")
    with open(path) as f:
        m = json.load(f)
    if m.get("format") not in FORMATS:
        raise packs.PackFormatError(f"{path}: format {m.get('format')!r} is not one of {FORMATS}")
    if not isinstance(m.get("tensors"), dict):
        raise packs.PackFormatError(f"{path}: no tensors table")
    for name, e in m["tensors"].items():
        for k in ("pack", "Q", "P"):
            if k not in e:
                raise packs.PackFormatError(f"{path}: tensor {name!r} lacks {k!r}")
        if e["pack"] != packs.pack_filename(name, m["format"]) and not os.path.exists(os.path.join(folder, e["pack"])):
            raise packs.PackFormatError(f"{path}: tensor {name!r} points to a missing file {e['pack']!r}")
    m.setdefault("failed", [])
    return m


def load_linear(folder: str, name: str, *, bias=None, device: str = "cuda", manifest: dict | None = None,
                shard: tuple | None = None, group=None):
    """The module of tensor `name`: QVBandLinearV8 for qvb8 / qvband packs, QVBandLinearV8R for qvb8r.

    shard = (rank, world, cut): only this rank's share is built and uploaded -- the whole file is parsed on the host,
    the shard is cut from its bytes there (nothing is re-encoded), and the device never sees the rest.  cut "rows":
    output rows [rank Q / world, (rank + 1) Q / world) (the bias is sliced with them); cut "cols": input columns
    [rank P / world, ...) of every row (a partial product: the bias stays with rank 0).  A qvb8r tensor has one cut,
    runs of whole tiles (``QVBandLinearV8RShard``, which all-gathers the ranks' rows over `group`)."""
    m = manifest or read_manifest(folder)
    if name not in m["tensors"]:
        raise KeyError(f"{name!r} is not in the manifest of {folder}" + (" (listed as failed)" if name in m["failed"] else ""))
    e = m["tensors"][name]
    path = os.path.join(folder, e["pack"])
    if shard is not None:
        rank, world, cut = int(shard[0]), int(shard[1]), (shard[2] if len(shard) > 2 else "rows")
        if not (0 <= rank < world) or cut not in ("rows", "cols"):
            raise ValueError("shard = (rank, world, 'rows' | 'cols') with 0 <= rank < world")
    if m["format"] == "qvb8r":
        from .linear_r import QVBandLinearV8R, QVBandLinearV8RShard
        if shard is not None and world > 1:
            with open(path, "rb") as fh:
                d = packs.read_qvb8r(fh.read(), str(path))
            if (int(d["Q"]), int(d["P"])) != (int(e["Q"]), int(e["P"])):
                raise packs.PackFormatError(f"{path}: shape {(d['Q'], d['P'])} differs from the manifest's {(e['Q'], e['P'])}")
            return QVBandLinearV8RShard(d, rank, world, bias=bias, device=device, group=group)
        mod = QVBandLinearV8R.from_packfile(path, bias=bias, device=device)
    else:
        from .linear import QVBandLinearV8
        if shard is not None and world > 1:
            from . import fuse
            from .synth import QVB8Pack
            with open(path, "rb") as fh:
                d = packs.read_qvb8(fh.read(), str(path))
            if (int(d["Q"]), int(d["P"])) != (int(e["Q"]), int(e["P"])):
                raise packs.PackFormatError(f"{path}: shape {(d['Q'], d['P'])} differs from the manifest's {(e['Q'], e['P'])}")
            packs.validate_pack(d, str(path))
            whole = QVB8Pack.from_parsed(d, device="cpu")
            Q, P = whole.Q, whole.P
            b = None if bias is None else torch.as_tensor(bias).detach()
            if cut == "rows":
                if Q % world:
                    raise ValueError(f"{name}: {Q} rows do not split over {world} ranks")
                r0, r1 = rank * (Q // world), (rank + 1) * (Q // world)
                part = fuse.row_shard(whole, r0, r1)
                b = None if b is None else b[r0:r1]
            else:
                if P % (8 * world):
                    raise ValueError(f"{name}: {P} columns do not split over {world} ranks in 8-column units")
                part = fuse.column_shard(whole, rank * (P // world), (rank + 1) * (P // world))
                b = b if rank == 0 else None
            mod = QVBandLinearV8.from_pack(part.to(device), bias=None if b is None else b.to(device))
            mod.fp16_table_missing = bool(d.get("fp16_table_missing", False))
            mod._where = f"{path} [{cut} shard {rank} of {world}]"
            return mod
        mod = QVBandLinearV8.from_packfile(path, bias=bias, device=device)
    if (mod.out_features, mod.in_features) != (int(e["Q"]), int(e["P"])):
        raise packs.PackFormatError(f"{path}: shape {(mod.out_features, mod.in_features)} differs from the manifest's {(e['Q'], e['P'])}")
    return mod


def expert_slices(manifest: dict, base: str) -> list[str]:
    """The manifest keys of the experts of stacked tensor `base`, in expert order (without gaps)."""
    found = {}
    for name in manifest["tensors"]:
        b, e = split_expert_key(name)
        if b == base and e is not None:
            found[e] = name
    if sorted(found) != list(range(len(found))):
        raise packs.PackFormatError(f"experts of {base!r} are not numbered 0..{len(found) - 1}")
    return [found[e] for e in range(len(found))]
