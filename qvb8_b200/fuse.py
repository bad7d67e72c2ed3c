"""Same-input fusion for QVB8: sibling linears that read the same activation (q/k/v, gate/up) run as ONE launch.

The reference does this for its entropy-coded format (formats/qvb8r/fuse.py:1-60: the members' data is concatenated
into one virtual tensor, every kernel path runs unchanged on it, the output is split back per member).  A QVB8 pack
concatenates even more simply, because its rows are independent: the bit-packed rows are laid back to back, the
per-row vectors are concatenated, row bit offsets are shifted by the bits that precede them, and escape positions
by the rows that precede them.  Each row's weights, band and escapes are the same bytes; the fused output equals the
members' outputs side by side bit for bit whenever the launches cut K into the same ranges (a taller pack may be given
fewer K-ranges, which changes the order of the fp32 partial sums and nothing else).
"""
from __future__ import annotations

import torch

from . import packs
from .synth import QVB8Pack


def concat_packs(members: list[QVB8Pack]) -> tuple[QVB8Pack, list[int]]:
    """One pack holding the rows of `members` in order.  Returns (pack, row split points for torch.tensor_split)."""
    if not members:
        raise ValueError("concat_packs: no members")
    P = members[0].P
    dev = members[0].device
    for m in members:
        if m.P != P:
            raise ValueError("concat_packs: members must share P (they read the same activation)")
        if m.device != dev:
            raise ValueError("concat_packs: members must live on one device")
        if m.restore != members[0].restore:
            raise ValueError("concat_packs: members must share the restore code")
    pad = packs.PAYLOAD_PAD
    ids, bit_off, e_idx, e_val, e_idx16, e_val16 = [], [], [], [], [], []
    bits = 0
    rows = 0
    for m in members:
        payload = m.ids[:m.ids.numel() - pad]
        if (bits % 8) or int(m.bit_off[0].item()) != 0:
            raise ValueError("concat_packs: member payloads must be byte-aligned and start at bit 0")
        ids.append(payload)
        bit_off.append(m.bit_off + bits)
        e_idx.append(m.esc_idx + rows * P)
        e_val.append(m.esc_vals)
        e_idx16.append(m.esc_idx_bf16 + rows * P)
        e_val16.append(m.esc_vals_bf16)
        bits += payload.numel() * 8
        rows += m.Q
    ids.append(torch.zeros(pad, dtype=torch.uint8, device=dev))
    hist: dict = {}
    for m in members:
        for b, n in m.stats.get("nbits_hist", {}).items():
            hist[b] = hist.get(b, 0) + n
    same_table = all(m.esc_idx_bf16 is m.esc_idx for m in members)
    esc_idx, esc_vals = torch.cat(e_idx), torch.cat(e_val)
    fused = QVB8Pack(
        Q=rows, P=P, tau=max(m.tau for m in members), restore=members[0].restore, ids=torch.cat(ids),
        min_s=torch.cat([m.min_s for m in members]), tau_s=torch.cat([m.tau_s for m in members]),
        nbits=torch.cat([m.nbits for m in members]), bit_off=torch.cat(bit_off), esc_idx=esc_idx, esc_vals=esc_vals,
        esc_idx_bf16=esc_idx if same_table else torch.cat(e_idx16),
        esc_vals_bf16=esc_vals if same_table else torch.cat(e_val16),
        max_err=max(m.max_err for m in members), stats={"nbits_hist": hist, "members": [m.Q for m in members]})
    splits, acc = [], 0
    for m in members[:-1]:
        acc += m.Q
        splits.append(acc)
    return fused, splits


def row_shard(pk: QVB8Pack, r0: int, r1: int) -> QVB8Pack:
    """The pack of output rows [r0, r1) of `pk`, made from its bytes: rows of a pack are independent (own origin, step,
    width and bit range), so a shard is a slice of the four per-row vectors, the byte range of those rows, and the
    escapes that fall into them renumbered.  Nothing is re-encoded: the shard restores to exactly rows [r0, r1) of
    the whole.  (The reference slices rows the same way, formats/qvb8/module.py:126-160.)"""
    if not 0 <= r0 < r1 <= pk.Q:
        raise ValueError(f"row_shard: rows [{r0}, {r1}) of {pk.Q}")
    bits = pk.nbits.to(torch.int64) * pk.P
    first_bit = int(pk.bit_off[r0].item())
    last_bit = int(pk.bit_off[r1 - 1].item()) + int(bits[r1 - 1].item())
    if first_bit % 8 or (last_bit % 8 and r1 != pk.Q):
        raise ValueError("row_shard: the rows do not start and end on byte boundaries (P * nbits must be a multiple of 8)")
    payload = pk.ids[first_bit // 8:(last_bit + 7) // 8]
    ids = torch.cat([payload, torch.zeros(packs.PAYLOAD_PAD, dtype=torch.uint8, device=pk.device)])

    def esc(idx, vals):
        keep = (idx >= r0 * pk.P) & (idx < r1 * pk.P)
        return idx[keep] - r0 * pk.P, vals[keep]
    ei, ev = esc(pk.esc_idx, pk.esc_vals)
    same = pk.esc_idx_bf16 is pk.esc_idx
    eib, evb = (ei, ev) if same else esc(pk.esc_idx_bf16, pk.esc_vals_bf16)
    nb = pk.nbits[r0:r1]
    hist = {int(b): int(n) for b, n in zip(*torch.unique(nb, return_counts=True))}
    return QVB8Pack(Q=r1 - r0, P=pk.P, tau=pk.tau, restore=pk.restore, ids=ids, min_s=pk.min_s[r0:r1].contiguous(),
                    tau_s=pk.tau_s[r0:r1].contiguous(), nbits=nb.contiguous(),
                    bit_off=(pk.bit_off[r0:r1] - first_bit).contiguous(), esc_idx=ei, esc_vals=ev, esc_idx_bf16=eib,
                    esc_vals_bf16=evb, max_err=pk.max_err, stats={"nbits_hist": hist})


def column_shard(pk: QVB8Pack, c0: int, c1: int) -> QVB8Pack:
    """The pack of input columns [c0, c1) of every row of `pk`, made from its bytes -- the shard a row-parallel
    (input-split) linear needs when a deployment holds only the pack, not the source weight.  A row's ids are a bit
    string of nbits * P bits; columns [c0, c1) are the bits [c0 * nbits, c1 * nbits) of it, which are whole bytes for
    every width when c0 and c1 are multiples of 8.  Origins and steps are unchanged, escapes inside the range are
    renumbered: the shard restores to exactly those columns of the whole, so the ranks' partial products add up to the
    unsharded product."""
    P, Q, dev = pk.P, pk.Q, pk.device
    if not (0 <= c0 < c1 <= P) or c0 % 8 or c1 % 8:
        raise ValueError(f"column_shard: columns [{c0}, {c1}) of {P} must be multiples of 8")
    if bool((pk.bit_off % 8 != 0).any()):
        raise ValueError("column_shard: rows must start on byte boundaries (P * nbits a multiple of 8)")
    nb = pk.nbits.to(torch.int64)
    width = c1 - c0
    row_bytes = nb * (width // 8)                                        # bytes of the slice, per row
    src0 = pk.bit_off // 8 + nb * (c0 // 8)                              # first source byte, per row
    dst0 = torch.cumsum(row_bytes, 0) - row_bytes                        # first destination byte, per row
    total = int(row_bytes.sum().item())
    row_of = torch.repeat_interleave(torch.arange(Q, device=dev), row_bytes)
    within = torch.arange(total, device=dev) - dst0[row_of]
    payload = pk.ids[src0[row_of] + within]
    ids = torch.cat([payload, torch.zeros(packs.PAYLOAD_PAD, dtype=torch.uint8, device=dev)])

    def esc(idx, vals):
        q, c = torch.div(idx, P, rounding_mode="floor"), torch.remainder(idx, P)
        keep = (c >= c0) & (c < c1)
        return q[keep] * width + (c[keep] - c0), vals[keep]
    ei, ev = esc(pk.esc_idx, pk.esc_vals)
    same = pk.esc_idx_bf16 is pk.esc_idx
    eib, evb = (ei, ev) if same else esc(pk.esc_idx_bf16, pk.esc_vals_bf16)
    return QVB8Pack(Q=Q, P=width, tau=pk.tau, restore=pk.restore, ids=ids, min_s=pk.min_s, tau_s=pk.tau_s, nbits=pk.nbits,
                    bit_off=(dst0 * 8).contiguous(), esc_idx=ei, esc_vals=ev, esc_idx_bf16=eib, esc_vals_bf16=evb,
                    max_err=pk.max_err, stats=dict(pk.stats))


# (group name, member names) of a decoder layer whose members are fed the same tensor
SAME_INPUT_GROUPS = (("qkv", ("q", "k", "v")), ("gate_up", ("gate", "up")))


def concat_qvb8r(members: list[dict]) -> tuple[dict, list[int]]:
    """Same-input fusion for the entropy-coded format (reference formats/qvb8r/fuse.py:18-119): the members' parsed
    ``.qvb8r`` dicts become ONE dict with the same keys.  Tiles keep their streams and states; only the bookkeeping
    is shifted: a member's classes follow the previous members' classes (frequency tables stacked, padded to the
    widest alphabet), its sorted rows and output rows follow theirs (`tiles[:, 1]`, `perm`, escape indices), its word
    offsets follow their words.  Every kernel path and :class:`qvb8_b200.linear_r.QVBandLinearV8R` run unchanged on
    the result; a row's symbols, band and escapes are the same bytes, so the output is the members' outputs side by
    side.  Returns (dict, row split points)."""
    import numpy as np
    if not members:
        raise ValueError("concat_qvb8r: no members")
    P = int(members[0]["P"])
    if any(int(m["P"]) != P for m in members):
        raise ValueError("concat_qvb8r: members must share P (they read the same activation)")
    N = max(int(np.asarray(m["freq"]).shape[1]) for m in members)
    out = {k: [] for k in ("perm", "freq", "tiles", "tile_off", "states", "words", "drow", "min_s", "tau_s",
                           "esc_idx", "esc_val", "esc_delta")}
    q0 = k0 = w0 = 0
    for m in members:
        Q = int(m["Q"])
        f = np.asarray(m["freq"])
        out["freq"].append(np.pad(f, ((0, 0), (0, N - f.shape[1]))))
        t = np.asarray(m["tiles"], np.int64).reshape(-1, 3).copy()
        t[:, 0] += k0
        t[:, 1] += q0
        out["tiles"].append(t)
        off = np.asarray(m["tile_off"], np.int64)
        out["tile_off"].append(off[:-1] + w0)
        out["states"].append(np.asarray(m["states"], np.uint64).reshape(-1, 32))
        out["words"].append(np.asarray(m["words"], np.uint32))
        out["perm"].append(np.asarray(m["perm"], np.int64) + q0)
        for k in ("drow", "min_s", "tau_s", "esc_val", "esc_delta"):
            out[k].append(np.asarray(m[k]))
        out["esc_idx"].append(np.asarray(m["esc_idx"], np.int64) + q0 * P)
        q0 += Q
        k0 += f.shape[0]
        w0 += int(off[-1])
    cat = lambda k, dt: np.concatenate(out[k]).astype(dt)
    first = members[0]
    fused = dict(
        Q=q0, P=P, K=k0, N=N, T=max(int(m["T"]) for m in members),
        perm=cat("perm", np.int32), freq=cat("freq", np.asarray(first["freq"]).dtype), tiles=cat("tiles", np.int32),
        tile_off=np.concatenate(out["tile_off"] + [np.asarray([w0], np.int64)]).astype(np.asarray(first["tile_off"]).dtype),
        states=cat("states", np.uint64), words=cat("words", np.uint32), drow=cat("drow", np.asarray(first["drow"]).dtype),
        min_s=cat("min_s", np.float32), tau_s=cat("tau_s", np.float32), esc_idx=cat("esc_idx", np.int64),
        esc_val=cat("esc_val", np.float32), esc_delta=cat("esc_delta", np.float32),
        tau=max(float(m.get("tau", 0.0)) for m in members), max_err=max(float(m.get("max_err", 0.0)) for m in members))
    splits, acc = [], 0
    for m in members[:-1]:
        acc += int(m["Q"])
        splits.append(acc)
    return fused, splits


def qvb8r_shard_bounds(d: dict, world: int) -> list[int]:
    """Tile boundaries t[0] = 0 <= t[1] <= ... <= t[world] = tiles that split an entropy-coded tensor into `world` runs of
    whole tiles with about the same number of coded words each (a rank's time is its decoder's time)."""
    import numpy as np
    off = np.asarray(d["tile_off"], np.int64)
    nt = off.size - 1
    total = int(off[-1])
    cuts = [0]
    for r in range(1, world):
        t = int(np.searchsorted(off, total * r / world, side="left"))
        cuts.append(min(nt, max(cuts[-1], t)))
    return cuts + [nt]


def qvb8r_tile_shard(d: dict, t0: int, t1: int) -> tuple[dict, "np.ndarray"]:
    """Tiles [t0, t1) of a parsed ``.qvb8r`` tensor as a tensor of its own, made from the file's arrays without
    re-encoding: rANS streams run per tile, so a rank can hold a contiguous run of tiles (their words, states and word
    offsets), the class tables, and the per-row metadata and escapes of the rows those tiles code.  A QVB8R tensor cannot
    be cut by columns (a stream is sequential along the row) and not by arbitrary rows either (tiles hold the rows in
    the coder's sorted order), so tiles are the unit -- the output rows of a shard are scattered over the whole tensor.

    Returns (dict, rows): the dict has the same keys as the parsed file, with the shard's rows numbered 0 .. Q' - 1 in the
    coder's sorted order; rows[i] is the row of the whole tensor that the shard's output row i is.  The whole product is
    ``y[..., rows_r] = y_r`` over the shards r."""
    import numpy as np
    tiles = np.asarray(d["tiles"], np.int64).reshape(-1, 3)
    if not (0 <= t0 <= t1 <= tiles.shape[0]):
        raise ValueError("qvb8r_tile_shard: tile range outside the tensor")
    P = int(d["P"])
    off = np.asarray(d["tile_off"], np.int64)
    perm = np.asarray(d["perm"], np.int64)
    if t0 == t1:
        r0 = r1 = 0
    else:
        r0 = int(tiles[t0, 1])
        r1 = int(tiles[t1 - 1, 1] + tiles[t1 - 1, 2])
    rows = perm[r0:r1]                                         # sorted position r0 + i -> row of the whole tensor
    local = np.full(int(d["Q"]), -1, np.int64)
    local[rows] = np.arange(rows.size)
    sub = tiles[t0:t1].copy()
    sub[:, 1] -= r0
    ei = np.asarray(d["esc_idx"], np.int64)
    mine = local[ei // P] >= 0 if ei.size else np.zeros(0, bool)
    new_idx = local[ei[mine] // P] * P + ei[mine] % P
    order = np.argsort(new_idx, kind="stable")
    first = d
    shard = dict(
        Q=int(rows.size), P=P, K=int(d["K"]), N=int(d["N"]), T=int(d["T"]),
        perm=np.arange(rows.size, dtype=np.int32), freq=np.asarray(d["freq"]),
        tiles=sub.astype(np.int32), tile_off=(off[t0:t1 + 1] - off[t0]).astype(np.asarray(first["tile_off"]).dtype),
        states=np.asarray(d["states"], np.uint64).reshape(-1, 32)[t0:t1].copy(),
        words=np.asarray(d["words"], np.uint32)[int(off[t0]):int(off[t1])].copy(),
        drow=np.asarray(d["drow"])[rows], min_s=np.asarray(d["min_s"], np.float32)[rows],
        tau_s=np.asarray(d["tau_s"], np.float32)[rows],
        esc_idx=new_idx[order], esc_val=np.asarray(d["esc_val"], np.float32)[mine][order],
        esc_delta=np.asarray(d["esc_delta"], np.float32)[mine][order],
        tau=float(d.get("tau", 0.0)), max_err=float(d.get("max_err", 0.0)))
    return shard, rows

