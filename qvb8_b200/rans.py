"""QVB8R (entropy-coded QVB8): a seeded synthetic encoder and the tables a reader builds at load.

The reference ships only the READER of this format (formats/qvb8r/codec.py:1 "the pack writer / calibration is not
included"; its C++ ``encode`` is the inverse walk of ``embed_rows``, qvb8r_cpu.cpp:60-110).  This module restates the
writer from the reader's contract so that seeded packs exist to test and time the kernels on:

  stream  a tile = `rows` consecutive sorted rows of one class, 32 interleaved 64-bit rANS states; state j codes
          column 32 * step + j; symbols go in pairs; after a lane decoded two symbols a state below 2^32 takes the
          tile's next 32-bit word, lanes in ascending order (qvb8r_cuda.cu:36-75, qvb8r_cpu.cpp:13-58)
  symbol  s = id - drow[row] in [0, N), N <= 2048; rows are coded centred: drow places the row's median id at CENTRE
          (codec.py:4-9)
  model   K classes of rows, one frequency table per class, sum 4096, every frequency <= 1024 (it is stored as F - 1
          in 10 bits of the slot entry, codec.py:11-20)

The encoder runs the decoder backwards: rows, step pairs and lanes in reverse; before coding a pair (F1, F2) a state
x >= (F1 * F2) << 40 emits its low 32 bits (exactly the states the decoder refills after that pair).
"""
from __future__ import annotations

import numpy as np

PB = 12
MQ = 1 << PB
MAX_ID = 2048
MAX_FREQ = 1024
CENTRE = 256
PAD_WORDS = 2048


def slot_tables(freq: np.ndarray) -> np.ndarray:
    """(K, N) frequencies -> (K, 4096) slot entries ``symbol | offset << 11 | (F - 1) << 22`` (codec.py:11-20)."""
    F = np.asarray(freq, np.int64)
    K, N = F.shape
    tab = np.zeros((K, MQ), np.uint32)
    for k in range(K):
        if int(F[k].sum()) != MQ or int(F[k].max()) > MAX_FREQ:
            raise ValueError("frequencies of a class must sum to 4096 with every entry <= 1024")
        sym = np.repeat(np.arange(N, dtype=np.int64), F[k])
        start = np.cumsum(F[k]) - F[k]
        tab[k] = (sym | ((np.arange(MQ, dtype=np.int64) - start[sym]) << 11) | ((F[k][sym] - 1) << 22)).astype(np.uint32)
    return tab


def quantise_freq(hist: np.ndarray) -> np.ndarray:
    """Symbol counts -> frequencies that sum to 4096, >= 1 for every symbol that occurs, <= 1024 for all."""
    h = np.asarray(hist, np.float64)
    present = h > 0
    if not present.any():
        raise ValueError("empty histogram")
    f = np.zeros(h.shape, np.int64)
    f[present] = np.clip(np.floor(h[present] / h.sum() * MQ), 1, MAX_FREQ).astype(np.int64)
    # hand the rounding remainder out (or take it back) one count at a time, largest symbols first
    order = np.argsort(-h, kind="stable")
    diff = MQ - int(f.sum())
    guard = 0
    while diff != 0:
        moved = False
        for s in order:
            if diff == 0:
                break
            if not present[s]:
                continue
            if diff > 0 and f[s] < MAX_FREQ:
                f[s] += 1; diff -= 1; moved = True
            elif diff < 0 and f[s] > 1:
                f[s] -= 1; diff += 1; moved = True
        guard += 1
        if not moved or guard > MQ:
            raise ValueError("cannot quantise: too few distinct symbols for a 1024 cap (needs >= 4 present symbols)")
    return f


def blocks_for(tiles: np.ndarray, tiles_per_block: int) -> np.ndarray:
    """The launch schedule of a tile table: (class, first tile, ntiles) per block, a block being at most
    `tiles_per_block` consecutive tiles of ONE class -- the eight (sixteen) tiles of a CTA share the class's slot
    table in shared memory (the reference derives the same schedule at load, container.py:74-82).  Computed from the
    class column alone: a new block starts where the class changes or where the running length within a class run
    reaches a multiple of `tiles_per_block`."""
    cls = np.asarray(tiles, np.int64).reshape(-1, 3)[:, 0]
    n = cls.size
    if n == 0:
        return np.zeros((0, 3), np.int32)
    change = np.flatnonzero(np.diff(cls)) + 1                  # first tile of every class run but the first
    run_start = np.concatenate([[0], change])
    run_len = np.diff(np.concatenate([run_start, [n]]))
    firsts, counts = [], []
    for s0, ln in zip(run_start.tolist(), run_len.tolist()):
        starts = np.arange(s0, s0 + ln, tiles_per_block)
        firsts.append(starts)
        counts.append(np.minimum(tiles_per_block, s0 + ln - starts))
    first = np.concatenate(firsts)
    return np.stack([cls[first], first, np.concatenate(counts)], axis=1).astype(np.int32)


def encode_symbols(sym: np.ndarray, tile_class: np.ndarray, tile_rows: np.ndarray, freq: np.ndarray):
    """rANS-code `sym` (rows in SORTED order, (R, P) ints in [0, N)) tile by tile.

    tile_class[t], tile_rows[t]: class and row count of tile t (tiles cover the rows in order).
    Returns (states u64 (nt, 32), words u32, tile_off u32 (nt + 1))."""
    sym = np.asarray(sym, np.int64)
    R, P = sym.shape
    if P % 64:
        raise ValueError("P must be a multiple of 64 (32 lanes, symbols in pairs)")
    F = np.asarray(freq, np.int64)
    C = np.cumsum(F, 1) - F
    nt = len(tile_rows)
    first = np.concatenate([[0], np.cumsum(tile_rows)[:-1]]).astype(np.int64)
    x = np.full((nt, 32), 1 << 32, np.uint64)              # the decoder's state after its last pair
    maxr = int(np.max(tile_rows))
    S2 = P // 64
    cls = np.asarray(tile_class, np.int64)
    trows = np.asarray(tile_rows, np.int64)
    lanes = np.arange(32)
    # every (row, pair) step of the backward walk leaves, per tile and lane, a flag "emitted a word" and the word; the
    # stream of a tile is those words with the steps in DECODING order (the reverse of this loop) and the lanes ascending
    steps = maxr * S2
    flags = np.zeros((steps, nt, 32), bool)
    lows = np.zeros((steps, nt, 32), np.uint32)
    k = 0
    for r in range(maxr - 1, -1, -1):
        act = np.nonzero(trows > r)[0]                     # tiles that have a row r
        rows = first[act] + r
        kk = cls[act][:, None]
        srow = sym[rows]
        for sp in range(S2 - 1, -1, -1):
            s0 = srow[:, (2 * sp) * 32 + lanes]            # first symbol of the pair per lane
            s1 = srow[:, (2 * sp + 1) * 32 + lanes]
            f0, f1 = F[kk, s0], F[kk, s1]
            if (f0 == 0).any() or (f1 == 0).any():
                raise ValueError("a coded symbol has frequency 0 in its class")
            xa = x[act]
            emit = xa >= ((f0 * f1).astype(np.uint64) << np.uint64(40))
            flags[k, act] = emit
            lows[k, act] = (xa & np.uint64(0xFFFFFFFF)).astype(np.uint32)
            xa = np.where(emit, xa >> np.uint64(32), xa)
            # decoder order inside a lane: symbol 0 then symbol 1 -> encode symbol 1 first
            for f, c in ((f1, C[kk, s1]), (f0, C[kk, s0])):
                fu = f.astype(np.uint64)
                xa = ((xa // fu) << np.uint64(PB)) + (xa % fu) + c.astype(np.uint64)
            x[act] = xa
            k += 1
    flags = flags[::-1].transpose(1, 0, 2)                 # (tile, decoding step, lane)
    lows = lows[::-1].transpose(1, 0, 2)
    words = lows[flags].astype(np.uint32)                  # tiles in order, steps in decoding order, lanes ascending
    tile_off = np.concatenate([[0], np.cumsum(flags.reshape(nt, -1).sum(1))]).astype(np.uint32)
    return x, words, tile_off


def model_for(ids: np.ndarray, K: int = 2, T: int = 8) -> dict:
    """The coding model of integer ids (Q, P) (each row >= 0): rows centred (drow), classed into K groups by their
    spread, sorted by class (perm), cut into tiles of <= T rows, one quantised frequency table per class.  Returns
    sym (Q, P) symbols in ORIGINAL row order, perm, freq, tiles, drow, T, K, N.  The reference does not ship this
    step (its writer is not in the release, codec.py:1); any model its reader accepts is a valid file."""
    ids = np.asarray(ids, np.int64)
    Q, P = ids.shape
    med = np.median(ids, axis=1).astype(np.int64)
    drow = med - CENTRE                                    # symbol = id - drow puts the median at CENTRE
    low = (ids - drow[:, None]).min(axis=1)
    drow = drow + np.minimum(low, 0)                       # no negative symbols
    sym = ids - drow[:, None]
    N = int(sym.max()) + 1
    if N > MAX_ID:
        raise ValueError(f"symbols span {N} > {MAX_ID}")
    spread = sym.std(axis=1)
    order = np.argsort(spread, kind="stable")
    cls_of_row = np.zeros(Q, np.int64)
    for k, part in enumerate(np.array_split(order, K)):
        cls_of_row[part] = k
    perm = np.argsort(cls_of_row, kind="stable").astype(np.int32)      # sorted position -> original row
    freq = np.zeros((K, N), np.int64)
    for k in range(K):
        rows = np.nonzero(cls_of_row == k)[0]
        if rows.size:
            freq[k] = quantise_freq(np.bincount(sym[rows].ravel(), minlength=N))
        else:
            freq[k, :4] = MAX_FREQ                          # an empty class still needs a valid table
    sorted_cls = cls_of_row[perm]
    # tiles: every class run cut into pieces of T rows
    bounds = np.concatenate([[0], np.flatnonzero(np.diff(sorted_cls)) + 1, [Q]])
    tiles = [(int(sorted_cls[a0]), int(p0), int(min(T, a1 - p0)))
             for a0, a1 in zip(bounds[:-1], bounds[1:]) for p0 in range(a0, a1, T)]
    tiles = np.asarray(tiles, np.int32).reshape(-1, 3)
    return dict(sym=sym, perm=perm, freq=freq.astype(np.uint16), tiles=tiles, drow=drow.astype(np.int16), T=int(T),
                K=int(K), N=int(N))


def encode_ids(ids: np.ndarray, K: int = 2, T: int = 8, seed: int = 0) -> dict:
    """Entropy-code integer ids (Q, P): :func:`model_for`, then :func:`encode_symbols` over the sorted rows.  Returns
    the container arrays (perm, freq, tiles, tile_off, states, words, drow, T, K, N)."""
    m = model_for(ids, K=K, T=T)
    sym = m.pop("sym")
    states, words, tile_off = encode_symbols(sym[m["perm"]], m["tiles"][:, 0], m["tiles"][:, 2], m["freq"])
    m.update(tile_off=tile_off, states=states, words=words)
    return m
