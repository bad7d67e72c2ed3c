"""Greedy head: the device argmax (largest value, lowest index among equals, NaNs passed over), the winner among the
ranks' candidates, and a head split by vocabulary rows against one argmax over all the logits."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qvb8_b200 import synth
from qvb8_b200.lm_head import GreedyHead, pick_best

DEV = "cuda:0"


def test_pick_best_prefers_value_then_lower_token():
    vals = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, 2.0], [3.0, 4.0, -1.0]])
    toks = torch.tensor([[7, 40, 9], [30, 12, 3], [11, 5, 1]])
    best, tok = pick_best(vals, toks)
    assert best.tolist() == [3.0, 5.0, 2.0]
    assert tok.tolist() == [11, 12, 3]                     # ties: the lower token index


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(3)
        logits = torch.randn(5, 96, generator=g)
        logits[2, 10] = logits[2, 70] = 9.0               # a tie across two ranks' slices
        per = 96 // world
        mine = logits[:, rank * per:(rank + 1) * per]
        val, idx = mine.max(dim=1)                         # (torch.max returns the first of equal values)
        vals = torch.empty(world * 5)
        toks = torch.empty(world * 5, dtype=torch.int64)
        dist.all_gather_into_tensor(vals, val.contiguous())
        dist.all_gather_into_tensor(toks, (idx + rank * per).contiguous())
        _, tok = pick_best(vals.view(world, -1), toks.view(world, -1))
        np.save(os.path.join(out_dir, f"tok_{rank}.npy"), tok.numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ranks_agree_with_one_argmax(tmp_path):
    world = 3
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(5, 96, generator=g)
    logits[2, 10] = logits[2, 70] = 9.0
    want = logits.argmax(dim=1).numpy()
    assert want[2] == 10
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"tok_{r}.npy"), want)


@pytest.mark.gpu
def test_device_argmax(cuda_lib):
    from qvb8_b200 import lib
    g = torch.Generator().manual_seed(1)
    for M, V in ((1, 151936), (7, 32000), (3, 5), (2, 1)):
        Y = torch.randn(M, V, generator=g).to(DEV)
        if V > 4:
            Y[0, 3] = Y[0, V - 1] = 50.0                   # equal maxima: the lower index
            Y[M - 1, 1] = float("nan")
        val, idx = lib.argmax_rows(Y, index_base=1000)
        ref = torch.where(torch.isnan(Y), torch.full_like(Y, -float("inf")), Y)
        assert torch.equal(idx, ref.argmax(dim=1) + 1000)
        assert torch.equal(val, ref.max(dim=1).values)
        if V > 4:
            assert int(idx[0]) == 1003
    nan_row = torch.full((1, 64), float("nan"), device=DEV)
    val, idx = lib.argmax_rows(nan_row, index_base=5)
    assert int(idx[0]) == 5 and float(val[0]) == -float("inf")
    sub = torch.randn(4, 100, generator=g).to(DEV)[:, 10:60]   # rows further apart than they are long
    val, idx = lib.argmax_rows(sub)
    assert torch.equal(idx, sub.argmax(dim=1))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 6])
def test_head_split_by_vocabulary_rows(cuda_lib, M):
    """three shards of a packed head on one device: their candidates, combined, are the tokens of the whole head"""
    from qvb8_b200 import fuse
    from qvb8_b200.linear import QVBandLinearV8
    V, P = 3000, 512
    pk = synth.synth_pack(V, P, seed=8, device=DEV)
    x = synth.synth_activation(M, P, seed=M, device=DEV, dtype=torch.float32)   # fp32 logits: no ties from rounding
    whole = GreedyHead(QVBandLinearV8.from_pack(pk))
    want = whole(x)
    logits = QVBandLinearV8.from_pack(pk)(x).float()
    assert torch.equal(want, logits.argmax(dim=-1))
    cands = []
    for r in range(3):
        head = GreedyHead(QVBandLinearV8.from_pack(fuse.row_shard(pk, r * 1000, (r + 1) * 1000)), first_row=r * 1000)
        cands.append(head.local_best(x))
    _, tok = pick_best(torch.stack([c[0] for c in cands]), torch.stack([c[1] for c in cands]))
    assert torch.equal(tok, want)
