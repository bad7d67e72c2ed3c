"""The N > 1 path on CPU: two gloo ranks, each holding its row shard of every projection (column-parallel split by
output rows, the split the reference's row_subset exploits, formats/qvb8/module.py:126-160), compute their shard of
the product with the oracle and all-gather it; the result must be the unsharded product, bit for bit."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from qvb8_b200 import synth
from util import pack_np


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Q, P, M = 96, 256, 3
        W = synth.synth_weight(Q, P, 4242)                     # same seed on every rank, as the stack does
        X = synth.synth_activation(M, P, seed=7)
        Qr = Q // world
        shard = synth.encode_qvb8(W[rank * Qr:(rank + 1) * Qr], tau=1e-3)
        y = torch.from_numpy(oracle.matmul_f32w(X.float().numpy(), oracle.qvb8_dense(pack_np(shard)), narrow_x=True))
        gathered = torch.empty(world * M, Qr, dtype=y.dtype)      # rank-major concatenation
        dist.all_gather_into_tensor(gathered, y.contiguous())
        if rank == 0:
            np.save(os.path.join(out_dir, "y.npy"), gathered.view(world, M, Qr).permute(1, 0, 2).reshape(M, Q).numpy())
        # row-parallel: each rank holds a column slice of every row as a pack of its own, multiplies its slice of X
        # and the partial sums are all-reduced
        Pr = P // world
        cshard = synth.encode_qvb8(W[:, rank * Pr:(rank + 1) * Pr].contiguous(), tau=1e-3)
        Wc = oracle.qvb8_dense(pack_np(cshard))
        yp = torch.from_numpy(oracle.matmul_f32w(X[:, rank * Pr:(rank + 1) * Pr].float().numpy(), Wc, narrow_x=True))
        dist.all_reduce(yp)
        parts = [torch.empty_like(torch.from_numpy(Wc)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(Wc))
        if rank == 0:
            np.save(os.path.join(out_dir, "y_row.npy"), yp.numpy())
            np.save(os.path.join(out_dir, "w_row.npy"), torch.cat(parts, dim=1).numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_row_sharded_product_equals_the_whole(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "y.npy")
    Q, P, M = 96, 256, 3
    full = synth.encode_qvb8(synth.synth_weight(Q, P, 4242), tau=1e-3)
    X = synth.synth_activation(M, P, seed=7)
    want = oracle.matmul_f32w(X.float().numpy(), oracle.qvb8_dense(pack_np(full)), narrow_x=True)
    assert got.dtype == want.dtype and np.array_equal(got, want)
    # row-parallel shards: the all-reduced partial sums are the product with the shards' restored weights side by side,
    # and every restored weight is within tau of the source
    y_row, w_row = np.load(tmp_path / "y_row.npy"), np.load(tmp_path / "w_row.npy")
    want_row = oracle.matmul_f32w(X.float().numpy(), w_row, narrow_x=True)
    assert np.allclose(y_row, want_row, rtol=1e-9, atol=1e-9)
    assert float(np.abs(w_row - synth.synth_weight(Q, P, 4242).float().numpy()).max()) <= 1e-3


def _expert_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, topk, P, hidden, M = 4, 2, 64, 16, 5
        per = E // world
        # every rank builds only ITS experts (seeded by the global expert number) and sees all tokens and the routing
        ups = [synth.encode_qvb8(synth.synth_weight(2 * hidden, P, 300 + e), tau=1e-3, policy="inband")
               for e in range(rank * per, (rank + 1) * per)]
        dns = [synth.encode_qvb8(synth.synth_weight(P, hidden, 400 + e), tau=1e-3, policy="inband")
               for e in range(rank * per, (rank + 1) * per)]
        g = torch.Generator().manual_seed(1)
        wts, idx = torch.topk(torch.softmax(torch.randn(M, E, generator=g), -1), topk, dim=-1)
        X = synth.synth_activation(M, P, seed=2).float().numpy()
        local = idx - rank * per                               # what the sharded module hands to the kernels
        mine = (local >= 0) & (local < per)                    # pairs outside the local stack contribute zero
        part = oracle.moe_experts(X, torch.where(mine, local, torch.zeros_like(local)).numpy(),
                                  (wts * mine).numpy(), np.stack([oracle.qvb8_dense(pack_np(u)) for u in ups]),
                                  np.stack([oracle.qvb8_dense(pack_np(d)) for d in dns]))
        t = torch.from_numpy(part)
        dist.all_reduce(t)
        if rank == 0:
            np.save(os.path.join(out_dir, "moe.npy"), t.numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_partial_sums_equal_the_whole_layer(tmp_path):
    world = 2
    mp.spawn(_expert_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    E, topk, P, hidden, M = 4, 2, 64, 16, 5
    ups = [synth.encode_qvb8(synth.synth_weight(2 * hidden, P, 300 + e), tau=1e-3, policy="inband") for e in range(E)]
    dns = [synth.encode_qvb8(synth.synth_weight(P, hidden, 400 + e), tau=1e-3, policy="inband") for e in range(E)]
    g = torch.Generator().manual_seed(1)
    wts, idx = torch.topk(torch.softmax(torch.randn(M, E, generator=g), -1), topk, dim=-1)
    X = synth.synth_activation(M, P, seed=2).float().numpy()
    want = oracle.moe_experts(X, idx.numpy(), wts.numpy(), np.stack([oracle.qvb8_dense(pack_np(u)) for u in ups]),
                              np.stack([oracle.qvb8_dense(pack_np(d)) for d in dns]))
    assert np.allclose(np.load(tmp_path / "moe.npy"), want, rtol=1e-12, atol=1e-12)


def _qvb8r_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qvb8_b200 import fuse
        from qvb8_b200.linear_r import gather_rows
        Q, P, M = 150, 128, 3
        d = synth.encode_qvb8r(synth.synth_weight(Q, P, 77), tau=2e-3, K=3, T=4)       # every rank reads the whole file
        bounds = fuse.qvb8r_shard_bounds(d, world)
        shards = [fuse.qvb8r_tile_shard(d, bounds[r], bounds[r + 1]) for r in range(world)]
        mine, rows = shards[rank]
        X = synth.synth_activation(M, P, seed=5).float().numpy()
        y = torch.from_numpy(oracle.matmul_f32w(X, oracle.qvb8r_dense(mine), narrow_x=True)) if mine["Q"] else \
            torch.zeros(M, 0, dtype=torch.float64)
        pad = max(len(r) for _, r in shards)
        place = np.full((world, pad), Q, np.int64)
        for r, (_, rr) in enumerate(shards):
            place[r, :len(rr)] = rr
        out = gather_rows(y, torch.from_numpy(place.reshape(-1)), pad, world, Q, dist.group.WORLD)
        np.save(os.path.join(out_dir, f"qvb8r_{rank}.npy"), out.numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_qvb8r_tile_shards_gathered_equal_the_whole(tmp_path):
    """an entropy-coded tensor split by tiles over three ranks: every rank's product rows, gathered and put in place,
    are the whole product bit for bit on every rank (rows are decoded from the same words)"""
    world = 3
    mp.spawn(_qvb8r_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    Q, P, M = 150, 128, 3
    d = synth.encode_qvb8r(synth.synth_weight(Q, P, 77), tau=2e-3, K=3, T=4)
    X = synth.synth_activation(M, P, seed=5).float().numpy()
    want = oracle.matmul_f32w(X, oracle.qvb8r_dense(d), narrow_x=True)
    for r in range(world):
        got = np.load(tmp_path / f"qvb8r_{r}.npy")
        assert got.dtype == want.dtype and np.array_equal(got, want)


def test_row_subset_of_a_module_is_the_rows_of_the_whole():
    """The zero-copy shard: a module over a subset of rows shares the packed ids and restores to those rows."""
    from qvb8_b200.linear import QVBandLinearV8
    pk = synth.encode_qvb8(synth.synth_weight(64, 256, 99), tau=1e-3)
    lin = QVBandLinearV8.from_pack(pk) if hasattr(QVBandLinearV8, "from_pack") else None
    if lin is None:
        import pytest
        pytest.skip("no from_pack constructor")
    rows = torch.arange(16, 48)
    sub = lin.row_subset(rows)
    d = dict(Q=32, P=256, ids=sub.ids.numpy(), nbits=sub.nbits.numpy(), bit_off=sub.bit_off.numpy(),
             min_s=sub.min_s.numpy(), tau_s=sub.tau_s.numpy(), esc_idx=sub.esc_idx.numpy(), esc_vals=sub.esc_vals.numpy(),
             esc_idx_bf16=sub.esc_idx_bf16.numpy(), esc_vals_bf16=sub.esc_vals_bf16.numpy())
    want = oracle.qvb8_dense(pack_np(pk))[16:48]
    assert np.array_equal(oracle.qvb8_dense(d).view(np.uint32), want.view(np.uint32))


def _peer_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qvb8_b200.peer import PeerAllReduce
        outcome = "no error"
        try:
            PeerAllReduce(dist.group.WORLD, 1024, "cpu")
        except RuntimeError as e:
            outcome = "RuntimeError: " + str(e)[:60]
        with open(os.path.join(out_dir, f"peer_{rank}.txt"), "w") as f:
            f.write(outcome)
        dist.barrier()                                   # still in step with the other rank after the failure
    finally:
        dist.destroy_process_group()


def test_peer_communicator_fails_on_all_ranks_together(tmp_path):
    """Without a CUDA device no rank can allocate its exchange area: every rank must raise (none may be left waiting
    in a collective), and the group stays usable afterwards."""
    world = 2
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"peer_{r}.txt").read_text().startswith("RuntimeError")
