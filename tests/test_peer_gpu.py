"""The push all-reduce on ONE GPU: all ranks of a small world in one cooperative launch (block r = rank r), and the
bounded wait made to run out (a flag that nothing sets) with the status word read back and cleared.  Separate launches
that wait on one another are never put on one GPU."""
import ctypes

import numpy as np
import pytest
import torch

from qvb8_b200 import lib as _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _areas(L, world, cap):
    nbytes = int(L.qvb8_peer_bytes(world, cap))
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    epochs = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(world)]
    return areas, epochs


def _ptrs(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


@pytest.mark.parametrize("world", [2, 4])
def test_all_ranks_in_one_cooperative_launch(cuda_lib, world):
    L = cuda_lib
    n, cap = 4096, 8192
    areas, epochs = _areas(L, world, cap)
    g = torch.Generator().manual_seed(world)
    for step in range(3):                                              # epochs alternate between the two buffers
        parts = [torch.randn(n, generator=g).to(DEV) for _ in range(world)]
        outs = [torch.empty(n, device=DEV) for _ in range(world)]
        with torch.cuda.device(DEV):
            _lib.check(L.qvb8_peer_allreduce_local(_ptrs(areas), world, cap, _ptrs(epochs), _ptrs(parts), _ptrs(outs), n,
                                                   0, _lib.stream_ptr(torch.device(DEV))), "qvb8_peer_allreduce_local")
        torch.cuda.synchronize()
        want = parts[0].clone()
        for p in parts[1:]:
            want += p                                                  # rank order, as the kernel adds
        for o in outs:
            assert torch.equal(o, want)                                # bit-identical on every rank
        assert all(int(e.item()) == step + 1 for e in epochs)
    assert _lib.device_status(DEV) == 0


@pytest.mark.parametrize("world", [2, 8])
def test_all_gather_in_one_cooperative_launch(cuda_lib, world):
    L = cuda_lib
    n, cap = 1536, 2048
    areas, epochs = _areas(L, world, cap)
    g = torch.Generator().manual_seed(10 + world)
    for step in range(3):
        parts = [torch.randn(n, generator=g).to(DEV) for _ in range(world)]
        outs = [torch.empty(world * n, device=DEV) for _ in range(world)]
        with torch.cuda.device(DEV):
            _lib.check(L.qvb8_peer_allgather_local(_ptrs(areas), world, cap, _ptrs(epochs), _ptrs(parts), _ptrs(outs), n,
                                                   0, _lib.stream_ptr(torch.device(DEV))), "qvb8_peer_allgather_local")
        torch.cuda.synchronize()
        want = torch.cat(parts)
        for o in outs:
            assert torch.equal(o, want)
    assert _lib.device_status(DEV) == 0


def test_in_place_reduction(cuda_lib):
    L = cuda_lib
    world, n, cap = 2, 1024, 1024
    areas, epochs = _areas(L, world, cap)
    parts = [torch.full((n,), float(r + 1), device=DEV) for r in range(world)]
    with torch.cuda.device(DEV):
        _lib.check(L.qvb8_peer_allreduce_local(_ptrs(areas), world, cap, _ptrs(epochs), _ptrs(parts), _ptrs(parts), n, 0,
                                               _lib.stream_ptr(torch.device(DEV))), "qvb8_peer_allreduce_local")
    torch.cuda.synchronize()
    assert all(bool((p == 3.0).all()) for p in parts)


def test_wait_for_an_absent_peer_runs_out(cuda_lib):
    """rank 0 of a world of two, alone: its wait for rank 1's flag (which nothing sets) ends after the given limit, the
    kernel returns, the status word says 31 and the context stays usable"""
    L = cuda_lib
    world, n, cap = 2, 256, 256
    areas, epochs = _areas(L, world, cap)
    part = torch.ones(n, device=DEV)
    out = torch.empty(n, device=DEV)
    assert _lib.device_status(DEV) == 0
    with torch.cuda.device(DEV):
        _lib.check(L.qvb8_peer_allreduce_ex(_ptrs(areas), 0, world, cap, epochs[0].data_ptr(), part.data_ptr(),
                                            out.data_ptr(), n, 0, 2_000_000, _lib.stream_ptr(torch.device(DEV))),
                   "qvb8_peer_allreduce_ex")
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 31
    assert bool((out == 1.0).all())                                    # what it had: its own part plus the empty slot
    _lib.check(L.qvb8_device_status_reset(), "qvb8_device_status_reset")
    assert _lib.device_status(DEV) == 0
    assert float((part * 2).sum()) == 2.0 * n                          # the context still computes


def test_multi_block_exchange_in_one_process(cuda_lib):
    """a vector long enough to be cut into many blocks, rank 0 and rank 1 of a world of two as two launches that do
    NOT wait on one another: each rank's call is made with the peer's slices and flags already in place (written here
    by a helper call of the peer rank into scratch areas), so no launch ever waits for a later one"""
    L = cuda_lib
    world, n, cap = 2, 131072, 131072
    areas, epochs = _areas(L, world, cap)
    g = torch.Generator().manual_seed(5)
    parts = [torch.randn(n, generator=g).to(DEV) for _ in range(world)]
    outs = [torch.empty(n, device=DEV) for _ in range(world)]
    # rank 1 first: its wait for rank 0's flags runs out after 1 ms (nothing has set them yet) -- but its pushes and
    # flags are now in both areas; then rank 0 finds everything it waits for and returns the full sum
    with torch.cuda.device(DEV):
        _lib.check(L.qvb8_peer_allreduce_ex(_ptrs(areas), 1, world, cap, epochs[1].data_ptr(), parts[1].data_ptr(),
                                            outs[1].data_ptr(), n, 0, 1_000_000, _lib.stream_ptr(torch.device(DEV))), "rank 1")
        torch.cuda.synchronize()
        assert _lib.device_status(DEV) == 31
        _lib.check(L.qvb8_device_status_reset(), "reset")
        _lib.check(L.qvb8_peer_allreduce_ex(_ptrs(areas), 0, world, cap, epochs[0].data_ptr(), parts[0].data_ptr(),
                                            outs[0].data_ptr(), n, 0, 0, _lib.stream_ptr(torch.device(DEV))), "rank 0")
    torch.cuda.synchronize()
    assert _lib.device_status(DEV) == 0
    assert torch.equal(outs[0], parts[0] + parts[1])
    assert int(epochs[0].item()) == 1 and int(epochs[1].item()) == 1
