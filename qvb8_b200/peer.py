"""All-reduce of the row-parallel projections' partial sums over NVLink peer memory (one node, one process per GPU).

The reference exchanges at the shard boundary of a split linear with NCCL (run/placement.py places the row subsets of
formats/qvb8/module.py:126-160 on the cards).  For decode the exchanged vector is a few tens of kilobytes, so a library
all-reduce costs its latency (measured here: 13 - 19 us each inside a captured graph); the kernel behind
:class:`PeerAllReduce` pushes the partial sums straight into the peers' memory and costs a few microseconds.

The exchange areas are plain ``cudaMalloc`` memory shared through CUDA IPC handles, which travel over the existing
process group (``all_gather_object``).  No multicast objects are used.
"""
from __future__ import annotations

import ctypes

import torch

from . import lib as _lib


class PeerAllReduce:
    """`cap_floats`: the largest number of floats one call may reduce.  Every rank must construct it collectively and
    then issue the same sequence of :meth:`allreduce` calls."""

    def __init__(self, group, cap_floats: int, device):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device(device)
        self.cap = (int(cap_floats) + 3) // 4 * 4
        L = _lib.load()
        nbytes = int(L.qvb8_peer_bytes(self.world, self.cap))
        if nbytes <= 0:
            raise RuntimeError("qvb8_b200: bad world size / capacity for the peer all-reduce")
        # Every step that can fail on one rank only is followed by an exchange of the outcome, so that all ranks raise
        # together (a rank that left alone would leave the others waiting in the next collective).
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        err = None
        try:
            if self.device.type != "cuda" or not torch.cuda.is_available():
                raise RuntimeError("the peer all-reduce needs a CUDA device")
            with torch.cuda.device(self.device):
                _lib.check(L.qvb8_peer_alloc(nbytes, ctypes.byref(own), handle), "qvb8_peer_alloc")
        except RuntimeError as e:
            err = str(e)
        handles = [None] * self.world
        dist.all_gather_object(handles, None if err else bytes(handle.raw), group=group)
        self._ptrs = (ctypes.c_void_p * self.world)()
        self._own = own.value
        if any(h is None for h in handles):
            self._release(L)
            raise RuntimeError(f"qvb8_b200: a rank could not allocate its exchange area ({err or 'another rank'})")
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if r == self.rank:
                    self._ptrs[r] = own.value
                    continue
                p = ctypes.c_void_p()
                if L.qvb8_peer_open(handles[r], ctypes.byref(p)) != 0:
                    err = L.qvb8_last_error().decode()
                    break
                self._ptrs[r] = p.value
        outcomes = [None] * self.world
        dist.all_gather_object(outcomes, err, group=group)
        if any(o is not None for o in outcomes):
            self._release(L)
            raise RuntimeError(f"qvb8_b200: a rank could not map a peer's exchange area ({[o for o in outcomes if o][0]})")
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                         # every area is zeroed and mapped before the first push

    def allreduce(self, partial: torch.Tensor, out: torch.Tensor | None = None, flags: int = 0) -> torch.Tensor:
        """out = sum over the ranks of `partial` (fp32, contiguous, numel % 4 == 0), on the current stream."""
        if partial.dtype != torch.float32 or not partial.is_contiguous() or partial.device != self.device:
            raise RuntimeError("qvb8_b200: the peer all-reduce takes contiguous fp32 tensors on its device")
        out = partial if out is None else out
        n = partial.numel()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().qvb8_peer_allreduce(self._ptrs, self.rank, self.world, self.cap, self.epoch.data_ptr(),
                                                       partial.data_ptr(), out.data_ptr(), n, int(flags), _lib.stream_ptr(self.device)),
                       "qvb8_peer_allreduce")
        return out

    def allgather(self, part: torch.Tensor, out: torch.Tensor, flags: int = 0) -> torch.Tensor:
        """out[r] = rank r's `part` (fp32, contiguous, numel % 4 == 0; out holds world x part.numel() floats), on the
        current stream, by the same push protocol."""
        if any(t.dtype != torch.float32 or not t.is_contiguous() or t.device != self.device for t in (part, out)):
            raise RuntimeError("qvb8_b200: the peer all-gather takes contiguous fp32 tensors on its device")
        n = part.numel()
        if out.numel() != n * self.world:
            raise RuntimeError("qvb8_b200: the all-gather's output holds world x part.numel() floats")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().qvb8_peer_allgather(self._ptrs, self.rank, self.world, self.cap, self.epoch.data_ptr(),
                                                       part.data_ptr(), out.data_ptr(), n, int(flags), 0,
                                                       _lib.stream_ptr(self.device)), "qvb8_peer_allgather")
        return out

    def _release(self, L) -> None:
        if self.device.type != "cuda" or not torch.cuda.is_available():
            return
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if self._ptrs[r] and r != self.rank:
                    L.qvb8_peer_close(self._ptrs[r], 0)
                self._ptrs[r] = None
            if self._own:
                L.qvb8_peer_close(self._own, 1)
                self._own = None

    def close(self) -> None:
        L = _lib.load()
        torch.cuda.synchronize(self.device)
        self.dist.barrier(group=self.group)              # nobody frees memory a peer may still write
        self._release(L)
