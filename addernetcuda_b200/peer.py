"""One-shot gradient averaging over the GPUs of one node through peer memory (host side).

`PeerArena` owns one receive area per process, exports it over CUDA IPC and maps the other ranks' areas;
`PeerAllReduce` binds one flat fp32 bucket to a slice of the arena and launches
`adder_b200_peer_allreduce` (one kernel: push to every rank, signal, bounded wait, add in rank order).
`ddp.BucketedDDP` uses them in place of NCCL's all-reduce for the small buckets of the CIFAR networks,
where a ring all-reduce is all latency.  The handles are exchanged through the existing process group
(`all_gather_object`), so nothing but torch.distributed is needed for the set-up.
"""
from __future__ import annotations

import ctypes
import socket
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib

# Waits are bounded: a poll costs 32-256 ns, so this is about fifteen seconds - beyond any skew between the ranks
# of a healthy job (a rank held up by its host for a moment must not cost the step), short enough that a lost
# rank surfaces as an error instead of a hang.
DEFAULT_MAX_POLLS = 1 << 26
# Buckets above this size stay on NCCL: one-shot moves (world - 1) x the bucket out of every GPU.
MAX_BUCKET_BYTES = 8 << 20

_opened = {}     # (peer rank, IPC handle bytes) -> base pointer in this process: a handle may be opened only once


def same_host(group=None) -> bool:
    """True when every rank of the group runs on this machine (peer mappings do not cross nodes)."""
    names: List[Optional[str]] = [None] * dist.get_world_size(group)
    dist.all_gather_object(names, socket.gethostname(), group=group)
    return len(set(names)) == 1


class PeerArena:
    """`nbytes` of zeroed device memory on every rank, each rank's block addressable from all the others."""

    def __init__(self, nbytes: int, device, group=None):
        lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        with torch.cuda.device(self.device):
            self.block = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            torch.cuda.synchronize(self.device)
            handle = (ctypes.c_ubyte * 64)()
            offset = ctypes.c_ulonglong(0)
            _lib.check(lib.adder_b200_ipc_export(self.block.data_ptr(), handle, ctypes.byref(offset)),
                       "adder_b200_ipc_export")
            mine = (bytes(handle), int(offset.value), self.device.index)
            everyone: List[Optional[tuple]] = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self.ptrs: List[int] = []
            for r, (h, off, _dev) in enumerate(everyone):
                if r == self.rank:
                    self.ptrs.append(self.block.data_ptr())
                    continue
                base = _opened.get((r, h))
                if base is None:
                    p = ctypes.c_void_p()
                    _lib.check(lib.adder_b200_ipc_open(h, 0, ctypes.byref(p)), "adder_b200_ipc_open")
                    base = int(p.value)
                    _opened[(r, h)] = base
                self.ptrs.append(base + off)
        # every area is zeroed and mapped everywhere before anyone pushes into it
        dist.barrier(group=group)


class PeerAllReduce:
    """Averages `flat` (fp32, CUDA, numel % 4 == 0) over the ranks in place: `launch(stream)`."""

    def __init__(self, flat: torch.Tensor, arena: PeerArena, arena_offset: int, max_polls: int = DEFAULT_MAX_POLLS,
                 chunks: int = 0):
        if flat.dtype != torch.float32 or not flat.is_cuda or not flat.is_contiguous() or flat.numel() % 4 != 0:
            raise ValueError("flat must be a contiguous fp32 CUDA tensor whose length is a multiple of 4")
        lib = _lib.load()
        self.flat = flat
        self.arena = arena
        need = lib.adder_b200_peer_area_bytes(flat.numel(), arena.world)
        if arena_offset % 16 != 0 or arena_offset + need > arena.nbytes:
            raise ValueError("arena slice misaligned or too small")
        data = (ctypes.c_void_p * 1)(flat.data_ptr())
        areas = (ctypes.c_void_p * arena.world)(*[p + arena_offset for p in arena.ptrs])
        self._comm = ctypes.c_void_p()
        with torch.cuda.device(flat.device):
            _lib.check(lib.adder_b200_peer_comm_create(ctypes.byref(self._comm), arena.world, arena.rank, 1, data, areas,
                                                       flat.numel(), int(chunks), int(max_polls)),
                       "adder_b200_peer_comm_create")

    @staticmethod
    def area_bytes(numel: int, world: int) -> int:
        n = int(_lib.load().adder_b200_peer_area_bytes(int(numel), int(world)))
        return (n + 255) // 256 * 256

    def launch(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream(self.flat.device)
        with torch.cuda.device(self.flat.device):
            _lib.check(_lib.load().adder_b200_peer_allreduce(self._comm, ctypes.c_void_p(s.cuda_stream)),
                       "adder_b200_peer_allreduce")

    def status(self, reset: bool = False) -> int:
        """The communicator's status word (0, or ADDER_ERR_TIMEOUT after a wait that ran out).  Synchronises."""
        st = ctypes.c_int(0)
        with torch.cuda.device(self.flat.device):
            _lib.check(_lib.load().adder_b200_peer_comm_status(self._comm, ctypes.byref(st), None, int(reset)),
                       "adder_b200_peer_comm_status")
        return int(st.value)

    def __del__(self):
        try:
            if self._comm:
                _lib.load().adder_b200_peer_comm_destroy(self._comm)
                self._comm = None
        except Exception:
            pass
