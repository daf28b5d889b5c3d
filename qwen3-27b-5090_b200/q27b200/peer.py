"""Device memory that the GPUs of a node can write into one another: the plumbing under the gather fused into the
grouped launch (q27b_skinny_fp4_group_gather). Every rank allocates a region of the same size; after the collective
set-up each rank holds a device pointer to every other rank's region, usable by its own kernels for plain stores over
NVLink. torch owns the memory and the exchange (symmetric memory); nothing here computes.

Layout of a region: a signal block of 16 int32 words at its head (zeroed; see q27b_group_peers in capi.h), payload from
byte 256 on. A store to byte x of the local payload is mirrored at the same byte of a peer's payload, so
out_delta[j] = ptr(peer j) - ptr(this rank).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

SIGNAL_BYTES = 256


class GroupPeers(ctypes.Structure):
    """Mirror of q27b_group_peers (include/q27b200/capi.h)."""

    _fields_ = [("n_peers", ctypes.c_int), ("my_slot", ctypes.c_int), ("out_delta", ctypes.c_int64 * 7),
                ("signals", ctypes.c_void_p), ("peer_signals", ctypes.c_void_p * 7)]


class PeerRegion:
    def __init__(self, payload_bytes: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert 2 <= self.world <= 8, "a node's GPUs: 2..8 ranks"
        dev = torch.device("cuda", torch.cuda.current_device())
        self.nbytes = SIGNAL_BYTES + (payload_bytes + 255) // 256 * 256
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self.local.zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.local, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert self.ptrs[self.rank] == self.local.data_ptr()
        dist.barrier(group)  # every region is zeroed before anyone signals into it

    def payload(self) -> torch.Tensor:
        """This rank's payload as a flat uint8 tensor (bytes 256.. of the region)."""
        return self.local[SIGNAL_BYTES:]

    def peer_slots(self):
        return [r for r in range(self.world) if r != self.rank]

    def peers(self) -> GroupPeers:
        p = GroupPeers()
        p.n_peers, p.my_slot, p.signals = self.world - 1, self.rank, self.ptrs[self.rank]
        for j, r in enumerate(self.peer_slots()):
            p.out_delta[j] = self.ptrs[r] - self.ptrs[self.rank]
            p.peer_signals[j] = self.ptrs[r]
        return p
