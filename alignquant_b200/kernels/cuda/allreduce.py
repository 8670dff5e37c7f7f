"""Peer-memory all-reduce for the partial outputs of row-parallel projections.

Stands in for the ``dist.all_reduce`` that tensor parallelism needs after o_proj / down_proj, for
the small FP32 messages of decode.  The reference has no counterpart: it runs on one GPU and
contains no collective.  One process per GPU; the exchange buffers are torch symmetric-memory allocations, so every rank
can store into every other rank's buffer over NVLink.  The kernel itself is
``aq_allreduce_f32`` of the C library (plain peer stores of values tagged with the call
number, bounded polls of the local receive area).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from alignquant_b200 import _lib


class PeerAllReduce:
    """Sum FP32 tensors of up to ``max_count`` elements over the ranks of ``group``.

    All ranks must construct the object collectively and call it in the same order with the
    same element counts.  Results are bit-identical on every rank (rank-ordered sum).
    """

    def __init__(self, max_count: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device(device)
        self.max_count = (int(max_count) + 3) // 4 * 4
        lib = _lib.load()
        size = int(lib.aq_allreduce_buffer_bytes(self.world, self.max_count))
        if size < 0:
            _lib.check(size)
        with torch.cuda.device(self.device):
            self.buffer = symm_mem.empty(size, dtype=torch.uint8, device=self.device)
            self.handle = symm_mem.rendezvous(self.buffer, self.group)
            self.buffer.zero_()
            torch.cuda.synchronize(self.device)
        # nobody may push into a buffer that its owner has not zeroed yet
        dist.barrier(group=self.group)
        pointers = [int(p) for p in self.handle.buffer_ptrs]
        if len(pointers) != self.world:
            raise RuntimeError("symmetric memory returned an unexpected number of peer pointers")
        self._peer_array = (ctypes.c_void_p * self.world)(*pointers)

    def peer_array_pointer(self) -> ctypes.c_void_p:
        """Host array of the ranks' exchange buffers, as the C entry points take it."""
        return ctypes.cast(self._peer_array, ctypes.c_void_p)

    def __call__(self, partial: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if partial.dtype != torch.float32 or not partial.is_contiguous() or partial.device != self.device:
            raise RuntimeError("partial must be a contiguous float32 tensor on the all-reduce's device")
        count = partial.numel()
        if count % 4 or count > self.max_count:
            raise RuntimeError(f"element count {count} must be a multiple of 4 and at most {self.max_count}")
        if out is None:
            out = partial
        elif out.dtype != torch.float32 or not out.is_contiguous() or out.numel() != count or out.device != self.device:
            raise RuntimeError("out must be a contiguous float32 tensor of the same size")
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(
                lib.aq_allreduce_f32(
                    ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(out.data_ptr()), count, self.rank, self.world,
                    ctypes.cast(self._peer_array, ctypes.c_void_p), self.max_count, ctypes.c_void_p(stream),
                )
            )
        return out
