"""Symmetric device memory across the ranks of one node.

Every rank allocates a block of the same size with ``cudaMalloc`` (zero-filled), exports it with a CUDA IPC
handle, gathers all handles over the ``torch.distributed`` control plane and maps every peer's block.  Kernels
then address a peer's memory with ordinary pointers over NVLink.  The reference opens peer access between
contexts of one process (crates/poot-ptx-runtime/src/context.rs:608-640); with one process per GPU the
equivalent is IPC mapping.  ``probe()`` is the start-up delivery check of every directed link.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_size_t, c_uint, c_void_p
from typing import List

import torch
import torch.distributed as dist

from ..ops._lib import check, kernels


class PeerLinkError(RuntimeError):
    """A peer mapping reports access but did not deliver the probe pattern."""


class SymmetricBlock:
    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, group=None):
        lib = kernels()
        self.lib, self.rank, self.world, self.device, self.nbytes = lib, rank, world, device, nbytes
        lib.poot_symm_alloc.argtypes = [c_size_t, ctypes.POINTER(c_void_p)]
        lib.poot_ipc_get_handle.argtypes = [c_void_p, c_void_p]
        lib.poot_ipc_open.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
        lib.poot_ipc_close.argtypes = [c_void_p]
        lib.poot_symm_free.argtypes = [c_void_p]
        torch.cuda.set_device(device)
        p = c_void_p()
        check(lib.poot_symm_alloc(nbytes, ctypes.byref(p)), "symm_alloc")
        self.local = p.value
        hs = lib.poot_ipc_handle_size()
        buf = ctypes.create_string_buffer(hs)
        check(lib.poot_ipc_get_handle(self.local, buf), "ipc_get_handle")
        handles: List[bytes] = [b""] * world
        dist.all_gather_object(handles, bytes(buf.raw), group=group)
        self.ptrs: List[int] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local)
            else:
                q = c_void_p()
                hb = ctypes.create_string_buffer(handles[r], hs)
                check(lib.poot_ipc_open(hb, ctypes.byref(q)), f"ipc_open(rank {r})")
                self.ptrs.append(q.value)
        self._closed = False

    def ptr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + offset

    def ptr_array(self, offset: int = 0):
        """Host array of ``void*`` (one per rank) at a byte offset inside the block."""
        arr = (c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def local_tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        """A torch view of this rank's own block (the block outlives the view; do not free while in use)."""
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        assert offset + n * esz <= self.nbytes

        class _Holder:
            pass

        holder = _Holder()
        holder.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": {torch.uint8: "|u1", torch.int32: "<i4", torch.float32: "<f4",
                                               torch.bfloat16: "<u2", torch.uint32: "<u4"}[dtype],
            "data": (self.local + offset, False), "version": 2}
        t = torch.as_tensor(holder, device=self.device)
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t

    def probe(self, group=None) -> None:
        """Write a pattern into every peer's block over its mapping, then check what arrived here."""
        lib = self.lib
        lib.poot_tp_probe_write.argtypes = [c_void_p, c_longlong, c_uint, c_void_p]
        lib.poot_tp_probe_check.argtypes = [c_void_p, c_longlong, c_uint, c_void_p, c_void_p]
        stream = torch.cuda.current_stream().cuda_stream
        bad = torch.zeros(1, dtype=torch.int32, device=self.device)
        for size in (256, 64 * 1024, 4 * 1024 * 1024):
            words = min(size, self.nbytes // self.world) // 4
            if words == 0:
                continue
            # rank r writes slice [rank] of every peer's block; each rank then checks all slices it received
            slice_bytes = (self.nbytes // self.world) // 16 * 16
            for d in range(self.world):
                check(lib.poot_tp_probe_write(self.ptr(d, self.rank * slice_bytes), words, 0xC0FFEE00 + self.rank,
                                              stream), "probe_write")
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
            for src in range(self.world):
                check(lib.poot_tp_probe_check(self.local + src * slice_bytes, words, 0xC0FFEE00 + src,
                                              bad.data_ptr(), stream), "probe_check")
            torch.cuda.synchronize(self.device)
            if int(bad.item()) != 0:
                raise PeerLinkError(f"rank {self.rank}: {int(bad.item())} words of a {size}-byte probe did not arrive")
            dist.barrier(group=group)
        # leave the block zeroed for its real use
        torch.cuda.synchronize(self.device)
        self.local_tensor(0, (self.nbytes,), torch.uint8).zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.lib.poot_ipc_close(p)
        self.lib.poot_symm_free(self.local)
