"""Host-to-device uploads through the pinned ring (``csrc/kernels/upload_ring.cu``).

Checkpoint tensors are views of memory-mapped files: copying one to the device from pageable memory makes the driver
stage it through its own small bounce buffer, serially.  The ring cuts the write into chunks of up to 64 MiB and keeps
four pinned slots in flight, so reading the file (page faults, disk) overlaps the DMA of the previous chunk - the
reference's loading scheme (crates/poot-runtime-common/src/ring.rs:1-17).  ``upload`` falls back to a plain copy on a
machine without a device.
"""
from __future__ import annotations

import ctypes
from ctypes import c_ulonglong, c_void_p
from typing import Optional

import numpy as np
import torch

from ..ops._lib import check, kernels

CHUNK_BYTES = 64 << 20
SLOTS = 4


def slot_bytes(need: int) -> int:
    """Pinned size of a slot asked to hold ``need`` bytes: the next power of two, at least 64 KiB, at most one chunk."""
    lib = kernels()
    lib.poot_ring_slot_bytes.argtypes, lib.poot_ring_slot_bytes.restype = [c_ulonglong], c_ulonglong
    return int(lib.poot_ring_slot_bytes(int(need)))


class UploadRing:
    def __init__(self, slot_hint: int = CHUNK_BYTES):
        lib = kernels()
        lib.poot_ring_create.argtypes = [c_ulonglong, ctypes.POINTER(c_void_p)]
        lib.poot_ring_upload.argtypes = [c_void_p, c_void_p, c_ulonglong, c_void_p, c_void_p]
        lib.poot_ring_drain.argtypes = [c_void_p]
        lib.poot_ring_stats.argtypes = [c_void_p, ctypes.POINTER(c_ulonglong)]
        lib.poot_ring_destroy.argtypes = [c_void_p]
        self.lib = lib
        h = c_void_p()
        check(lib.poot_ring_create(int(slot_hint), ctypes.byref(h)), "ring_create")
        self.handle = h

    def upload(self, src: np.ndarray, dst: torch.Tensor) -> None:
        """Enqueue the copy of ``src`` (contiguous host array) into ``dst`` (contiguous device tensor of the same byte
        size) on the current stream; ``drain`` before the source mapping goes away or the data is needed."""
        src = np.ascontiguousarray(src)
        assert dst.is_cuda and dst.is_contiguous() and src.nbytes == dst.numel() * dst.element_size()
        check(self.lib.poot_ring_upload(self.handle, src.ctypes.data, src.nbytes, dst.data_ptr(),
                                        torch.cuda.current_stream(dst.device).cuda_stream), "ring_upload")

    def drain(self) -> None:
        check(self.lib.poot_ring_drain(self.handle), "ring_drain")

    def stats(self) -> dict:
        out = (c_ulonglong * 4)()
        check(self.lib.poot_ring_stats(self.handle, out), "ring_stats")
        return {"bytes": int(out[0]), "chunks": int(out[1]), "waits": int(out[2]), "slot_bytes": int(out[3])}

    def close(self) -> None:
        if self.handle is not None:
            self.lib.poot_ring_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_ring: Optional[UploadRing] = None


def shared_ring() -> UploadRing:
    global _ring
    if _ring is None:
        _ring = UploadRing()
    return _ring


def upload(src: np.ndarray, device, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """A device tensor holding ``src``'s bytes (viewed as ``dtype`` when given).  On a CUDA device the bytes go through
    the shared ring (the call returns with the last chunks in flight on the current stream, which orders them before any
    kernel launched after); elsewhere this is a plain copy."""
    device = torch.device(device)
    src = np.ascontiguousarray(src)
    if device.type != "cuda":
        t = torch.from_numpy(np.array(src))
        return t.view(dtype) if dtype is not None and t.dtype != dtype else t
    raw = torch.empty(src.nbytes, dtype=torch.uint8, device=device)
    ring = shared_ring()
    ring.upload(src.view(np.uint8).reshape(-1), raw)
    ring.drain()            # the source may be a view of a mapping the caller releases next
    tdt = dtype if dtype is not None else torch.from_numpy(np.zeros(0, src.dtype)).dtype
    return raw.view(tdt).view(*src.shape[:-1], -1) if src.ndim else raw.view(tdt)
