"""Handing KV-cache tensors to an engine in another process.

``CudaIPCWrapper`` has the role and the picklable shape of the reference's class of the same name
(python/pegaflow/ipc_wrapper.py:15-163): built from a CUDA tensor in the worker process, sent as
bytes, opened where the engine lives.  The reference rebuilds a torch storage on the server side;
here the importing side is three C calls (``pf_ipc_open``) and yields what registration needs —
``(data_ptr, nbytes, device_id)`` — without torch.
"""
from __future__ import annotations

import ctypes as C
import pickle
from typing import Tuple

from . import _native as N


class CudaIPCWrapper:
    def __init__(self, tensor):
        """Export the tensor's whole storage (the tensor may be a strided view of it, as vLLM's
        HND-ordered caches are); it must start at storage offset 0 like in the reference."""
        if tensor.storage_offset() != 0:
            raise ValueError("Tensor must have zero storage offset")
        storage = tensor.untyped_storage()
        region = N.IpcRegion()
        N.check(N.lib.pf_ipc_export(storage.data_ptr(), storage.nbytes(), C.byref(region)))
        self.region = bytes(region)
        self.dtype = str(tensor.dtype)
        self.shape = tuple(tensor.shape)
        self.stride = tuple(tensor.stride())
        self.element_size = tensor.element_size()

    # what layout inference reads from a tensor (worker.py:65-151)
    def element_size_bytes(self) -> int:
        return self.element_size

    def open(self) -> Tuple[int, int, int]:
        """(data_ptr, nbytes, device_id) in the calling process; keep the wrapper until close()."""
        region = N.IpcRegion.from_buffer_copy(self.region)
        ptr, device = C.c_uint64(), C.c_int()
        N.check(N.lib.pf_ipc_open(C.byref(region), C.byref(ptr), C.byref(device)))
        return ptr.value, int(region.nbytes), device.value

    def close(self) -> None:
        region = N.IpcRegion.from_buffer_copy(self.region)
        N.check(N.lib.pf_ipc_close(C.byref(region)))

    def open_for(self, accessing_device: int) -> Tuple[int, int, int]:
        """(data_ptr, nbytes, owner_device) for a reader on another GPU of this process: the pointer is
        valid for kernels and copies of ``accessing_device`` only (the source of a peer copy)."""
        region = N.IpcRegion.from_buffer_copy(self.region)
        ptr, owner = C.c_uint64(), C.c_int()
        N.check(N.lib.pf_ipc_open_for(C.byref(region), accessing_device, C.byref(ptr), C.byref(owner)))
        return ptr.value, int(region.nbytes), owner.value

    def close_for(self, accessing_device: int) -> None:
        region = N.IpcRegion.from_buffer_copy(self.region)
        N.check(N.lib.pf_ipc_close_for(C.byref(region), accessing_device))

    def to_bytes(self) -> bytes:
        return pickle.dumps(self)

    @staticmethod
    def from_bytes(data: bytes) -> "CudaIPCWrapper":
        obj = pickle.loads(data)
        if not isinstance(obj, CudaIPCWrapper):
            raise TypeError("not a CudaIPCWrapper")
        return obj

    def __eq__(self, other) -> bool:
        return isinstance(other, CudaIPCWrapper) and (self.region, self.dtype, self.shape, self.stride) == (
            other.region, other.dtype, other.shape, other.stride)

    def __hash__(self):
        return hash((self.region, self.shape, self.stride))
