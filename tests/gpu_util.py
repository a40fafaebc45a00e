"""Helpers for the GPU parity tests: torch is used only to own device memory and streams."""
import ctypes

import numpy as np


class CudaMem:
    """"GPU memory" for the product engine: torch uint8 tensors on one CUDA device."""

    def __init__(self, device=0):
        import torch

        self.torch = torch
        self.device = torch.device("cuda", device)

    def alloc(self, nbytes):
        return self.torch.zeros(nbytes, dtype=self.torch.uint8, device=self.device)

    def ptr(self, buf):
        return buf.data_ptr()

    def write(self, buf, data):
        buf.copy_(self.torch.from_numpy(np.ascontiguousarray(data)))
        self.torch.cuda.synchronize(self.device)

    def read(self, buf):
        return buf.cpu().numpy().copy()

    def zero(self, buf):
        buf.zero_()
        self.torch.cuda.synchronize(self.device)

    def sync(self):
        self.torch.cuda.synchronize(self.device)


def host_view(addr, nbytes):
    """numpy uint8 view of `nbytes` of host memory at `addr` (pinned pool memory)."""
    return np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(addr))


def make_event(torch, timing=False):
    """A torch event whose cudaEvent_t already exists (torch creates it on the first record)."""
    ev = torch.cuda.Event(enable_timing=timing)
    ev.record()
    ev.synchronize()
    assert ev.cuda_event, "event handle was not created"
    return ev
