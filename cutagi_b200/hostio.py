"""Host I/O path of a training step: ctypes mirror of the ``tagi_io_*`` entry points (include/tagi_b200.h).

``HostPipeline`` stages batches in pinned memory, uploads them on its own stream while the previous step computes, and
reads back exactly the B x n_out output moments. The arrays it hands out are numpy views of the pinned buffers, so a
data loader fills them in place (no list conversion, no pageable copy).
"""
import ctypes as C

import numpy as np

from .capi import lib


class HostPipeline:
    def __init__(self, in_floats, obs_floats, idx_ints, out_floats, depth=2):
        self.h = C.c_void_p()
        lib.tagi_io_create(in_floats, obs_floats, idx_ints, out_floats, depth, C.byref(self.h))
        self.depth, self.out_floats = depth, out_floats
        self.sizes = (in_floats, obs_floats, idx_ints)
        self.host, self.dev = [], []
        for s in range(depth):
            a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
            lib.tagi_io_host_buffers(self.h, s, C.byref(a), C.byref(b), C.byref(c))
            self.host.append((self._view(a, in_floats, np.float32), self._view(b, obs_floats, np.float32),
                              self._view(c, idx_ints, np.int32)))
            lib.tagi_io_device_buffers(self.h, s, C.byref(a), C.byref(b), C.byref(c))
            self.dev.append((a.value, b.value, c.value))

    @staticmethod
    def _view(ptr, n, dtype):
        if n == 0:
            return np.empty(0, dtype)
        ctype = C.c_float if dtype == np.float32 else C.c_int
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ctype)), shape=(n,))

    def host_arrays(self, slot):
        """(inputs, observations, indices) of the slot: numpy views of pinned memory, to be filled in place."""
        return self.host[slot]

    def device_tensors(self, slot):
        """The slot's device copies (inputs, observations, indices) as torch tensors: views, no copy."""
        import torch
        return tuple(None if n == 0 else _as_tensor(ptr, n, dt)
                     for ptr, n, dt in zip(self.dev[slot], self.sizes, (torch.float32, torch.float32, torch.int32)))

    def upload(self, slot, stream_ptr):
        lib.tagi_io_upload(self.h, slot, stream_ptr)

    def consumed(self, slot, stream_ptr):
        lib.tagi_io_consumed(self.h, slot, stream_ptr)

    def download(self, slot, mu, var, stream_ptr):
        """mu, var: CUDA tensors of the output moments (B x n_out)."""
        lib.tagi_io_download(self.h, slot, mu.data_ptr(), var.data_ptr(), mu.numel(), stream_ptr)

    def wait_output(self, slot, n):
        a, b = C.c_void_p(), C.c_void_p()
        lib.tagi_io_wait_output(self.h, slot, C.byref(a), C.byref(b))
        return self._view(a, n, np.float32), self._view(b, n, np.float32)

    def close(self):
        if self.h:
            lib.tagi_io_destroy(self.h)
            self.h = C.c_void_p()


def _as_tensor(ptr, n, dtype):
    """torch tensor over n elements of device memory owned by the pipeline."""
    import torch

    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4" if dtype == torch.float32 else "<i4",
                                  "data": (ptr, False), "version": 2}
    return torch.as_tensor(h, device="cuda")
