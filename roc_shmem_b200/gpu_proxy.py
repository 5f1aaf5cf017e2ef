"""Reverse-offload mode on the GPU backend: kernels enqueue descriptors into a pinned host
ring (bshmem_proxy_device.cuh), a CPU thread executes them through a second runtime handle
with its own CUDA stream.  See csrc/cuda/gpu_proxy.cu."""
from __future__ import annotations

import ctypes as C

import torch

from .proxy import Proxy
from .utils.errors import raise_for_status


class GpuProxy(Proxy):
    """Host handle of the GPU PE's ring; host producers (Proxy methods) and device producers share it."""

    def __init__(self, rt, capacity: int):
        lib = rt.lib
        VP, I, U64 = C.c_void_p, C.c_int, C.c_uint64
        lib.bshmem_gpu_proxy_last_error.restype = C.c_char_p
        lib.bshmem_gpu_proxy_create.restype = I
        lib.bshmem_gpu_proxy_create.argtypes = [VP, VP, U64, U64, I, C.POINTER(VP), C.POINTER(VP), C.POINTER(VP)]
        lib.bshmem_gpu_proxy_set_timeout_us.restype, lib.bshmem_gpu_proxy_set_timeout_us.argtypes = I, [VP, U64]
        lib.bshmem_gpu_proxy_destroy.restype, lib.bshmem_gpu_proxy_destroy.argtypes = I, [VP]
        lib.bshmem_gpu_proxy_selftest.restype, lib.bshmem_gpu_proxy_selftest.argtypes = I, [VP, VP, VP, VP, I, I, VP]
        lib.bshmem_gpu_proxy_expect_timeout.restype, lib.bshmem_gpu_proxy_expect_timeout.argtypes = I, [VP, VP, VP, I, VP]
        gh, ring, px = C.c_void_p(), C.c_void_p(), C.c_void_p()
        st = lib.bshmem_gpu_proxy_create(rt.heap, rt.h, capacity, rt.config.timeout_ms * 1000, rt.device.index, C.byref(gh),
                                         C.byref(ring), C.byref(px))
        if st != 0:
            raise_for_status(st, lib.bshmem_gpu_proxy_last_error().decode())
        self.gh, self.ring_dev = gh, ring
        super().__init__(rt, capacity, handle=px.value)

    def submit(self, d, blocking: bool = True) -> int:
        # The ticket counter of a GPU ring lives in device memory (device producers reserve slots with
        # one atomic per warp); host threads cannot draw tickets from it.  Host code uses the runtime's
        # ordinary host API instead.
        from .utils.errors import ShmemError
        raise ShmemError(8, "host-side submission to a GPU proxy ring is not supported; use the host API")

    def set_timeout_ms(self, ms: int) -> None:
        raise_for_status(self.lib.bshmem_gpu_proxy_set_timeout_us(self.gh, ms * 1000))

    def device_selftest(self, peer: int, threads: int = 96) -> list[int]:
        """Runs put/get/p/g/atomics/quiet/fence through the ring from inside a kernel."""
        rt = self.rt
        sym = rt.zeros((64,), torch.int64)
        scratch = torch.zeros(64, dtype=torch.int64, device=rt.device)
        res = torch.full((32,), -2, dtype=torch.int32, device=rt.device)
        raise_for_status(self.lib.bshmem_gpu_proxy_selftest(rt.h, self.ring_dev, sym.data_ptr(), scratch.data_ptr(), peer, threads,
                                                            res.data_ptr()), "proxy selftest")
        out = res.tolist()
        return out[:out.index(-1)]

    def device_expect_timeout(self, sym: torch.Tensor, peer: int) -> int:
        status = torch.zeros(1, dtype=torch.int32, device=self.rt.device)
        raise_for_status(self.lib.bshmem_gpu_proxy_expect_timeout(self.rt.h, self.ring_dev, sym.data_ptr(), peer, status.data_ptr()))
        return int(status.item())

    def stop(self) -> None:
        if not self.stopped:
            self.stopped = True
            self.lib.bshmem_gpu_proxy_destroy(self.gh)


def attach_gpu_proxy(rt, capacity: int) -> GpuProxy:
    return GpuProxy(rt, capacity)
