"""Host-side mirror of the reference's src/cuda/vmm.rs over the library's C entries: a Pool of 2 MiB device pages and
Regions that map them on demand behind fixed device addresses."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ._lib import check, lib


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Pool:
    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib().qb_pool_create(device, C.byref(h)), "qb_pool_create")
        self.h = h
        self.page = lib().qb_pool_page(h)

    def set_budget(self, pages: int):
        check(lib().qb_pool_set_budget(self.h, pages), "qb_pool_set_budget")

    def fill(self):
        check(lib().qb_pool_fill(self.h), "qb_pool_fill")

    def release(self, n: int) -> int:
        k = C.c_size_t(0)
        check(lib().qb_pool_release(self.h, n, C.byref(k)), "qb_pool_release")
        return k.value

    def usage(self) -> tuple[int, int]:
        u, b = C.c_size_t(0), C.c_size_t(0)
        check(lib().qb_pool_usage(self.h, C.byref(u), C.byref(b)), "qb_pool_usage")
        return u.value, b.value

    def available(self) -> int:
        return lib().qb_pool_available(self.h)

    def close(self):
        if self.h:
            lib().qb_pool_destroy(self.h)
            self.h = None


class Region:
    def __init__(self, pool: Pool, size: int):
        h = C.c_void_p()
        check(lib().qb_region_reserve(pool.h, size, C.byref(h)), "qb_region_reserve")
        self.h, self.pool = h, pool
        self.size = lib().qb_region_size(h)
        self.ptr = lib().qb_region_ptr(h)

    def map(self, start: int, end: int) -> bool:
        ok = C.c_int(0)
        check(lib().qb_region_map(self.h, _stream(), start, end, C.byref(ok)), "qb_region_map")
        return bool(ok.value)

    def unmap(self, start: int, end: int):
        check(lib().qb_region_unmap(self.h, _stream(), start, end), "qb_region_unmap")

    def is_mapped(self, start: int, end: int) -> bool:
        return bool(lib().qb_region_is_mapped(self.h, start, end))

    def read(self, start: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint8)
        check(lib().qb_region_read(self.h, _stream(), start, out.ctypes.data_as(C.c_void_p), n), "qb_region_read")
        return out

    def write(self, start: int, data: np.ndarray):
        d = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        check(lib().qb_region_write(self.h, _stream(), start, d.ctypes.data_as(C.c_void_p), len(d)), "qb_region_write")

    def close(self):
        if self.h:
            check(lib().qb_region_free(self.h, _stream()), "qb_region_free")
            self.h = None
