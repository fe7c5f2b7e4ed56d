"""Thin torch-tensor front end of the C ABI: each function takes CUDA tensors, passes their device pointers and the
current stream to the library, and returns/fills tensors. torch is plumbing here (device memory, streams); all the
arithmetic happens in the library's kernels."""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib

EPI = {"plain": 0, "silu": 1, "argmax": 2}


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Context:
    """The library context of one device (scratch, tickets, error word): Gemm::load of the reference."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("qwenny_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = device
        h = C.c_void_p()
        check(lib().qb_create(device, C.byref(h)), "qb_create")
        self.h = h

    def close(self):
        if self.h:
            lib().qb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def sms(self) -> int:
        return lib().qb_sm_count(self.h)

    def device_error(self) -> int:
        return lib().qb_device_error(self.h)

    def set_pdl(self, on: bool):
        check(lib().qb_set_pdl(self.h, int(on)), "qb_set_pdl")

    def tune(self, cg=0, kg=0, nstages=0, ctas=0):
        check(lib().qb_marlin_tune(self.h, cg, kg, nstages, ctas), "qb_marlin_tune")

    # ---- products
    def marlin_gemm(self, x, words, scales, epi="plain", y=None, row0=0, m=None, xrows=None, keys=None,
                    n_valid=None):
        """x f16 [rows][k]; words int32 [k/16][2n]; scales f16 [k/128][n]. Returns y (f32 [m][n] or f16 [m][n/2])."""
        k = x.shape[1]
        n = words.shape[1] // 2
        if m is None:
            m = (xrows.numel() if xrows is not None else x.shape[0] - row0)
        if y is None:
            rows = m if xrows is not None else row0 + m
            y = torch.empty((rows, n // 2), dtype=torch.float16, device=x.device) if epi == "silu" else \
                torch.empty((rows, n), dtype=torch.float32, device=x.device)
        check(lib().qb_marlin_gemm(self.h, _stream(), _p(x), _p(words), _p(y), _p(scales), m, n, k, row0, EPI[epi],
                                   _p(xrows), _p(keys), n if n_valid is None else n_valid), "qb_marlin_gemm")
        return y
