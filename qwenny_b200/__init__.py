"""qwenny_b200: B200-native (sm_100a) kernels for the decode / verify step of a Qwen3.5-style hybrid decoder,
behind the kernel-launch boundary of hellerchr/qwenny. The product is the CUDA library (csrc/, C ABI in
include/qwenny_b200.h); this package is its ctypes binding and the host-side mirror of the reference's launcher."""
from ._lib import LIB_PATH, QbError, lib  # noqa: F401

__all__ = ["lib", "LIB_PATH", "QbError"]
