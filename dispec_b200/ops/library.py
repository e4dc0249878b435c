"""Loads the compiled kernel libraries (ctypes, C ABI over raw device pointers).

There is no fallback: if the library cannot be built or loaded, importing an op raises.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from dispec_b200.csrc import build

F32, BF16 = 0, 1

_core = None
_special: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


def core() -> ctypes.CDLL:
    global _core
    if _core is None:
        with _lock:
            if _core is None:
                path = build.core_library()
                # global: libraries loaded later resolve the runtime's symbols against this one
                lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
                lib.dsp_last_error.restype = ctypes.c_char_p
                _core = lib
    return _core


def attention_library(head_dim: int) -> ctypes.CDLL:
    key = f"attn_mma_d{head_dim}"
    if key not in _special:
        with _lock:
            if key not in _special:
                _special[key] = ctypes.CDLL(build.attention_library(head_dim))
    return _special[key]


def prefill_attention_library(head_dim: int) -> ctypes.CDLL:
    key = f"attn_tcgen05_d{head_dim}"
    if key not in _special:
        with _lock:
            if key not in _special:
                _special[key] = ctypes.CDLL(build.prefill_attention_library(head_dim))
    return _special[key]


def loaded_libraries() -> list[str]:
    out = [] if _core is None else [_core._name]
    return out + [lib._name for lib in _special.values()]


class LaunchCounter:
    """Counts kernels of this package launched (or replayed from a captured graph)."""
    n = 0


def check(rc: int, lib: ctypes.CDLL | None = None, launches: int = 1) -> None:
    LaunchCounter.n += launches
    if rc != 0:
        msg = core().dsp_last_error()
        raise KernelError(msg.decode() if msg else f"kernel library returned {rc}")


def device_error() -> int:
    """Reads and clears the device error word (synchronises)."""
    return int(core().dsp_device_error())


def raise_on_device_error(where: str) -> None:
    v = device_error()
    if v:
        names = [n for bit, n in ((1, "page id outside the pool"), (2, "token id outside the vocabulary"),
                                  (4, "a bounded wait ran out")) if v & bit]
        raise KernelError(f"{where}: device reported: {', '.join(names) or v}")


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle is asked for at every launch (some 250 times in a step that is not
# replayed from a graph); torch's own accessors build a Stream object and look the device up through
# several Python layers each time (7 us a call, a third of such a step's host time), the two raw
# entry points below return the same numbers in a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_handle() -> ctypes.c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def i64(v: int) -> ctypes.c_long:
    return ctypes.c_long(int(v))


def f32(v: float) -> ctypes.c_float:
    return ctypes.c_float(float(v))
