"""ctypes binding of libfrnnt_sm100.so (the C ABI declared in include/frnnt.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised.  Tensors are passed as raw device pointers plus sizes; the current
torch CUDA stream is passed to every call.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfrnnt_sm100.so")

F32, F64, F16, BF16 = 0, 1, 2, 3
_lib = None

_c_int, _c_vp, _c_sz, _c_f64 = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_double
_c_longlong = ctypes.c_longlong


class FrnntError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FrnntError(
                f"{LIB_PATH} is missing: build it with `python -m fast_rnnt_b200.build` "
                "(needs nvcc; sm_100a). There is no CPU or PyTorch fallback.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.frnnt_last_error.restype = ctypes.c_char_p
        for name in ("frnnt_mi_lattice_bytes", "frnnt_simple_saved_bytes",
                     "frnnt_simple_scratch_bytes", "frnnt_matmul_tn_scratch_floats",
                     "frnnt_joiner_input_grads_scratch_bytes", "frnnt_pruned_joiner_saved_bytes",
                     "frnnt_pruned_joiner_forward_scratch_bytes",
                     "frnnt_pruned_joiner_backward_scratch_bytes"):
            if hasattr(_lib, name):
                getattr(_lib, name).restype = _c_sz
    return _lib


def dtype_code(dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.float64:
        return F64
    raise TypeError(f"only float32 and float64 are supported (as in the reference), got {dtype}")


_HALF_CODES = {torch.float16: F16, torch.bfloat16: BF16}


def is_16bit(t) -> bool:
    return t is not None and t.dtype in _HALF_CODES


def input_code(dtype) -> int:
    """dtype code of an INPUT that a kernel may read as 16-bit values."""
    return _HALF_CODES[dtype] if dtype in _HALF_CODES else dtype_code(dtype)


def ptr(t):
    """Device pointer of a contiguous CUDA tensor (None -> NULL)."""
    if t is None:
        return None
    assert t.is_cuda, "fast_rnnt_b200 runs on CUDA tensors only (no CPU path)"
    assert t.is_contiguous()
    return _c_vp(t.data_ptr())


def stream_ptr(device):
    return _c_vp(torch.cuda.current_stream(device).cuda_stream)


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().frnnt_last_error().decode("utf-8", "replace")
        raise FrnntError(f"{what} failed with code {rc}: {msg}")


def call(name: str, *args):
    fn = getattr(lib(), name)
    check(fn(*args), name)
