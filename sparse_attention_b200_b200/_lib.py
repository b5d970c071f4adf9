"""ctypes binding of libsparse_b200.so. There is no fallback: if the library is
missing or a call fails, an exception is raised."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# SPARSE_B200_LIB selects another build of the same library (kernel tuning experiments).
LIB_PATH = os.environ.get("SPARSE_B200_LIB") or os.path.join(HERE, "libsparse_b200.so")

ERR_INVALID, ERR_CUDA, ERR_TIMEOUT = -1, -2, -3


class SparseB200Error(RuntimeError):
    """Raised for every non-zero return code of the C ABI (the reference raises
    RuntimeError from TORCH_CHECK, attention/q_centric/progression_attention.cpp:23-92)."""


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SparseB200Error(
                f"{LIB_PATH} is missing: build it with `python -m sparse_attention_b200_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.sparse_b200_last_error.restype = ctypes.c_char_p
    return _lib


def check(code):
    if code != 0:
        raise SparseB200Error(f"sparse_b200 error {code}: {lib().sparse_b200_last_error().decode()}")


def ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def current_stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status(reset=True):
    """Synchronising read of the device status word; raises on a kernel timeout."""
    value = lib().sparse_b200_device_status(1 if reset else 0)
    if value < 0:
        check(value)
    if value > 0:
        raise SparseB200Error(f"a kernel abandoned a bounded wait (code 0x{value:x})")
    return value
