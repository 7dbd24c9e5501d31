"""ctypes binding of ``libmoda_b200.so`` (declarations: ``include/moda_b200.h``).

The library is the only compute path of this package: there is no eager / CPU
fallback.  Loading fails loudly when the shared object has not been built
(``python -m moda_b200.build``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoda_b200.so")

MODE_CAUSAL, MODE_NONCAUSAL, MODE_CHUNK_VISIBLE, MODE_DEPTH_ONLY = 0, 1, 2, 3
DTYPE_BF16, DTYPE_FP16 = 0, 1
PATH_AUTO, PATH_SIMT_MMA, PATH_TCGEN05 = 0, 1, 2
PATH_TCGEN05_ONE_TILE, PATH_TCGEN05_TWO_TILES = 3, 4   # tcgen05 with the forward kernel fixed (tests)
PATH_TCGEN05_FUSED_BWD = 5                             # tcgen05 with the fused five-matmul backward (D = 128)
STATIC_SCRATCH_BYTES = 8 << 20   # MODA_B200_STATIC_SCRATCH_BYTES

# every symbol include/moda_b200.h declares
EXPORTED_SYMBOLS = (
    "moda_b200_fwd",
    "moda_b200_bwd_workspace_bytes",
    "moda_b200_bwd",
    "moda_b200_bwd_static_scratch",
    "moda_b200_depth_append",
    "moda_b200_check_problem",
    "moda_b200_resolve_path",
    "moda_b200_profile_begin",
    "moda_b200_profile_end",
    "moda_b200_kernel_name",
    "moda_b200_device_status",
    "moda_b200_tensor_pipe_rates",
    "moda_b200_last_launch_count",
    "moda_b200_last_cuda_error",
    "moda_b200_status_string",
    "moda_b200_version",
)


class Tensor4(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("stride_b", ctypes.c_int64),
        ("stride_t", ctypes.c_int64),
        ("stride_h", ctypes.c_int64),
    ]


class Problem(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32),
        ("T_kv", ctypes.c_int32),
        ("H", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("G", ctypes.c_int32),
        ("L", ctypes.c_int32),
        ("mode", ctypes.c_int32),
        ("chunk_rows", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("path", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("device", ctypes.c_int32),
        ("depth_rows_per_pos", ctypes.c_int32),      # 0 / L: packed depth KV; Lmax > L: in-place layer cache
        ("accumulate_depth_grads", ctypes.c_int32),  # backward adds the depth gradients instead of overwriting
    ]


class ModaLibraryError(RuntimeError):
    """The shared library is missing or returned a non-zero status."""

    def __init__(self, message: str, status: int = -1, cuda_error: int = 0):
        super().__init__(message)
        self.status = status
        self.cuda_error = cuda_error


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ModaLibraryError(
            f"{LIB_PATH} not found: build it with `python -m moda_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    P, T, V = ctypes.POINTER(Problem), ctypes.POINTER(Tensor4), ctypes.c_void_p
    lib.moda_b200_fwd.argtypes = [P, T, T, T, T, T, T, V, V]
    lib.moda_b200_fwd.restype = ctypes.c_int
    lib.moda_b200_bwd_workspace_bytes.argtypes = [P, ctypes.POINTER(ctypes.c_size_t)]
    lib.moda_b200_bwd_workspace_bytes.restype = ctypes.c_int
    lib.moda_b200_bwd.argtypes = [P] + [T] * 6 + [V] + [T] * 6 + [V, ctypes.c_size_t, V]
    lib.moda_b200_bwd.restype = ctypes.c_int
    lib.moda_b200_bwd_static_scratch.argtypes = [P] + [T] * 6 + [V] + [T] * 6 + [V]
    lib.moda_b200_bwd_static_scratch.restype = ctypes.c_int
    lib.moda_b200_depth_append.argtypes = [P, T, T, T, T, ctypes.c_int32, V]
    lib.moda_b200_depth_append.restype = ctypes.c_int
    lib.moda_b200_check_problem.argtypes = [P]
    lib.moda_b200_check_problem.restype = ctypes.c_int
    lib.moda_b200_resolve_path.argtypes = [P, ctypes.c_int]
    lib.moda_b200_resolve_path.restype = ctypes.c_int
    IP, FP = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_float)
    lib.moda_b200_profile_begin.restype = ctypes.c_int
    lib.moda_b200_profile_end.argtypes = [ctypes.c_int, IP, IP, IP, FP]
    lib.moda_b200_profile_end.restype = ctypes.c_int
    lib.moda_b200_kernel_name.argtypes = [ctypes.c_int]
    lib.moda_b200_kernel_name.restype = ctypes.c_char_p
    lib.moda_b200_device_status.argtypes = [IP]
    lib.moda_b200_device_status.restype = ctypes.c_int
    lib.moda_b200_tensor_pipe_rates.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.moda_b200_tensor_pipe_rates.restype = ctypes.c_int
    lib.moda_b200_last_launch_count.restype = ctypes.c_int
    lib.moda_b200_last_cuda_error.restype = ctypes.c_int
    lib.moda_b200_status_string.argtypes = [ctypes.c_int]
    lib.moda_b200_status_string.restype = ctypes.c_char_p
    lib.moda_b200_version.restype = ctypes.c_int
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().moda_b200_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        cuda_err = lib.moda_b200_last_cuda_error() if status == 9 else 0
        extra = f" (cudaError {cuda_err})" if cuda_err else ""
        raise ModaLibraryError(f"{what}: {status_string(status)}{extra}", status, cuda_err)


def profile_begin() -> None:
    check(load().moda_b200_profile_begin(), "moda_b200_profile_begin")


def profile_end() -> dict:
    """{kernel name: (launches, total_ms)} for the kernels launched since profile_begin."""
    lib = load()
    n = ctypes.c_int(0)
    ids = (ctypes.c_int * 16)()
    cnt = (ctypes.c_int * 16)()
    ms = (ctypes.c_float * 16)()
    check(lib.moda_b200_profile_end(16, ctypes.byref(n), ids, cnt, ms), "moda_b200_profile_end")
    return {lib.moda_b200_kernel_name(ids[i]).decode(): (int(cnt[i]), float(ms[i])) for i in range(n.value)}


TENSOR_PIPE_SHAPES = ("ss_n64", "ss_n128", "ss_n256", "ts_n64", "ts_n128", "ts_n256")


def tensor_pipe_rates(device_ptr: int, device: int, stream: int = 0) -> None:
    """Enqueue the tcgen05.mma rate probe: six floats (clocks per instruction, in the order of
    ``TENSOR_PIPE_SHAPES``) are written to the DEVICE buffer at ``device_ptr``."""
    check(load().moda_b200_tensor_pipe_rates(int(device), ctypes.c_void_p(device_ptr), ctypes.c_void_p(stream)),
          "moda_b200_tensor_pipe_rates")


def device_status() -> int:
    """Sticky status word of the tcgen05 kernels' bounded waits; synchronises.

    0 = every launch since the previous read ran to completion.  Non-zero = the first wait that
    expired since then ((1 << 8) | barrier id): that launch returned early and left outputs
    unwritten.  Reading resets the word, so callers poll it at their next synchronisation point."""
    v = ctypes.c_int(0)
    check(load().moda_b200_device_status(ctypes.byref(v)), "moda_b200_device_status")
    return int(v.value)
