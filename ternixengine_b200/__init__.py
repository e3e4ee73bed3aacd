"""B200-native ternary matrix product behind TernixEngine's API.

    C[M,N] int32 = A[M,K] int8 x W[K,N] ternary, W packed K x (N/4) bytes (00 -> 0, 01 -> +1, 11 -> -1)

This package is the Python host side: a ctypes binding of the C ABI (``include/ternix_b200.h``,
built in-tree as ``libternix_b200.so``) plus the N-column sharding layer that runs one process
per GPU over ``torch.distributed``.  PyTorch is used for device memory, streams and the process
group only; all arithmetic happens in the library's own sm_100a kernels.  There is no CPU
implementation here and no fallback: if the library is missing, importing fails.

The reference's Python surface (``bindings/python/pybind11_wrapper.cpp:75-98``: ``pack_ternary``,
``unpack_ternary``, ``ternary_matmul``, ``has_cuda``) is re-exported from the compiled module
``ternix_engine`` that is built next to this file.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("TERNIX_B200_LIB") or os.path.join(_HERE, "libternix_b200.so")

OK = 0
ERR_INVALID_SHAPE = 1
ERR_INVALID_ARG = 2
ERR_CUDA = 3
ERR_TIMEOUT = 4
ERR_UNSUPPORTED = 5
ERR_TOO_LARGE = 6

KERNEL_AUTO = 0
KERNEL_GENERIC = 1
KERNEL_GEMV = 2
KERNEL_GEMM_TC = 3
KERNEL_DECODE_MMA = 4
KERNEL_SKINNY_TC = 5
KERNELS = {"auto": KERNEL_AUTO, "generic": KERNEL_GENERIC, "gemv": KERNEL_GEMV, "gemm_tc": KERNEL_GEMM_TC,
           "decode_mma": KERNEL_DECODE_MMA, "skinny_tc": KERNEL_SKINNY_TC}

# every symbol include/ternix_b200.h declares
EXPORTS = (
    "ternix_b200_status_string", "ternix_b200_last_cuda_error", "ternix_b200_cuda_error_string",
    "ternix_b200_version", "ternix_b200_last_launched_kernel", "ternix_b200_launched_kernel_name",
    "ternix_b200_set_option", "ternix_b200_release_cached_memory",
    "ternix_b200_weights_create", "ternix_b200_weights_matmul", "ternix_b200_weights_matmul_host", "ternix_b200_weights_destroy",
    "ternix_b200_pack_ternary_device", "ternix_b200_selftest_wait_timeout",
    "ternix_b200_pack_ternary", "ternix_b200_unpack_ternary", "ternix_b200_interleave_offline",
    "ternix_b200_find_non_ternary", "ternix_b200_slice_columns",
    "ternix_b200_matmul", "ternix_b200_matmul_ex", "ternix_b200_select_kernel", "ternix_b200_matmul_host",
    "ternix_b200_group_create", "ternix_b200_group_create_ex", "ternix_b200_group_create_prepacked",
    "ternix_b200_prepack_k4", "ternix_b200_prepack_k4_bytes", "ternix_b200_group_run", "ternix_b200_group_launches", "ternix_b200_group_destroy",
    "ternix_b200_gemv_batch_noalloc", "ternix_b200_gemv_batch_noalloc_limits",
    "ternix_b200_quantize_rows", "ternix_b200_matmul_dequant",
    "ternix_b200_matmul_bcast", "ternix_b200_peer_alloc", "ternix_b200_peer_free", "ternix_b200_peer_export",
    "ternix_b200_peer_import", "ternix_b200_peer_close", "ternix_b200_peer_barrier",
    "ternix_b200_shard_columns", "ternix_b200_unpack_gathered",
    "ternix_b200_synth_activations", "ternix_b200_synth_packed_weights", "ternix_b200_synth_weights",
)


class _Problem(ctypes.Structure):
    """struct ternix_b200_problem"""
    _fields_ = [("dA", ctypes.c_void_p), ("dW", ctypes.c_void_p), ("dC", ctypes.c_void_p),
                ("M", ctypes.c_int), ("K", ctypes.c_int), ("N", ctypes.c_int), ("ldc", ctypes.c_longlong)]


class TernixError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(what)
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `make -C ternixengine_b200/csrc` "
            "(or __graft_entry__.build()).  There is no fallback implementation.")
    lib = ctypes.CDLL(_LIB_PATH)
    c = ctypes
    vp, i32, i64, sz, u64 = c.c_void_p, c.c_int, c.c_longlong, c.c_size_t, c.c_uint64
    sig = {
        "ternix_b200_status_string": (c.c_char_p, [i32]),
        "ternix_b200_last_cuda_error": (i32, []),
        "ternix_b200_cuda_error_string": (c.c_char_p, [i32]),
        "ternix_b200_version": (i32, []),
        "ternix_b200_last_launched_kernel": (i32, []),
        "ternix_b200_launched_kernel_name": (c.c_char_p, [i32]),
        "ternix_b200_set_option": (i32, [c.c_char_p, c.c_char_p]),
        "ternix_b200_release_cached_memory": (i32, []),
        "ternix_b200_weights_create": (i32, [c.POINTER(vp), vp, i32, i32]),
        "ternix_b200_weights_matmul": (i32, [vp, vp, vp, i32, i64, vp, vp]),
        "ternix_b200_weights_matmul_host": (i32, [vp, vp, vp, i32]),
        "ternix_b200_weights_destroy": (None, [vp]),
        "ternix_b200_pack_ternary_device": (i32, [vp, vp, sz, vp]),
        "ternix_b200_selftest_wait_timeout": (i32, [c.c_ulonglong, vp, vp, vp]),
        "ternix_b200_pack_ternary": (None, [vp, vp, sz]),
        "ternix_b200_unpack_ternary": (None, [vp, vp, sz]),
        "ternix_b200_interleave_offline": (None, [vp, vp, sz]),
        "ternix_b200_find_non_ternary": (i64, [vp, sz]),
        "ternix_b200_slice_columns": (i32, [vp, vp, sz, sz, sz, sz]),
        "ternix_b200_matmul": (i32, [vp, vp, vp, i32, i32, i32, vp]),
        "ternix_b200_matmul_ex": (i32, [vp, vp, vp, i32, i32, i32, i64, i32, vp, vp]),
        "ternix_b200_select_kernel": (i32, [vp, vp, vp, i32, i32, i32, i64]),
        "ternix_b200_matmul_host": (i32, [vp, vp, vp, i32, i32, i32, i32]),
        "ternix_b200_group_create": (i32, [c.POINTER(vp), c.POINTER(_Problem), i32]),
        "ternix_b200_group_create_ex": (i32, [c.POINTER(vp), c.POINTER(_Problem), i32, c.POINTER(vp), i32]),
        "ternix_b200_group_create_prepacked": (i32, [c.POINTER(vp), c.POINTER(_Problem), i32]),
        "ternix_b200_prepack_k4": (i32, [vp, vp, i32, i32, vp]),
        "ternix_b200_prepack_k4_bytes": (sz, [i32, i32]),
        "ternix_b200_group_run": (i32, [vp, vp, vp]),
        "ternix_b200_group_launches": (i32, [vp]),
        "ternix_b200_group_destroy": (None, [vp]),
        "ternix_b200_gemv_batch_noalloc": (i32, [c.POINTER(_Problem), i32, vp, vp]),
        "ternix_b200_gemv_batch_noalloc_limits": (i32, [c.POINTER(i32), c.POINTER(i32), c.POINTER(i64)]),
        "ternix_b200_quantize_rows": (i32, [vp, i32, i64, vp, vp, i32, i32, vp]),
        "ternix_b200_matmul_dequant": (i32, [vp, vp, c.POINTER(vp), i32, vp, c.c_float, i32, i32, i32, i64, vp, vp]),
        "ternix_b200_matmul_bcast": (i32, [vp, vp, c.POINTER(vp), i32, i32, i32, i32, i64, vp, vp]),
        "ternix_b200_peer_alloc": (i32, [c.POINTER(vp), sz]),
        "ternix_b200_peer_free": (i32, [vp]),
        "ternix_b200_peer_export": (i32, [vp, c.c_char_p]),
        "ternix_b200_peer_import": (i32, [c.c_char_p, c.POINTER(vp)]),
        "ternix_b200_peer_close": (i32, [vp]),
        "ternix_b200_peer_barrier": (i32, [c.POINTER(vp), i32, i32, c.c_uint, u64, vp, vp]),
        "ternix_b200_shard_columns": (i32, [i32, i32, i32, i32, c.POINTER(i32), c.POINTER(i32)]),
        "ternix_b200_unpack_gathered": (i32, [vp, vp, i32, i32, i64, i32, i32, i32, vp]),
        "ternix_b200_synth_activations": (None, [vp, sz, u64, i32]),
        "ternix_b200_synth_packed_weights": (None, [vp, sz, sz, u64]),
        "ternix_b200_synth_weights": (None, [vp, sz, sz, u64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.ternix_b200_status_string(status).decode()


def _check(status: int, where: str) -> None:
    if status == OK:
        return
    msg = f"{where}: {status_string(status)}"
    if status == ERR_CUDA:
        e = lib.ternix_b200_last_cuda_error()
        msg += f" [cudaError {e}: {lib.ternix_b200_cuda_error_string(e).decode()}]"
    if status in (ERR_INVALID_SHAPE, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_TOO_LARGE):
        raise ValueError(msg)
    raise TernixError(status, msg)


def set_option(name: str, value=None) -> None:
    """Sets a tuning option of the library (ternix_b200_set_option); value None restores the default."""
    v = None if value is None else str(value).encode()
    _check(lib.ternix_b200_set_option(name.encode(), v), f"set_option({name})")


def last_launched_kernel() -> str:
    """Name of the kernel the calling thread's last single-product call launched."""
    return lib.ternix_b200_launched_kernel_name(lib.ternix_b200_last_launched_kernel()).decode()


def release_cached_memory() -> None:
    """Hands the device memory cached by the host-pointer entry point back to the driver."""
    _check(lib.ternix_b200_release_cached_memory(), "release_cached_memory")


def _np_ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


# --------------------------------------------------------------------------- host: packed format
def pack_ternary(w: np.ndarray) -> np.ndarray:
    """(K, N) int8 in {-1,0,+1} -> (K, N/4) uint8.  Same checks and errors as the reference binding
    (bindings/python/pybind11_wrapper.cpp:21-31)."""
    w = np.ascontiguousarray(w, dtype=np.int8)
    if w.ndim != 2:
        raise ValueError("pack_ternary expects a 2-D (K, N) array")
    K, N = w.shape
    if N % 4:
        raise ValueError("N must be a multiple of 4")
    if lib.ternix_b200_find_non_ternary(_np_ptr(w), w.size) >= 0:
        raise ValueError("weights must be in {-1, 0, +1}")
    out = np.empty((K, N // 4), dtype=np.uint8)
    lib.ternix_b200_pack_ternary(_np_ptr(out), _np_ptr(w), w.size)
    return out


def unpack_ternary(packed: np.ndarray) -> np.ndarray:
    """(K, N/4) uint8 -> (K, N) int8 (bindings/python/pybind11_wrapper.cpp:33-39)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    if packed.ndim != 2:
        raise ValueError("unpack_ternary expects a 2-D (K, N/4) array")
    K, n4 = packed.shape
    out = np.empty((K, n4 * 4), dtype=np.int8)
    lib.ternix_b200_unpack_ternary(_np_ptr(out), _np_ptr(packed), out.size)
    return out


def slice_columns(packed: np.ndarray, n0: int, n_cols: int) -> np.ndarray:
    """Column shard [n0, n0+n_cols) of a packed matrix, itself a valid packed matrix."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    K, n4 = packed.shape
    out = np.empty((K, n_cols // 4), dtype=np.uint8)
    _check(lib.ternix_b200_slice_columns(_np_ptr(out), _np_ptr(packed), K, n4 * 4, n0, n_cols), "slice_columns")
    return out


def ternary_matmul_host(a: np.ndarray, b_packed: np.ndarray, kernel: str = "auto") -> np.ndarray:
    """Host arrays in, host array out, through ternix_b200_matmul_host (upload, kernel, download)."""
    a = np.ascontiguousarray(a, dtype=np.int8)
    b_packed = np.ascontiguousarray(b_packed, dtype=np.uint8)
    if a.ndim != 2 or b_packed.ndim != 2:
        raise ValueError("A must be (M, K) and B_packed (K, N/4)")
    M, K = a.shape
    if b_packed.shape[0] != K:
        raise ValueError("inner dimensions do not match")
    N = b_packed.shape[1] * 4
    c = np.empty((M, N), dtype=np.int32)
    _check(lib.ternix_b200_matmul_host(_np_ptr(a), _np_ptr(b_packed), _np_ptr(c), M, K, N, KERNELS[kernel]),
           "ternary_matmul_host")
    return c


# --------------------------------------------------------------------------- host: synthetic inputs
def synth_activations(shape, seed: int, lo: int = -128) -> np.ndarray:
    """Seeded int8 activations, uniform on [lo, 127] with lo in {-128, -127}."""
    if lo not in (-128, -127):
        raise ValueError("lo must be -128 or -127")
    out = np.empty(shape, dtype=np.int8)
    lib.ternix_b200_synth_activations(_np_ptr(out), out.size, seed, 1 if lo == -127 else 0)
    return out


def synth_packed_weights(K: int, N: int, seed: int) -> np.ndarray:
    """Seeded iid ternary weights, P(0)=0.4, P(+1)=P(-1)=0.3, already packed (K, N/4)."""
    if N % 4:
        raise ValueError("N must be a multiple of 4")
    out = np.empty((K, N // 4), dtype=np.uint8)
    lib.ternix_b200_synth_packed_weights(_np_ptr(out), K, N, seed)
    return out


def synth_weights(K: int, N: int, seed: int) -> np.ndarray:
    out = np.empty((K, N), dtype=np.int8)
    lib.ternix_b200_synth_weights(_np_ptr(out), K, N, seed)
    return out


# --------------------------------------------------------------------------- device path (torch tensors)
def select_kernel(M: int, K: int, N: int, a_ptr: int = 0, w_ptr: int = 0) -> int:
    return lib.ternix_b200_select_kernel(a_ptr, w_ptr, 0, M, K, N, N)


def matmul(a, w_packed, out=None, kernel: str = "auto", status=None, stream=None):
    """Device tensors: a (M,K) int8, w_packed (K,N/4) uint8 -> (M,N) int32, asynchronous on the
    current (or given) CUDA stream.  `out` may be a column slice of a wider row-major matrix."""
    import torch

    if not (a.is_cuda and w_packed.is_cuda):
        raise ValueError("matmul() takes CUDA tensors; use ternary_matmul_host() for host arrays")
    if a.dtype != torch.int8 or w_packed.dtype != torch.uint8 or a.dim() != 2 or w_packed.dim() != 2:
        raise ValueError("A must be (M, K) int8 and W_packed (K, N/4) uint8")
    if not (a.is_contiguous() and w_packed.is_contiguous()):
        raise ValueError("A and W_packed must be contiguous")
    M, K = a.shape
    if w_packed.shape[0] != K:
        raise ValueError("inner dimensions do not match")
    N = w_packed.shape[1] * 4
    if out is None:
        out = torch.empty((M, N), dtype=torch.int32, device=a.device)
    if out.dtype != torch.int32 or tuple(out.shape) != (M, N) or (N > 1 and out.stride(1) != 1):
        raise ValueError("out must be (M, N) int32 with unit column stride")
    ldc = out.stride(0) if M > 1 else max(N, out.stride(0))
    s = stream if stream is not None else torch.cuda.current_stream(a.device)
    with torch.cuda.device(a.device):
        rc = lib.ternix_b200_matmul_ex(a.data_ptr(), w_packed.data_ptr(), out.data_ptr(), M, K, N, ldc,
                                       KERNELS[kernel], status.data_ptr() if status is not None else None,
                                       s.cuda_stream)
    _check(rc, "matmul")
    return out


class TernaryWeights:
    """A packed weight matrix on the device with its TMA descriptors encoded once (ternix_b200_weights_create):
    matmul() through the handle encodes nothing for operands it saw on the previous call."""

    def __init__(self, w_packed):
        import torch

        if not w_packed.is_cuda or w_packed.dtype != torch.uint8 or w_packed.dim() != 2 or not w_packed.is_contiguous():
            raise ValueError("TernaryWeights takes a contiguous CUDA uint8 (K, N/4) tensor")
        self.w = w_packed
        self.K, self.N = w_packed.shape[0], w_packed.shape[1] * 4
        h = ctypes.c_void_p()
        with torch.cuda.device(w_packed.device):
            _check(lib.ternix_b200_weights_create(ctypes.byref(h), w_packed.data_ptr(), self.K, self.N), "weights_create")
        self._h = h

    def matmul(self, a, out=None, status=None, stream=None):
        import torch

        if not a.is_cuda or a.dtype != torch.int8 or a.dim() != 2 or not a.is_contiguous() or a.shape[1] != self.K:
            raise ValueError("A must be a contiguous CUDA int8 (M, K) tensor")
        M = a.shape[0]
        if out is None:
            out = torch.empty((M, self.N), dtype=torch.int32, device=a.device)
        if out.dtype != torch.int32 or tuple(out.shape) != (M, self.N) or (self.N > 1 and out.stride(1) != 1):
            raise ValueError("out must be (M, N) int32 with unit column stride")
        ldc = out.stride(0) if M > 1 else max(self.N, out.stride(0))
        s = stream if stream is not None else torch.cuda.current_stream(a.device)
        with torch.cuda.device(a.device):
            _check(lib.ternix_b200_weights_matmul(self._h, a.data_ptr(), out.data_ptr(), M, ldc,
                                                  status.data_ptr() if status is not None else None, s.cuda_stream),
                   "weights_matmul")
        return out

    def matmul_host(self, a_host, out_host=None):
        """C = A x W with the activations and the result in host memory (numpy arrays or CPU torch tensors, ideally
        pinned) and the weights resident on the device: row slabs on three streams, so the call takes little more
        than the download of C (ternix_b200_weights_matmul_host).  Synchronous."""
        import torch

        def host_ptr(x, dtype_np, dtype_t, shape, what):
            if isinstance(x, np.ndarray):
                if x.dtype != dtype_np or x.shape != shape or not x.flags["C_CONTIGUOUS"]:
                    raise ValueError(f"{what} must be a C-contiguous {np.dtype(dtype_np).name} array of shape {shape}")
                return x.ctypes.data
            if x.is_cuda or x.dtype != dtype_t or tuple(x.shape) != shape or not x.is_contiguous():
                raise ValueError(f"{what} must be a contiguous CPU tensor of shape {shape}")
            return x.data_ptr()

        M = a_host.shape[0]
        if out_host is None:
            out_host = torch.empty((M, self.N), dtype=torch.int32, pin_memory=True)
        pa = host_ptr(a_host, np.int8, torch.int8, (M, self.K), "A")
        pc = host_ptr(out_host, np.int32, torch.int32, (M, self.N), "out")
        with torch.cuda.device(self.w.device):
            _check(lib.ternix_b200_weights_matmul_host(self._h, pa, pc, M), "weights_matmul_host")
        return out_host

    def close(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.ternix_b200_weights_destroy(self._h)
        self._h = None

    def __del__(self):
        self.close()


def pack_ternary_device(w):
    """(K, N) int8 CUDA tensor in {-1,0,+1} -> (K, N/4) uint8 CUDA tensor, packed on the device
    (ternix_b200_pack_ternary_device); the same bytes as pack_ternary()."""
    import torch

    if not w.is_cuda or w.dtype != torch.int8 or w.dim() != 2 or not w.is_contiguous() or w.shape[1] % 4:
        raise ValueError("pack_ternary_device takes a contiguous CUDA int8 (K, N) tensor with N % 4 == 0")
    out = torch.empty((w.shape[0], w.shape[1] // 4), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        _check(lib.ternix_b200_pack_ternary_device(out.data_ptr(), w.data_ptr(), w.numel(),
                                                   torch.cuda.current_stream(w.device).cuda_stream), "pack_ternary_device")
    return out


def quantize_rows(x):
    """Per-row absmax int8 quantisation of a CUDA float32 / bfloat16 (M, K) tensor -> (int8 (M, K), float32 (M,))."""
    import torch

    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1 or x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("quantize_rows takes a CUDA float32 or bfloat16 (M, K) tensor with unit column stride")
    M, K = x.shape
    a = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.ternix_b200_quantize_rows(x.data_ptr(), 0 if x.dtype == torch.float32 else 1, x.stride(0) if M > 1 else K,
                                             a.data_ptr(), scale.data_ptr(), M, K,
                                             torch.cuda.current_stream(x.device).cuda_stream), "quantize_rows")
    return a, scale


def matmul_dequant(a, w_packed, row_scale, w_scale: float, out=None, status=None, extra_dest_ptrs=()):
    """bfloat16 (M, N) = (A x W) * row_scale[:, None] * w_scale with the integer product exact."""
    import torch

    M, K = a.shape
    N = w_packed.shape[1] * 4
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or out.stride(1) != 1:
        raise ValueError("out must be (M, N) bfloat16 with unit column stride")
    ptrs = (ctypes.c_void_p * (1 + len(extra_dest_ptrs)))(out.data_ptr(), *extra_dest_ptrs)
    with torch.cuda.device(a.device):
        _check(lib.ternix_b200_matmul_dequant(a.data_ptr(), w_packed.data_ptr(), ptrs, len(ptrs), row_scale.data_ptr(),
                                              ctypes.c_float(w_scale), M, K, N, out.stride(0) if M > 1 else N,
                                              status.data_ptr() if status is not None else None,
                                              torch.cuda.current_stream(a.device).cuda_stream), "matmul_dequant")
    return out


class ProjectionGroup:
    """A fixed list of projections (a, w_packed, out) on one GPU, run with as few launches as possible:
    decode-regime members share one persistent kernel (ternix_b200_group_create / _run)."""

    def __init__(self, problems, peer_ptrs=None, prepacked=False):
        """problems: list of (a, w_packed, out); with prepacked=True the weights are prepack_k4() outputs.  peer_ptrs: optional list (one entry per problem) of lists of raw
        device addresses that receive the same C as `out` (peer GPUs' buffers), all lists of equal length."""
        import torch

        self._keep = []
        arr = (_Problem * len(problems))()
        for i, (a, w, out) in enumerate(problems):
            if not (a.is_cuda and w.is_cuda and out.is_cuda):
                raise ValueError("ProjectionGroup takes CUDA tensors")
            if a.dtype != torch.int8 or w.dtype != torch.uint8 or out.dtype != torch.int32:
                raise ValueError("A int8, W_packed uint8, out int32")
            if not (a.is_contiguous() and w.is_contiguous()) or a.dim() != 2 or w.dim() != 2:
                raise ValueError("A and W_packed must be contiguous 2-D tensors")
            M, K = a.shape
            N = w.shape[1] if prepacked else w.shape[1] * 4
            if w.shape[0] != ((K + 3) // 4 if prepacked else K) or tuple(out.shape) != (M, N) or \
                    (N > 1 and out.stride(1) != 1):
                raise ValueError("shape mismatch")
            arr[i] = _Problem(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, K, N,
                              out.stride(0) if M > 1 else max(N, out.stride(0)))
            self._keep.append((a, w, out))
        self.device = problems[0][0].device if problems else None
        handle = ctypes.c_void_p()
        n_peers = len(peer_ptrs[0]) if peer_ptrs else 0
        with torch.cuda.device(self.device):
            if prepacked:
                _check(lib.ternix_b200_group_create_prepacked(ctypes.byref(handle), arr, len(problems)),
                       "group_create_prepacked")
            elif n_peers:
                flat = (ctypes.c_void_p * (len(problems) * n_peers))(*[p for row in peer_ptrs for p in row])
                _check(lib.ternix_b200_group_create_ex(ctypes.byref(handle), arr, len(problems), flat, n_peers),
                       "group_create_ex")
            else:
                _check(lib.ternix_b200_group_create(ctypes.byref(handle), arr, len(problems)), "group_create")
        self._h = handle
        self.launches = lib.ternix_b200_group_launches(self._h)

    def run(self, status=None, stream=None):
        import torch

        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            _check(lib.ternix_b200_group_run(self._h, status.data_ptr() if status is not None else None,
                                             s.cuda_stream), "group_run")

    def close(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.ternix_b200_group_destroy(self._h)
        self._h = None

    def __del__(self):
        self.close()


def prepack_k4(w_packed):
    """Device tensor (K, N/4) uint8 in the packed format -> (ceil(K/4), N) uint8 in the decode-friendly layout
    (ternix_b200_prepack_k4): same bytes, the four k-rows of a group interleaved per packed byte column."""
    import torch

    if not w_packed.is_cuda or w_packed.dtype != torch.uint8 or w_packed.dim() != 2 or not w_packed.is_contiguous():
        raise ValueError("prepack_k4 takes a contiguous CUDA uint8 (K, N/4) tensor")
    K, N = w_packed.shape[0], w_packed.shape[1] * 4
    out = torch.empty(((K + 3) // 4, N), dtype=torch.uint8, device=w_packed.device)
    with torch.cuda.device(w_packed.device):
        _check(lib.ternix_b200_prepack_k4(w_packed.data_ptr(), out.data_ptr(), K, N,
                                          torch.cuda.current_stream(w_packed.device).cuda_stream), "prepack_k4")
    return out


# --------------------------------------------------------------------------- N-column sharding
@dataclass(frozen=True)
class ColumnShard:
    """Columns [n0, n0 + n_cols) of an N-column matrix owned by `rank` of `world`."""
    N: int
    world: int
    rank: int
    granule: int
    n0: int
    n_cols: int

    @property
    def n_pad(self) -> int:
        """Width of the equal-sized block every rank contributes to the all-gather."""
        return shard_columns(self.N, self.world, 0, self.granule).n_cols


def shard_columns(N: int, world: int, rank: int, granule: int = 64) -> ColumnShard:
    n0, nc = ctypes.c_int(), ctypes.c_int()
    _check(lib.ternix_b200_shard_columns(N, world, rank, granule, ctypes.byref(n0), ctypes.byref(nc)),
           "shard_columns")
    return ColumnShard(N, world, rank, granule, n0.value, nc.value)


def gathered_to_row_major(gathered: np.ndarray, N: int, granule: int = 64) -> np.ndarray:
    """Host-side mirror of ternix_b200_unpack_gathered for arrays already on the host: rank-major
    [world][M][n_pad] blocks -> row-major [M][N].  Layout bookkeeping only, no arithmetic."""
    world, M, n_pad = gathered.shape
    out = np.empty((M, N), dtype=gathered.dtype)
    for r in range(world):
        sh = shard_columns(N, world, r, granule)
        if sh.n_cols > n_pad:
            raise ValueError("gather blocks are narrower than the widest shard")
        out[:, sh.n0:sh.n0 + sh.n_cols] = gathered[r, :, :sh.n_cols]
    return out


# Rates behind should_shard(), measured on B200: what one GPU sustains on the paired tensor-core GEMM, and what one
# rank's epilogue stores sustain towards its peers over NVLink (per direction).
_GEMM_OPS_PER_S = 3.5e15
_PEER_STORE_BYTES_PER_S = 6.0e11
_GATHER_FIXED_S = 30e-6            # the stream barrier after the stores, the tail of stores behind the last tile


def should_shard(M: int, K: int, N: int, world: int, granule: int = 64, out_bytes: int = 4) -> bool:
    """Whether N-column sharding of one projection over `world` GPUs beats computing it whole on one GPU when every
    GPU needs the full C.  Sharding divides the compute by `world` but each rank must ship its columns to world - 1
    peers and all ranks meet at a barrier: per step max(compute / world, out_bytes * M * N * (world - 1) / world /
    link) + a fixed cost, against compute.  With int32 outputs that favours sharding only for large products with
    deep K (K > ~12000 * (world - 1) / world): config 3 (K = 8192) gains at 2 GPUs and is even at 4 (measured 0.43
    and 0.56 ms against 0.53-0.55 ms on one GPU), BitNet-2B projections
    (K = 2560, 6912; microseconds each) never do.  Small or skinny problems stay whole:
    a shard must keep at least one 256-column tile per rank and the problem must be in the tensor-core regime."""
    if not (world > 1 and M > 64 and N // world >= 256 and N % granule == 0):
        return False
    compute = 2.0 * M * K * N / _GEMM_OPS_PER_S
    gather = out_bytes * M * N * (world - 1) / world / _PEER_STORE_BYTES_PER_S
    return max(compute / world, gather) + _GATHER_FIXED_S < compute


def host_slab_rows(M: int, N: int) -> int:
    """Rows per slab of the host-operand step (forward_host): about 64 MB of int32 C per slab, at most 16 slabs,
    multiples of 256 rows (whole tiles of the prefill kernel), never more than M."""
    if M <= 0:
        return 0
    slabs = min(16, max(1, (4 * M * N) // (64 << 20)))
    rows = -(-M // slabs)
    return min(M, -(-rows // 256) * 256)


def gather_buffer_index(step: int) -> int:
    """Which of a rank's two gathered-C buffers step `step` fills.  Two buffers, because the barrier after a step
    only says that every rank's stores have landed: a fast rank may start its next step, and store into its peers,
    while a slow rank still reads the step before.  With alternating buffers those stores go to the buffer the slow
    rank is not reading; the buffer of step i is written again only by step i + 2, which no rank can start before
    every rank has passed the barrier of step i + 1, i.e. has enqueued its own step i + 1 behind its readers of
    step i."""
    return step & 1


class _DeviceBuffer:
    """A cudaMalloc'ed buffer owned by the library, viewable as a torch tensor and exportable to the
    other processes of the node (CUDA IPC)."""

    def __init__(self, nbytes: int):
        p = ctypes.c_void_p()
        _check(lib.ternix_b200_peer_alloc(ctypes.byref(p), nbytes), "peer_alloc")
        self.ptr, self.nbytes = p.value, nbytes

    def export(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        _check(lib.ternix_b200_peer_export(self.ptr, buf), "peer_export")
        return buf.raw

    def as_tensor(self, shape, dtype, device):
        import torch

        itemsize = torch.empty((), dtype=dtype).element_size()
        if dtype == torch.bfloat16:          # no array-interface code for bfloat16: view 16-bit words, reinterpret
            return self.as_tensor(shape, torch.int16, device).view(torch.bfloat16)
        typestr = {torch.int32: "<i4", torch.int8: "|i1", torch.uint8: "|u1", torch.int16: "<i2"}[dtype]
        strides = []
        acc = itemsize
        for d in reversed(shape):
            strides.insert(0, acc)
            acc *= d
        view = type("_View", (), {"__cuda_array_interface__": {
            "shape": tuple(shape), "typestr": typestr, "data": (self.ptr, False), "version": 3,
            "strides": tuple(strides)}})()
        t = torch.as_tensor(view, device=device)
        t._ternix_owner = self          # keep the allocation alive as long as the view
        return t

    def free(self):
        if self.ptr and lib is not None:
            lib.ternix_b200_peer_free(self.ptr)
        self.ptr = None


class PeerBarrier:
    """A barrier between the ranks of a torch.distributed group on the current CUDA stream, made of one small kernel
    per rank (ternix_b200_peer_barrier): every rank raises a flag in every peer's memory and waits for theirs.  When
    it has passed on a rank, every rank's kernels enqueued before its own call have finished and their stores into
    this rank's memory are visible.  Collective: construct it and call it on every rank, equally often.
    A peer that does not arrive within the library's wait limit sets the timeout code in `status`."""

    def __init__(self, group=None, device=None):
        import torch
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.epoch = 0
        self._own = None
        self._arrays = None
        if self.world == 1:
            return
        with torch.cuda.device(self.device):
            self._own = _DeviceBuffer(256)
            flags = self._own.as_tensor((64,), torch.int32, self.device)
            flags.zero_()
            torch.cuda.synchronize(self.device)       # zeroed before any peer can learn the handle
            handles = [None] * self.world
            dist.all_gather_object(handles, self._own.export(), group=group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._own.ptr)
                else:
                    p = ctypes.c_void_p()
                    _check(lib.ternix_b200_peer_import(h, ctypes.byref(p)), "peer_import")
                    ptrs.append(p.value)
            self._arrays = (ctypes.c_void_p * self.world)(*ptrs)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def __call__(self, status=None):
        import torch

        if self.world == 1:
            return
        self.epoch += 1
        st = status if status is not None else self._status
        with torch.cuda.device(self.device):
            _check(lib.ternix_b200_peer_barrier(self._arrays, self.world, self.rank, self.epoch & 0xFFFFFFFF, 0,
                                                st.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream),
                   "peer_barrier")

    def timed_out(self) -> bool:
        """Whether a barrier without a caller's status word has run out of time so far (synchronises the stream)."""
        return self.world > 1 and int(self._status.item()) != 0


class ShardedTernaryLinear:
    """One projection W[K,N], N-column-sharded over the ranks of a torch.distributed group (one process
    per GPU).  Each rank keeps only its packed column shard on its GPU; forward(a) returns the full
    row-major C[M,N] on every rank.

    mode="peer" (default when world > 1): C lives in a buffer every rank maps from every other rank; the
        GEMM epilogue of each rank stores its columns into all of them (ternix_b200_matmul_bcast) and a
        flag barrier on the same stream (PeerBarrier) says when all of them have landed.  The transfer overlaps
        the main loop.
    mode="nccl": the baseline -- compute the local block, ncclAllGather equal-sized blocks, scatter to
        row-major with ternix_b200_unpack_gathered.
    """

    def __init__(self, w_packed_host: np.ndarray, group=None, granule: int = 64, device=None, mode: str = "peer"):
        import torch
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        K, n4 = w_packed_host.shape
        self.K, self.N = K, n4 * 4
        self.shard = shard_columns(self.N, self.world, self.rank, granule)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        local = slice_columns(w_packed_host, self.shard.n0, self.shard.n_cols)
        self.w_local = torch.from_numpy(local).to(self.device)
        self.mode = mode if self.world > 1 else "local"
        self._gather = None
        self._block = None
        self._M = None
        self._c_bufs = None
        self._c = None
        self._peer_ptrs = None
        self._barrier = None
        self._step = 0

    def local(self, a, out=None):
        """This rank's columns only: (M, n_cols) int32."""
        return matmul(a, self.w_local, out=out)

    # ---- peer mode plumbing: two C buffers per rank (see gather_buffer_index), mapped by all ranks
    def _map_peer_buffers(self, nbytes, n_buffers=2):
        """Allocates n_buffers exportable buffers on this rank and maps every peer's: returns (own buffers,
        ptrs[buffer][rank])."""
        import torch
        import torch.distributed as dist

        with torch.cuda.device(self.device):
            bufs = [_DeviceBuffer(nbytes) for _ in range(n_buffers)]
            handles = [None] * self.world
            dist.all_gather_object(handles, [b.export() for b in bufs], group=self.group)
            ptrs = []
            for b in range(n_buffers):
                row = []
                for r, hs in enumerate(handles):
                    if r == self.rank:
                        row.append(bufs[b].ptr)
                    else:
                        p = ctypes.c_void_p()
                        _check(lib.ternix_b200_peer_import(hs[b], ctypes.byref(p)), "peer_import")
                        row.append(p.value)
                ptrs.append(row)
        return bufs, ptrs

    def _setup_peer(self, M):
        import torch

        self._c_bufs, ptrs = self._map_peer_buffers(M * self.N * 4)
        self._c = [b.as_tensor((M, self.N), torch.int32, self.device) for b in self._c_bufs]
        # own buffer first, then the peers, each offset to this rank's first column
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        self._peer_ptrs = [(ctypes.c_void_p * self.world)(*[row[r] + 4 * self.shard.n0 for r in order]) for row in ptrs]
        self._M = M
        self._step = 0

    def stream_barrier(self, status=None):
        """A barrier on the current stream: when it has passed, every rank's kernels enqueued before it have finished
        and what they stored into this rank's buffers is visible.  The first call sets the flag arrays up (collective)."""
        if self.world > 1:
            if self._barrier is None:
                self._barrier = PeerBarrier(self.group, self.device)
            self._barrier(status)

    def forward(self, a, out=None, status=None, barrier=True):
        """Full row-major C[M, N] on every rank.  In peer mode the result is a view of one of two internal buffers
        that alternate from call to call: it stays valid until the call after the next one, and whatever reads it
        must be ordered on the calling stream before the next forward().  barrier=False leaves out the barrier
        that makes the peers' columns complete (for timing the pieces)."""
        import torch

        M = a.shape[0]
        if self.mode == "local":
            if out is None:
                out = torch.empty((M, self.N), dtype=torch.int32, device=a.device)
            return matmul(a, self.w_local, out=out, status=status)
        if self.mode == "peer":
            if self._M != M:
                if self._M is not None:
                    raise ValueError("peer mode keeps its C buffers: M must not change between calls")
                self._setup_peer(M)
            b = gather_buffer_index(self._step)
            self._step += 1
            s = torch.cuda.current_stream(a.device)
            if self.shard.n_cols:
                with torch.cuda.device(a.device):
                    _check(lib.ternix_b200_matmul_bcast(a.data_ptr(), self.w_local.data_ptr(), self._peer_ptrs[b],
                                                        self.world, M, self.K, self.shard.n_cols, self.N,
                                                        status.data_ptr() if status is not None else None,
                                                        s.cuda_stream), "matmul_bcast")
            if barrier:
                self.stream_barrier(status)      # every rank's stores of this step have landed
            if out is not None:
                out.copy_(self._c[b])
                return out
            return self._c[b]
        return self._forward_nccl(a, out, status)

    def forward_host(self, a_host, out_host=None, slab_rows=None, status=None):
        """The step with its operands in host memory: every rank passes the same activations (a CPU tensor, ideally
        pinned); a rank that passes `out_host` (a CPU int32 (M, N) tensor) gets the full C there.  Collective: every
        rank calls it, with the same M and slab_rows.  The rows are cut into slabs (about 64 MB of C each, multiples
        of 256 rows): the activations of slab j+1 go up while slab j is computed and gathered and slab j-1 comes down,
        so the call takes little more than the download of C.  On one GPU this is TernaryWeights.matmul_host.
        Synchronous."""
        import torch

        M = a_host.shape[0]
        if self.mode == "local":
            if getattr(self, "_handle", None) is None:
                self._handle = TernaryWeights(self.w_local)
            if out_host is None:
                out_host = torch.empty((M, self.N), dtype=torch.int32, pin_memory=True)
            return self._handle.matmul_host(a_host, out_host)
        if slab_rows is None:
            slab_rows = host_slab_rows(M, self.N)
        n_slabs = -(-M // slab_rows)
        dev = self.device
        hs = getattr(self, "_host_state", None)
        if hs is None or hs["rows"] != slab_rows:
            if hs is not None:
                raise ValueError("the slab extent is fixed by the first call (the gathered C buffers are kept)")
            hs = {"rows": slab_rows,
                  "a": [torch.zeros((slab_rows, self.K), dtype=torch.int8, device=dev) for _ in range(2)],
                  "stage": None,
                  "s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
                  "ev_in": [torch.cuda.Event() for _ in range(2)], "ev_fwd": [torch.cuda.Event() for _ in range(2)],
                  "ev_out": [torch.cuda.Event() for _ in range(2)]}
            self._host_state = hs
        if out_host is not None and hs["stage"] is None:
            hs["stage"] = [torch.empty((slab_rows, self.N), dtype=torch.int32, device=dev) for _ in range(2)]
        main = torch.cuda.current_stream(dev)
        hs["s_in"].wait_stream(main)
        for j in range(n_slabs):
            r0 = j * slab_rows
            ext = min(slab_rows, M - r0)
            b = j & 1
            with torch.cuda.stream(hs["s_in"]):
                if j >= 2:
                    hs["s_in"].wait_event(hs["ev_fwd"][b])        # the product of slab j-2 has read this buffer
                hs["a"][b][:ext].copy_(a_host[r0:r0 + ext], non_blocking=True)
                if ext < slab_rows:
                    hs["a"][b][ext:].zero_()
                hs["ev_in"][b].record(hs["s_in"])
            main.wait_event(hs["ev_in"][b])
            c = self.forward(hs["a"][b], status=status)           # gathered on every rank; valid until the call after next
            if out_host is not None:
                # a private copy, on the calling stream (the gather protocol wants the readers of a step there), so
                # that the download can still run while the peers store the slab after next into the same buffer
                if j >= 2:
                    main.wait_event(hs["ev_out"][b])
                hs["stage"][b][:ext].copy_(c[:ext], non_blocking=True)
            hs["ev_fwd"][b].record(main)
            if out_host is not None:
                hs["s_out"].wait_event(hs["ev_fwd"][b])
                with torch.cuda.stream(hs["s_out"]):
                    out_host[r0:r0 + ext].copy_(hs["stage"][b][:ext], non_blocking=True)
                    hs["ev_out"][b].record(hs["s_out"])
        main.wait_stream(hs["s_out"])
        main.wait_stream(hs["s_in"])
        main.synchronize()
        return out_host

    def forward_dequant(self, a, row_scale, w_scale: float, status=None):
        """bfloat16 C = (A x W) * row_scale[:, None] * w_scale on every rank.  With more than one rank the GEMM
        epilogue of each rank scales, rounds and stores its columns into all ranks' bfloat16 C: half the NVLink
        bytes of the int32 gather.  The result alternates between two buffers like forward()'s."""
        import torch

        M = a.shape[0]
        if self.world == 1:
            return matmul_dequant(a, self.w_local, row_scale, w_scale, status=status)
        if getattr(self, "_y_M", None) != M:
            if getattr(self, "_y_M", None) is not None:
                raise ValueError("the bfloat16 C buffers are kept: M must not change between calls")
            self._y_bufs, ptrs = self._map_peer_buffers(M * self.N * 2)
            self._y = [b.as_tensor((M, self.N), torch.bfloat16, self.device) for b in self._y_bufs]
            self._y_peers = [tuple(row[r] + 2 * self.shard.n0 for r in range(self.world) if r != self.rank) for row in ptrs]
            self._y_M = M
            self._y_step = 0
        b = gather_buffer_index(self._y_step)
        self._y_step += 1
        if self.shard.n_cols:
            matmul_dequant(a, self.w_local, row_scale, w_scale,
                           out=self._y[b][:, self.shard.n0:self.shard.n0 + self.shard.n_cols], status=status,
                           extra_dest_ptrs=self._y_peers[b])
        self.stream_barrier(status)
        return self._y[b]

    def _forward_nccl(self, a, out, status):
        import torch
        import torch.distributed as dist

        M = a.shape[0]
        # ---- NCCL baseline
        if out is None:
            out = torch.empty((M, self.N), dtype=torch.int32, device=a.device)
        n_pad = self.shard.n_pad
        if self._gather is None or self._gather.shape[1] != M:
            self._gather = torch.empty((self.world, M, n_pad), dtype=torch.int32, device=a.device)
            self._block = torch.zeros((M, n_pad), dtype=torch.int32, device=a.device)
        if self.shard.n_cols:
            matmul(a, self.w_local, out=self._block[:, : self.shard.n_cols], status=status)
        dist.all_gather_into_tensor(self._gather.view(-1), self._block.view(-1), group=self.group)
        s = torch.cuda.current_stream(a.device)
        _check(lib.ternix_b200_unpack_gathered(self._gather.data_ptr(), out.data_ptr(), M, self.N, out.stride(0),
                                               self.world, self.shard.granule, n_pad, s.cuda_stream),
               "unpack_gathered")
        return out


class ShardedProjectionSet:
    """Many projections at once (e.g. every linear layer of a model).  One process per GPU.  Each projection is
    N-column-sharded over the ranks where that pays off (shard="auto": should_shard(); shard=True: wherever the shape
    allows it; shard=False: never) and computed whole by every rank otherwise.  run() is one launch per regime on
    each rank (ternix_b200_group_run): the paired-CTA GEMM writes every sharded projection's columns into all ranks'
    outputs from its epilogue, and a 4-byte all-reduce on the stream is the barrier.  With sharded members the
    outputs live in two buffers that alternate from run to run (gather_buffer_index): the tensors run() returns stay
    valid until the run after the next one.
    """

    def __init__(self, weights_host, activations, group=None, granule: int = 64, device=None, shard="auto"):
        """weights_host: list of packed (K, N/4) uint8 arrays; activations: list of (M, K) int8 CUDA tensors."""
        import torch
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.count = len(weights_host)
        plans, offsets, total = [], [], 0
        for w, a in zip(weights_host, activations):
            K, N = w.shape[0], w.shape[1] * 4
            M = a.shape[0]
            if shard == "auto":
                sharded = should_shard(M, K, N, self.world, granule)
            else:
                sharded = bool(shard) and self.world > 1 and M > 16 and N // self.world >= 256 and N % granule == 0
            sh = shard_columns(N, self.world, self.rank, granule) if sharded else ColumnShard(N, 1, 0, granule, 0, N)
            plans.append((M, K, N, sharded, sh))
            offsets.append(total)
            total += M * N * 4
            total = (total + 255) & ~255
        self.any_sharded = any(p[3] for p in plans)
        self.sharded_count = sum(1 for p in plans if p[3])
        n_buffers = 2 if self.any_sharded else 1
        with torch.cuda.device(self.device):
            self._bufs = [_DeviceBuffer(max(total, 256)) for _ in range(n_buffers)]
            ptrs = [[b.ptr] for b in self._bufs]
            if self.world > 1 and self.any_sharded:
                handles = [None] * self.world
                dist.all_gather_object(handles, [b.export() for b in self._bufs], group=self.group)
                ptrs = []
                for bi in range(n_buffers):
                    row = []
                    for r, hs in enumerate(handles):
                        if r == self.rank:
                            row.append(self._bufs[bi].ptr)
                        else:
                            p = ctypes.c_void_p()
                            _check(lib.ternix_b200_peer_import(hs[bi], ctypes.byref(p)), "peer_import")
                            row.append(p.value)
                    ptrs.append(row)
        others = [r for r in range(self.world) if r != self.rank]
        self._w_local = []
        for (M, K, N, sharded, sh), w in zip(plans, weights_host):
            local = slice_columns(w, sh.n0, sh.n_cols) if sharded else w
            self._w_local.append(torch.from_numpy(np.ascontiguousarray(local)).to(self.device))
        self._outputs, self._groups = [], []
        for bi in range(n_buffers):
            outputs, problems, peer_rows = [], [], []
            for (M, K, N, sharded, sh), off, w_dev, a in zip(plans, offsets, self._w_local, activations):
                view = _OffsetView(self._bufs[bi], off).as_tensor((M, N), torch.int32, self.device)
                outputs.append(view)
                if sh.n_cols == 0:
                    continue
                problems.append((a, w_dev, view[:, sh.n0:sh.n0 + sh.n_cols]))
                if self.any_sharded:
                    # sharded: the same columns in every peer's buffer; unsharded: nobody else needs them, but the
                    # table wants equally many pointers per problem, so point the "peers" at this rank's own C
                    base = [ptrs[bi][r] if sharded else self._bufs[bi].ptr for r in others]
                    peer_rows.append([b + off + 4 * sh.n0 for b in base])
            self._outputs.append(outputs)
            self._groups.append(ProjectionGroup(problems, peer_ptrs=peer_rows if self.any_sharded else None))
        self.outputs = self._outputs[0]
        self.launches = self._groups[0].launches
        self._barrier = PeerBarrier(self.group, self.device) if self.world > 1 and self.any_sharded else None
        self._step = 0

    def run(self, status=None):
        b = gather_buffer_index(self._step) if self.any_sharded else 0
        self._step += 1
        self._groups[b].run(status=status)
        if self._barrier is not None:
            self._barrier(status)
        self.outputs = self._outputs[b]
        return self.outputs


class _OffsetView:
    """A window into a _DeviceBuffer (same lifetime), viewable as a torch tensor."""

    def __init__(self, buf: "_DeviceBuffer", offset: int):
        self._buf, self.ptr = buf, buf.ptr + offset

    def as_tensor(self, shape, dtype, device):
        return _DeviceBuffer.as_tensor(self, shape, dtype, device)
