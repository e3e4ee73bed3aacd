"""ctypes access to the CPU checkers under oracle/ -- for tests, the smoke check and the benchmark's
CPU-baseline leg only.  Builds them with oracle/Makefile when they are missing."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_build", "libternary_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libternix_ref.so")

_sz, _vp, _i32, _u32 = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def build():
    subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)


_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build()
        lib = ctypes.CDLL(ORACLE_SO)
        for n in ("oracle_pack_ternary", "oracle_unpack_ternary", "oracle_interleave_offline"):
            getattr(lib, n).argtypes = [_vp, _vp, _sz]
            getattr(lib, n).restype = None
        for n in ("oracle_matmul_scalar", "oracle_matmul_naive", "oracle_matmul_avx2_semantics",
                  "oracle_matmul_unpacked"):
            getattr(lib, n).argtypes = [_vp, _vp, _vp, _sz, _sz, _sz]
            getattr(lib, n).restype = None
        lib.oracle_matmul_fast.argtypes = [_vp, _vp, _vp, _sz, _sz, _sz, _i32]
        lib.oracle_matmul_fast.restype = _i32
        lib.oracle_matmul_columns.argtypes = [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _i32]
        lib.oracle_matmul_columns.restype = _i32
        _oracle = lib
    return _oracle


def have_ref():
    return os.path.exists(REF_SO)


def ref():
    """The reference's own CPU sources compiled unmodified (None when the build is absent)."""
    global _ref
    if _ref is None:
        if not have_ref():
            return None
        lib = ctypes.CDLL(REF_SO)
        for n in ("ref_pack_ternary", "ref_unpack_ternary", "ref_interleave_offline"):
            getattr(lib, n).argtypes = [_vp, _vp, _sz]
            getattr(lib, n).restype = None
        lib.ref_matmul.argtypes = [_i32, _vp, _vp, _vp, _sz, _sz, _sz]
        lib.ref_matmul.restype = _i32
        lib.ref_matmul_threads.argtypes = [_i32, _vp, _vp, _vp, _sz, _sz, _sz, _i32]
        lib.ref_matmul_threads.restype = _i32
        lib.ref_make_problem.argtypes = [_sz, _sz, _sz, _u32, _i32, _vp, _vp, _vp]
        lib.ref_make_problem.restype = None
        _ref = lib
    return _ref


REF_KERNELS = {"naive": 0, "scalar": 1, "avx2": 2, "avx2_blocked": 3}


# ---- numpy-friendly wrappers ------------------------------------------------------------------
def pack(w):
    w = np.ascontiguousarray(w, dtype=np.int8)
    out = np.empty(w.size // 4, dtype=np.uint8)
    oracle().oracle_pack_ternary(_ptr(out), _ptr(w), w.size)
    return out.reshape(w.shape[0], -1) if w.ndim == 2 and w.shape[1] % 4 == 0 else out


def unpack(p, size=None):
    p = np.ascontiguousarray(p, dtype=np.uint8)
    size = p.size * 4 if size is None else size
    out = np.empty(size, dtype=np.int8)
    oracle().oracle_unpack_ternary(_ptr(out), _ptr(p), size)
    return out.reshape(p.shape[0], -1) if p.ndim == 2 else out


def matmul(a, wp, variant="fast", threads=0):
    """variant: scalar | naive | avx2_semantics | fast (unpack once + threaded unpacked GEMM)."""
    a = np.ascontiguousarray(a, dtype=np.int8)
    wp = np.ascontiguousarray(wp, dtype=np.uint8)
    M, K = a.shape
    N = wp.shape[1] * 4
    assert wp.shape[0] == K
    c = np.full((M, N), -999, dtype=np.int32)
    if variant == "fast":
        assert oracle().oracle_matmul_fast(_ptr(a), _ptr(wp), _ptr(c), M, K, N, threads) == 0
    else:
        getattr(oracle(), "oracle_matmul_" + variant)(_ptr(a), _ptr(wp), _ptr(c), M, K, N)
    return c


def matmul_columns(a, wp, n0, n_cols, threads=0):
    a = np.ascontiguousarray(a, dtype=np.int8)
    wp = np.ascontiguousarray(wp, dtype=np.uint8)
    M, K = a.shape
    N = wp.shape[1] * 4
    c = np.full((M, n_cols), -999, dtype=np.int32)
    assert oracle().oracle_matmul_columns(_ptr(a), _ptr(wp), _ptr(c), M, K, N, n0, n_cols, threads) == 0
    return c


def matmul_unpacked(a, w):
    a = np.ascontiguousarray(a, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    M, K = a.shape
    N = w.shape[1]
    c = np.full((M, N), -999, dtype=np.int32)
    oracle().oracle_matmul_unpacked(_ptr(a), _ptr(w), _ptr(c), M, K, N)
    return c


def ref_matmul(a, wp, kernel="avx2_blocked", threads=1):
    lib = ref()
    a = np.ascontiguousarray(a, dtype=np.int8)
    wp = np.ascontiguousarray(wp, dtype=np.uint8)
    M, K = a.shape
    N = wp.shape[1] * 4
    c = np.full((M, N), -999, dtype=np.int32)
    if threads == 1:
        rc = lib.ref_matmul(REF_KERNELS[kernel], _ptr(a), _ptr(wp), _ptr(c), M, K, N)
    else:
        rc = lib.ref_matmul_threads(REF_KERNELS[kernel], _ptr(a), _ptr(wp), _ptr(c), M, K, N, threads)
    assert rc == 0, rc
    return c


def ref_make_problem(M, K, N, seed, act_lo):
    lib = ref()
    a = np.empty((M, K), dtype=np.int8)
    w = np.empty((K, N), dtype=np.int8)
    wp = np.empty((K, N // 4), dtype=np.uint8)
    lib.ref_make_problem(M, K, N, seed, act_lo, _ptr(a), _ptr(w), _ptr(wp))
    return a, w, wp
