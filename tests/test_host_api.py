"""CPU-side checks of the product library: it loads, exports the whole C ABI, packs byte-for-byte like
the oracle, plans shards, selects kernels, validates arguments -- and refuses to compute without a GPU."""
import ctypes
import os
import re
import sys

import numpy as np
import pytest

import oracle_lib
import ternixengine_b200 as tb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ternix_b200.h")).read()
    declared = set(re.findall(r"\b(ternix_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "header parse failed"
    assert declared == set(tb.EXPORTS)
    raw = ctypes.CDLL(os.path.join(ROOT, "ternixengine_b200", "libternix_b200.so"))
    for name in declared:
        assert hasattr(raw, name), name
    assert tb.lib.ternix_b200_version() >= 100
    assert tb.status_string(tb.ERR_TIMEOUT)


def test_cpp_api_symbols_present():
    """The reference's C++ names (include/ternix/*.h*) are exported with C++ linkage."""
    out = os.popen(f"nm -DC {ROOT}/ternixengine_b200/libternix_b200.so").read()
    for name in ("ternix::pack_ternary_weights", "ternix::unpack_ternary_weights", "ternix::interleave_weights_offline",
                 "ternix::mul_mat_ternary_naive", "ternix::mul_mat_ternary_scalar", "ternix::mul_mat_ternary_avx2",
                 "ternix::mul_mat_ternary_avx2_blocked", "ternix::mul_mat_ternary_cuda_naive",
                 "ternix::mul_mat_ternary_cuda_tiled", "ternix::mul_mat_ternary_cuda_host"):
        assert name + "(" in out, name


def test_pack_matches_oracle_bytes():
    rng = np.random.default_rng(0)
    w = rng.integers(-1, 2, size=(33, 24), dtype=np.int8)
    p = tb.pack_ternary(w)
    assert p.shape == (33, 6) and p.dtype == np.uint8
    assert np.array_equal(p, oracle_lib.pack(w))
    assert np.array_equal(tb.unpack_ternary(p), w)
    assert list(tb.pack_ternary(np.array([[1, 0, -1, 1, -1, 0, 1, 0]], dtype=np.int8))[0]) == [0x71, 0x13]
    assert list(tb.unpack_ternary(np.array([[0xAA]], dtype=np.uint8))[0]) == [0, 0, 0, 0]     # code 10 -> 0
    big = rng.integers(-1, 2, size=(1500, 2800), dtype=np.int8)                                 # threaded path
    assert np.array_equal(tb.pack_ternary(big), oracle_lib.pack(big))
    assert np.array_equal(tb.unpack_ternary(tb.pack_ternary(big)), big)


def test_pack_validation_errors():
    w = np.zeros((4, 8), dtype=np.int8)
    with pytest.raises(ValueError):
        tb.pack_ternary((w + 2).astype(np.int8))
    with pytest.raises(ValueError):
        tb.pack_ternary(np.zeros((4, 6), dtype=np.int8))
    with pytest.raises(ValueError):
        tb.pack_ternary(np.zeros(8, dtype=np.int8))


def test_interleave_is_identity():
    src = np.arange(40, dtype=np.uint8)
    dst = np.zeros_like(src)
    tb.lib.ternix_b200_interleave_offline(dst.ctypes.data, src.ctypes.data, 160)
    assert np.array_equal(dst, src)


def test_synth_distribution_and_determinism():
    a = tb.synth_activations((512, 1024), seed=5)
    assert a.min() == -128 and a.max() == 127
    assert np.array_equal(a, tb.synth_activations((512, 1024), seed=5))
    assert not np.array_equal(a, tb.synth_activations((512, 1024), seed=6))
    b = tb.synth_activations((512, 1024), seed=5, lo=-127)
    assert b.min() == -127 and b.max() == 127
    w = tb.synth_weights(512, 1024, seed=9)
    frac = [(w == v).mean() for v in (-1, 0, 1)]
    assert abs(frac[0] - 0.3) < 0.01 and abs(frac[1] - 0.4) < 0.01 and abs(frac[2] - 0.3) < 0.01
    assert np.array_equal(tb.synth_packed_weights(512, 1024, seed=9), oracle_lib.pack(w))


def test_slice_columns_is_a_valid_packed_shard():
    w = tb.synth_weights(37, 256, seed=1)
    p = tb.pack_ternary(w)
    for n0, nc in [(0, 256), (64, 64), (252, 4), (128, 0)]:
        assert np.array_equal(tb.slice_columns(p, n0, nc), oracle_lib.pack(np.ascontiguousarray(w[:, n0:n0 + nc]))
                              .reshape(37, nc // 4))
    with pytest.raises(ValueError):
        tb.slice_columns(p, 2, 8)


@pytest.mark.parametrize("N,world,granule", [(28672, 8, 64), (6912, 8, 64), (6912, 4, 64), (2560, 8, 64), (640, 8, 64),
                                             (1028, 3, 4), (64, 8, 64), (11008, 2, 256)])
def test_shard_plan_partitions_columns(N, world, granule):
    shards = [tb.shard_columns(N, world, r, granule) for r in range(world)]
    assert shards[0].n0 == 0 and sum(s.n_cols for s in shards) == N
    for a, b in zip(shards, shards[1:]):
        assert a.n0 + a.n_cols == b.n0
    widths = [s.n_cols for s in shards]
    assert widths == sorted(widths, reverse=True)                       # leading ranks are never narrower
    assert all(s.n0 % granule == 0 for s in shards if s.n_cols)
    assert max(widths) - min(w for w in widths if w or True) <= granule
    assert shards[0].n_pad == max(widths)


def test_kernel_selection_by_shape_and_alignment():
    sel = tb.select_kernel
    assert sel(1, 2560, 6912) == tb.KERNEL_GEMV
    assert sel(16, 4096, 11008) == tb.KERNEL_DECODE_MMA
    assert sel(32, 4096, 11008) == tb.KERNEL_DECODE_MMA                 # config 2
    assert sel(33, 4096, 11008) == tb.KERNEL_SKINNY_TC                  # three mma.sync passes or one tcgen05 pass
    assert sel(64, 4096, 11008) == tb.KERNEL_SKINNY_TC
    assert sel(65, 4096, 11008) == tb.KERNEL_GEMM_TC
    tb.set_option("skinny_rows", "2,64")                                # the row range of the tensor-memory decode kernel
    try:
        assert sel(32, 4096, 11008) == tb.KERNEL_SKINNY_TC
        tb.set_option("skinny_rows", "0,0")
        assert sel(64, 4096, 11008) == tb.KERNEL_DECODE_MMA
        assert sel(65, 4096, 11008) == tb.KERNEL_GEMM_TC
    finally:
        tb.set_option("skinny_rows", None)
    with pytest.raises(ValueError):
        tb.set_option("no_such_option", "1")
    assert sel(4, 2560, 6912, a_ptr=8) == tb.KERNEL_GEMV                # small M, A not 16-byte aligned: no TMA view of A
    assert sel(4096, 8192, 28672) == tb.KERNEL_GEMM_TC
    for (m, k, n) in [(1, 3001, 1028), (7, 129, 4), (37, 4099, 2052), (255, 2561, 6916)]:
        assert sel(m, k, n) == tb.KERNEL_GENERIC                        # packed rows are not 16-byte multiples
    assert sel(64, 100, 128) == tb.KERNEL_GENERIC                       # K % 16 != 0: no TMA view of A
    assert sel(64, 128, 128, a_ptr=8) == tb.KERNEL_GENERIC              # misaligned A
    assert sel(1, 300000, 64) == tb.KERNEL_GENERIC                      # too deep for the scaled accumulators
    assert sel(4, 8, 6) < 0                                             # N % 4 != 0


def test_benchmark_numpy_generator_matches_the_library():
    """bench.py's reference arm regenerates the inputs with numpy, without loading this library: same bytes."""
    sys.path.insert(0, ROOT)
    import bench
    for seed, shape in [(20240531, (7, 1000)), (5, (3, 4097))]:
        assert np.array_equal(bench.np_synth_activations(shape, seed), tb.synth_activations(shape, seed))
    for seed, (k, n) in [(20240532, (33, 1028)), (9, (257, 64))]:
        assert np.array_equal(bench.np_synth_packed_weights(k, n, seed), tb.synth_packed_weights(k, n, seed))


def test_shape_errors_come_before_pointer_checks():
    # the reference promises cudaErrorInvalidValue with null pointers (tests/test_cuda_matmul.cu:41-43)
    assert tb.lib.ternix_b200_matmul(None, None, None, 4, 8, 6, None) == tb.ERR_INVALID_SHAPE
    assert tb.lib.ternix_b200_matmul(None, None, None, -1, 8, 8, None) == tb.ERR_INVALID_SHAPE
    assert tb.lib.ternix_b200_matmul(None, None, None, 4, 8, 8, None) == tb.ERR_INVALID_ARG
    assert tb.lib.ternix_b200_matmul(None, None, None, 0, 8, 8, None) == tb.OK
    assert tb.lib.ternix_b200_matmul_ex(None, None, None, 4, 8, 8, 4, 0, None, None) == tb.ERR_INVALID_ARG   # ldc < N
    assert tb.lib.ternix_b200_matmul_ex(None, None, None, 4, 8, 8, 8, 9, None, None) == tb.ERR_INVALID_ARG   # selector
    assert tb.lib.ternix_b200_matmul_host(None, None, None, 4, 8, 6, 0) == tb.ERR_INVALID_SHAPE


def test_python_module_surface_and_errors():
    sys.path.insert(0, os.path.join(ROOT, "ternixengine_b200"))
    te = pytest.importorskip("ternix_engine")
    assert te.has_cuda is True
    rng = np.random.default_rng(0)
    w = rng.integers(-1, 2, size=(32, 24), dtype=np.int8)
    packed = te.pack_ternary(w)
    assert packed.shape == (32, 6) and packed.dtype == np.uint8          # tests/test_python_binding.py:21-25
    assert np.array_equal(te.unpack_ternary(packed), w)
    a = rng.integers(-128, 128, size=(4, 32), dtype=np.int8)
    with pytest.raises(ValueError):
        te.pack_ternary((w * 2).astype(np.int8))                          # tests/test_python_binding.py:44-49
    with pytest.raises(ValueError):
        te.ternary_matmul(a, packed, "nope")
    with pytest.raises(ValueError):
        te.ternary_matmul(a, te.pack_ternary(w[:, :12]), "avx2")          # N % 8 != 0 on an AVX2 name
    with pytest.raises(ValueError):
        te.ternary_matmul(a[:, :16], packed)                              # K mismatch
    m = te.Model("x")
    m.load()
    assert (m.vocab_size, m.hidden_size, m.num_layers) == (32000, 4096, 32)


def test_no_cpu_fallback_without_gpu():
    """Without a GPU the compute entry points fail loudly instead of computing on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    a = np.zeros((2, 8), dtype=np.int8)
    p = np.zeros((8, 2), dtype=np.uint8)
    with pytest.raises(tb.TernixError) as e:
        tb.ternary_matmul_host(a, p)
    assert e.value.status == tb.ERR_CUDA
