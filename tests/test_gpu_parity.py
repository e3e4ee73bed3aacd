"""Parity of the CUDA path with the CPU oracle, bit for bit, through the C ABI.  Needs a B200."""
import os
import sys

import numpy as np
import pytest

import oracle_lib
import ternixengine_b200 as tb

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cases.npz"))
CASES = [str(n) for n in GOLDEN["names"]]


def device_matmul(a, wp, kernel="auto", pad_cols=0):
    """Upload, run one kernel through ternix_b200_matmul_ex into a poisoned C, download; checks the status word."""
    import torch
    da = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dw = torch.from_numpy(np.ascontiguousarray(wp)).cuda()
    M, N = a.shape[0], wp.shape[1] * 4
    full = torch.full((M, N + pad_cols), -999, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tb.matmul(da, dw, out=full[:, :N], kernel=kernel, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded device-side wait ran out"
    got = full.cpu().numpy()
    if pad_cols:
        assert (got[:, N:] == -999).all(), "kernel wrote outside its columns"
    return got[:, :N]


def kernels_for(M, K, N):
    ks = ["generic"]
    if N % 64 == 0 and M <= 16:
        ks.append("gemv")
    if N % 64 == 0 and K % 16 == 0:
        ks.append("gemm_tc")
        if K >= 16:
            ks.append("decode_mma")
            if M <= 64:
                ks.append("skinny_tc")
    return ks + ["auto"]


def assert_same(got, expect, what):
    if not np.array_equal(got, expect):
        bad = np.argwhere(got != expect)
        i, j = bad[0]
        raise AssertionError(f"{what}: {len(bad)} of {got.size} entries differ; first at ({i},{j}): "
                             f"got {got[i, j]}, expect {expect[i, j]}; rows {sorted(set(bad[:, 0]))[:8]} "
                             f"cols {sorted(set(bad[:, 1]))[:16]}")


# ---------------------------------------------------------------- the reference's own test cases
@pytest.mark.parametrize("name", CASES)
def test_golden_cases_all_kernels(name):
    a, wp, c = GOLDEN[name + "/A"], GOLDEN[name + "/Wp"], GOLDEN[name + "/C"]
    M, K = a.shape
    N = wp.shape[1] * 4
    for kern in kernels_for(M, K, N):
        assert_same(device_matmul(a, wp, kern), c, f"{name} [{kern}]")


def test_host_entry_point_and_python_module():
    sys.path.insert(0, os.path.join(ROOT, "ternixengine_b200"))
    import ternix_engine as te
    rng = np.random.default_rng(3)                       # tests/test_python_binding.py:14-41
    for (m, k, n) in [(1, 8, 8), (5, 33, 24), (64, 256, 128), (128, 256, 192)]:
        a = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
        w = rng.integers(-1, 2, size=(k, n), dtype=np.int8)
        expect = a.astype(np.int32) @ w.astype(np.int32)
        packed = te.pack_ternary(w)
        for impl in ("naive", "scalar", "avx2", "avx2_blocked", "cuda_naive", "cuda_tiled", "b200_generic"):
            assert_same(te.ternary_matmul(a, packed, impl), expect, f"{impl} {m}x{k}x{n}")
        assert_same(te.ternary_matmul(a, packed), expect, "default impl")
        assert_same(tb.ternary_matmul_host(a, packed), expect, "ctypes host entry")


# ---------------------------------------------------------------- BASELINE configs
def synth(M, K, N, seed, lo=-128):
    return tb.synth_activations((M, K), seed, lo=lo), tb.synth_packed_weights(K, N, seed + 1000)


def test_config1_bitnet_gemv():
    a, wp = synth(1, 2560, 6912, 11)
    expect = oracle_lib.matmul(a, wp, "scalar")
    if oracle_lib.have_ref():
        assert_same(oracle_lib.ref_matmul(a, wp, "avx2_blocked"), expect, "reference avx2_blocked vs oracle")
    for kern in ("gemv", "gemm_tc", "generic", "auto"):
        assert_same(device_matmul(a, wp, kern), expect, f"config1 [{kern}]")


@pytest.mark.parametrize("plan", ["16,1", "16,2", "16,4", "16,8", "32,1", "32,2", "32,4", "32,8"])
def test_gemv_every_split_plan(plan, option):
    option("gemv_plan", plan)
    for (m, k, n) in [(1, 2560, 6912), (3, 1000, 320), (16, 4096, 1024), (2, 64, 64), (5, 8200, 192)]:
        a, wp = synth(m, k, n, 7 * m + n)
        assert_same(device_matmul(a, wp, "gemv", pad_cols=8), oracle_lib.matmul(a, wp), f"gemv plan {plan} {m}x{k}x{n}")


def test_config2_skinny_gemm():
    a, wp = synth(32, 4096, 11008, 21, lo=-127)
    expect = oracle_lib.matmul(a, wp)
    if oracle_lib.have_ref():
        assert_same(oracle_lib.ref_matmul(a, wp, "avx2_blocked"), expect, "reference avx2_blocked vs oracle")
    for kern in ("skinny_tc", "gemm_tc", "decode_mma", "generic", "auto"):
        assert_same(device_matmul(a, wp, kern), expect, f"config2 [{kern}]")
    assert tb.select_kernel(32, 4096, 11008) == tb.KERNELS["decode_mma"]


@pytest.mark.parametrize("slices", ["", "SLICES=1", "SLICES=3", "SLICES=1000", "CLUSTER=0", "CLUSTER=2", "CLUSTER=4",
                                    "CLUSTER=8"])
def test_decode_mma_rows_slices_and_edges(option, slices):
    """Batched decode on mma.sync: every row count of a row group and across row groups, K not a multiple of the
    64-row stage, column tails, unaligned and padded C, the largest magnitudes; with the automatic plan, with forced
    K-slice counts (whole-K stores and sliced adds into a zeroed C) and with forced cluster sizes (slices reduced
    through distributed shared memory, some of them empty)."""
    if slices:
        key, value = slices.split("=")
        option("mma_" + key.lower(), value)
    for (m, k, n, pad) in [(1, 64, 64, 0), (2, 2560, 6912, 0), (3, 1040, 320, 1), (7, 4112, 1088, 0), (15, 16, 64, 3),
                           (16, 6912, 2560, 0), (17, 272, 576, 0), (33, 8192, 128, 4), (64, 1024, 2112, 0),
                           (100, 144, 704, 0)]:
        a, wp = synth(m, k, n, 40 + m + k)
        assert_same(device_matmul(a, wp, "decode_mma", pad_cols=pad), oracle_lib.matmul(a, wp),
                    f"decode_mma slices={slices!r} {m}x{k}x{n} pad {pad}")
    m, k, n = 16, 8192, 512
    a = np.full((m, k), -128, dtype=np.int8)
    wp = tb.pack_ternary(np.full((k, n), -1, dtype=np.int8))
    assert_same(device_matmul(a, wp, "decode_mma"), np.full((m, n), 128 * k, dtype=np.int32), "decode_mma worst case")


@pytest.mark.parametrize("bn", ["128", "256", "2", "3"])
def test_gemm_tc_tile_widths_and_ragged_edges(bn, option):
    # 128 / 256: single-CTA tiles; 2: paired CTAs, weights expanded into shared memory; 3: paired CTAs, weights decoded
    # into tensor memory (the default)
    option("tc_bn", "2" if bn in ("2", "3") else bn)
    option("tc3", "1" if bn == "3" else "0")
    for (m, k, n) in [(128, 128, 256), (128, 512, 128), (256, 1024, 512), (300, 2064, 832), (1, 16, 64),
                      (129, 144, 320), (640, 4096, 1024), (1000, 272, 1984)]:
        a, wp = synth(m, k, n, m + k + n)
        assert_same(device_matmul(a, wp, "gemm_tc", pad_cols=4), oracle_lib.matmul(a, wp), f"gemm_tc bn={bn} {m}x{k}x{n}")
    # a pitch that is not a multiple of 16 bytes: no TMA view of C, no vector stores
    a, wp = synth(300, 272, 576, 99)
    assert_same(device_matmul(a, wp, "gemm_tc", pad_cols=3), oracle_lib.matmul(a, wp), f"gemm_tc bn={bn} odd pitch")


@pytest.mark.parametrize("tile_rows", ["128", "256"])
def test_prefill_kernel_tile_forms(tile_rows, option):
    """Both tile forms of the tensor-memory prefill kernel on products of any row count: the 128-row form alternates
    between two accumulators (several tiles per CTA pair here), the 256-row form pads products with few rows."""
    option("tc_tile_rows", tile_rows)
    for (m, k, n) in [(100, 4096, 1024), (129, 272, 1984), (300, 1040, 832), (512, 2560, 2560), (384, 528, 45056)]:
        a, wp = synth(m, k, n, 7 * m + k + n)
        assert_same(device_matmul(a, wp, "gemm_tc", pad_cols=4), oracle_lib.matmul(a, wp),
                    f"gemm_tc tile_rows={tile_rows} {m}x{k}x{n}")
        assert tb.last_launched_kernel() == "ternary_gemm_tc3_kernel"


def test_prefill_kernel_deepest_k():
    """The largest K the scaled accumulators allow (64 * 128 * K < 2^31) at the worst-case magnitudes."""
    m, k, n = 256, 262128, 256
    a = np.full((m, k), -128, dtype=np.int8)
    wp = np.full((k, n // 4), 0xFF, dtype=np.uint8)
    assert (device_matmul(a, wp, "gemm_tc") == 128 * k).all()
    a[:] = 127
    a[::2, ::2] = -128
    expect = -a.astype(np.int64).sum(axis=1)
    got = device_matmul(a, wp, "gemm_tc")
    assert (got == expect[:, None]).all()


@pytest.mark.parametrize("shape", [(1, 3001, 1028), (7, 129, 4), (37, 4099, 2052), (255, 2561, 6916)])
def test_config4_ragged_and_worst_case(shape):
    m, k, n = shape
    a, wp = synth(m, k, n, sum(shape))
    expect = oracle_lib.matmul(a, wp, "scalar") if m * k * n < 4e8 else oracle_lib.matmul(a, wp)
    assert_same(device_matmul(a, wp, "auto", pad_cols=4), expect, f"config4 random {shape}")
    a2 = np.full((m, k), -128, dtype=np.int8)
    w2 = np.full((k, n // 4), 0xFF, dtype=np.uint8)
    got = device_matmul(a2, w2, "auto")
    assert (got == 128 * k).all(), f"config4 worst case {shape}: {np.unique(got)[:5]} != {128 * k}"


@pytest.mark.parametrize("shape", [(1, 8192, 1024), (16, 8192, 512), (128, 8192, 256), (256, 8192, 512)])
def test_worst_case_magnitude_fast_kernels(shape):
    """A == -128 and W == -1 on the scaled-accumulator kernels: 64 * 128 * K stays inside int32."""
    m, k, n = shape
    a = np.full((m, k), -128, dtype=np.int8)
    wp = np.full((k, n // 4), 0xFF, dtype=np.uint8)
    for kern in kernels_for(m, k, n):
        assert (device_matmul(a, wp, kern) == 128 * k).all(), f"{kern} {shape}"
    a[:] = 127
    for kern in kernels_for(m, k, n):
        assert (device_matmul(a, wp, kern) == -127 * k).all(), f"{kern} {shape} (+127)"


BITNET_LAYER = [("q", 2560, 2560), ("k", 2560, 640), ("v", 2560, 640), ("o", 2560, 2560),
                ("gate", 2560, 6912), ("up", 2560, 6912), ("down", 6912, 2560)]


@pytest.mark.parametrize("M", [1, 256])
def test_config5_bitnet_projection_set_one_layer(M):
    for i, (name, k, n) in enumerate(BITNET_LAYER):
        a, wp = synth(M, k, n, 100 * M + i)
        assert_same(device_matmul(a, wp, "auto"), oracle_lib.matmul(a, wp), f"config5 {name} M={M}")


def test_config3_prefill_gemm_full_size():
    """4096 x 8192 x 28672 on one GPU: every entry of C against the reference's AVX2 kernel, then size-independent
    properties."""
    import torch
    M, K, N = 4096, 8192, 28672
    a, wp = synth(M, K, N, 31)
    da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = tb.matmul(da, dw, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # every entry against the reference's own AVX2 kernel, compiled from its sources (row bands over the host cores;
    # the plain-C port stands in when that build is absent): the gate the reference's benchmark applies,
    # benchmarks/bench_cuda.cu:69-81
    threads = os.cpu_count() or 1
    if oracle_lib.have_ref():
        expect = oracle_lib.ref_matmul(a, wp, "avx2_blocked", threads=threads)
    else:
        expect = oracle_lib.matmul(a, wp, "fast", threads=threads)
    got = c.cpu().numpy()
    assert_same(got, expect, "config3, whole C vs avx2_blocked")
    # and sampled rows against the unpacked-int GEMM of the reference's unit tests (tests/test_ternary_matmul.cpp:31-39)
    rows = np.r_[0:4, 2046:2050, 4092:4096]
    assert_same(got[rows], oracle_lib.matmul_unpacked(a[rows], tb.unpack_ternary(wp)), "config3 rows vs unpacked GEMM")
    del expect, got
    # the generic kernel shares no decode or MMA code with the tensor-core kernel: compare every entry
    c2 = tb.matmul(da, dw, kernel="generic")
    assert bool((c == c2).all()), "tensor-core and generic kernels disagree"
    # linearity in A: (A1 + A2) W == A1 W + A2 W for small-magnitude halves (no int8 overflow)
    a1 = (da >> 1)
    a2 = da - a1
    assert bool((tb.matmul(a1, dw) + tb.matmul(a2, dw) == c).all())
    # column-sum checksum: sum_j C[i,j] == sum_k A[i,k] * rowsum(W)[k]
    wsum = torch.from_numpy(tb.unpack_ternary(wp).astype(np.int32).sum(axis=1)).cuda()
    lhs = c.sum(dim=1, dtype=torch.int64)
    rhs = (da.to(torch.int64) * wsum.to(torch.int64)).sum(dim=1)
    assert bool((lhs == rhs).all())


def test_column_slice_output_pitch():
    """A shard can be written straight into its columns of a wider C (ldc > N)."""
    import torch
    a, wp = synth(130, 512, 1024, 5)
    expect = oracle_lib.matmul(a, wp)
    da = torch.from_numpy(a).cuda()
    wide = torch.full((130, 1024), -7, dtype=torch.int32, device="cuda")
    for r in range(4):
        sh = tb.shard_columns(1024, 4, r)
        dws = torch.from_numpy(tb.slice_columns(wp, sh.n0, sh.n_cols)).cuda()
        tb.matmul(da, dws, out=wide[:, sh.n0:sh.n0 + sh.n_cols])
    torch.cuda.synchronize()
    assert_same(wide.cpu().numpy(), expect, "column shards written in place")


def test_unpack_gathered_layout():
    import torch
    M, N, world, granule = 37, 6912, 8, 64
    c = np.random.default_rng(1).integers(-1000, 1000, size=(M, N), dtype=np.int32)
    n_pad = tb.shard_columns(N, world, 0, granule).n_cols
    g = np.zeros((world, M, n_pad), dtype=np.int32)
    for r in range(world):
        sh = tb.shard_columns(N, world, r, granule)
        g[r, :, :sh.n_cols] = c[:, sh.n0:sh.n0 + sh.n_cols]
    dg = torch.from_numpy(g).cuda()
    out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    rc = tb.lib.ternix_b200_unpack_gathered(dg.data_ptr(), out.data_ptr(), M, N, N, world, granule, n_pad,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert_same(out.cpu().numpy(), c, "unpack_gathered")


def test_k_zero_and_empty_shapes():
    import torch
    out = torch.full((3, 8), 5, dtype=torch.int32, device="cuda")
    rc = tb.lib.ternix_b200_matmul(None, None, out.data_ptr(), 3, 0, 8, None)
    torch.cuda.synchronize()
    assert rc == 0 and bool((out == 0).all())
    assert tb.lib.ternix_b200_matmul(None, None, None, 0, 5, 8, None) == 0


def test_legacy_tiled_contract_rejects_before_touching_memory():
    # tests/test_cuda_matmul.cu:41-43 through the exported C++ symbol
    import ctypes
    raw = ctypes.CDLL(os.path.join(ROOT, "ternixengine_b200", "libternix_b200.so"))
    sym = [l.split()[-1] for l in os.popen(f"nm -D {ROOT}/ternixengine_b200/libternix_b200.so").read().splitlines()
           if "mul_mat_ternary_cuda_tiled" in l][0]
    fn = getattr(raw, sym)
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    assert fn(None, None, None, 65, 64, 64, None) == 1          # cudaErrorInvalidValue


def test_projection_group_bitnet_layers_m1():
    """config 5 at M=1: two BitNet-shaped layers (14 projections) in one persistent launch."""
    import torch
    probs, expect = [], []
    for layer in range(2):
        for i, (name, k, n) in enumerate(BITNET_LAYER):
            a, wp = synth(1, k, n, 1000 * layer + i)
            expect.append(oracle_lib.matmul(a, wp, "scalar"))
            probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                          torch.full((1, n), -999, dtype=torch.int32, device="cuda")))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs)
    assert group.launches == 1
    for _ in range(2):                       # a group can be run again and again
        group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, "grouped GEMV")
    group.close()


@pytest.mark.parametrize("M", [2, 3, 7, 16])
def test_projection_group_mixed_rows_and_fallbacks(M):
    """Row groups, ragged K tails, a column tail, and members the persistent kernel cannot take."""
    import torch
    shapes = [(M, 2560, 640), (1, 1040, 320), (M, 6912, 2560), (M, 144, 64), (3, 4099, 2052), (64, 256, 128),
              (M, 8208, 128)]
    probs, expect = [], []
    for i, (m, k, n) in enumerate(shapes):
        a, wp = synth(m, k, n, 77 * M + i)
        expect.append(oracle_lib.matmul(a, wp))
        wide = torch.full((m, n + 8), -999, dtype=torch.int32, device="cuda")
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(), wide[:, :n]))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs)
    # one-row member: dp4a kernel; 2..16 rows: one mma.sync launch per row-group size (8 rows, 16 rows); the M = 64
    # member: the tensor-memory decode kernel; the member with ragged K and N runs on its own
    assert group.launches == 4
    group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, f"group member {tuple(a.shape)}")
        assert bool((out.base[:, out.shape[1]:] == -999).all()) if hasattr(out, "base") else True


def test_bcast_two_destinations_one_gpu():
    """The fused-gather entry point with two destination buffers on one GPU: both get the same exact C,
    neighbouring columns stay untouched (paired-CTA epilogue), and the copy fallback for small problems."""
    import ctypes
    import torch
    for (m, k, n) in [(300, 1024, 832), (512, 2048, 1024), (7, 129, 4), (16, 256, 128)]:
        a, wp = synth(m, k, n, m + n)
        expect = oracle_lib.matmul(a, wp)
        da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
        wide = [torch.full((m, n + 64), -5, dtype=torch.int32, device="cuda") for _ in range(2)]
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        ptrs = (ctypes.c_void_p * 2)(*[w.data_ptr() + 4 * 32 for w in wide])      # columns 32 .. 32+n of each
        rc = tb.lib.ternix_b200_matmul_bcast(da.data_ptr(), dw.data_ptr(), ptrs, 2, m, k, n, n + 64,
                                             status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        for w in wide:
            got = w.cpu().numpy()
            assert_same(got[:, 32:32 + n], expect, f"bcast {m}x{k}x{n}")
            assert (got[:, :32] == -5).all() and (got[:, 32 + n:] == -5).all()


@pytest.mark.parametrize("kernel,shape,launches", [("gemm_tc", (1024, 8192, 3584), 150), ("gemm_tc", (128, 4096, 2048), 100),
                                                   ("gemv", (1, 2560, 6912), 200), ("gemv", (4, 4096, 1024), 100)])
def test_repeated_launches_are_bit_identical(kernel, shape, launches):
    """Pipeline races show up as rare, launch-dependent errors: every one of many launches must equal the oracle."""
    import torch
    m, k, n = shape
    a, wp = synth(m, k, n, 3 * m + n)
    expect = torch.from_numpy(oracle_lib.matmul(a, wp)).cuda()
    da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = [torch.empty((m, n), dtype=torch.int32, device="cuda") for _ in range(2)]
    bad_launches = 0
    for i in range(launches):
        c = outs[i & 1]
        c.fill_(-1)
        tb.matmul(da, dw, out=c, kernel=kernel, status=status)
        bad_launches += int(bool((c != expect).any()))
    assert int(status.item()) == 0
    assert bad_launches == 0, f"{bad_launches} of {launches} launches differ from the oracle"


def test_repeated_group_runs_are_bit_identical():
    import torch
    probs, expect = [], []
    for i, (name, k, n) in enumerate(BITNET_LAYER * 3):
        a, wp = synth(1, k, n, 500 + i)
        expect.append(torch.from_numpy(oracle_lib.matmul(a, wp, "scalar")).cuda())
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                      torch.empty((1, n), dtype=torch.int32, device="cuda")))
    group = tb.ProjectionGroup(probs)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = 0
    for _ in range(100):
        for p in probs:
            p[2].fill_(-1)
        group.run(status=status)
        bad += sum(int(bool((p[2] != e).any())) for p, e in zip(probs, expect))
    assert int(status.item()) == 0 and bad == 0


def test_projection_group_prefill_members_share_one_launch():
    """config 5 at M=256: the seven projections of a BitNet-shaped layer in one launch of the paired-CTA GEMM,
    with a second destination per projection (as for a peer GPU) written by the same epilogue."""
    import torch
    probs, peers, expect = [], [], []
    for i, (name, k, n) in enumerate(BITNET_LAYER):
        a, wp = synth(256, k, n, 300 + i)
        expect.append(oracle_lib.matmul(a, wp))
        out = torch.full((256, n), -999, dtype=torch.int32, device="cuda")
        twin = torch.full((256, n), -998, dtype=torch.int32, device="cuda")
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(), out))
        peers.append(twin)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs, peer_ptrs=[[t.data_ptr()] for t in peers])
    assert group.launches == 1
    for _ in range(3):
        group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), twin, e in zip(probs, peers, expect):
        assert_same(out.cpu().numpy(), e, "grouped GEMM")
        assert_same(twin.cpu().numpy(), e, "grouped GEMM, second destination")
    group.close()


def test_projection_group_mixed_regimes():
    import torch
    shapes = [(1, 2560, 6912), (300, 1040, 832), (512, 8192, 256), (3, 4099, 2052), (64, 256, 128), (130, 144, 320)]
    probs, expect = [], []
    for i, (m, k, n) in enumerate(shapes):
        a, wp = synth(m, k, n, 40 + i)
        expect.append(oracle_lib.matmul(a, wp))
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                      torch.full((m, n), -999, dtype=torch.int32, device="cuda")))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs)
    assert group.launches == 1 + 1 + 2          # decode kernel, paired GEMM, and the ragged and M=64 members
    group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, f"group member {tuple(a.shape)}")


@pytest.mark.parametrize("tc3", ["0", "1"])
@pytest.mark.parametrize("shape", [(4096, 2048, 5120), (2304, 2048, 9216), (4000, 4096, 5056)])
def test_paired_kernels_partial_last_round(shape, tc3, option):
    """Shapes whose last round of tiles fills only part of the machine, through the paired kernel that expands weights
    into shared memory (tc3 = 0) and the default one that keeps them in tensor memory: bit-exact, launch after
    launch, including ragged M and N edges and a C wider than N."""
    import torch
    option("tc3", tc3)
    m, k, n = shape
    a, wp = synth(m, k, n, m + n)
    expect = torch.from_numpy(oracle_lib.matmul(a, wp)).cuda()
    da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    wide = torch.full((m, n + 8), -3, dtype=torch.int32, device="cuda")
    for i in range(20):
        wide.fill_(-3)
        tb.matmul(da, dw, out=wide[:, :n], kernel="gemm_tc", status=status)
        assert bool((wide[:, :n] == expect).all()), f"launch {i} differs"
        assert bool((wide[:, n:] == -3).all())
    assert int(status.item()) == 0


def test_group_run_inside_a_cuda_graph():
    """A projection set captured once and replayed as a CUDA graph (run() only launches)."""
    import torch
    probs, expect = [], []
    for i, (name, k, n) in enumerate(BITNET_LAYER):
        for m in (1, 256):
            a, wp = synth(m, k, n, 600 + 2 * i + m)
            expect.append(oracle_lib.matmul(a, wp))
            probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                          torch.full((m, n), -999, dtype=torch.int32, device="cuda")))
    group = tb.ProjectionGroup(probs)
    assert group.launches == 2
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        group.run(stream=s)                     # warm-up outside capture (function attributes, first launches)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            group.run(stream=s)
    for p in probs:
        p[2].fill_(-1)
    g.replay()
    torch.cuda.synchronize()
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, "graph replay")


@pytest.mark.parametrize("M", [1, 2, 4, 7])
def test_prepacked_weights_group(M):
    """Decode batch on weights in the K-interleaved prepack layout: identical results, ragged K and N tails."""
    import torch
    shapes = [(M, 2560, 6912), (M, 2560, 640), (1, 1040, 320), (M, 6912, 2560), (M, 144, 64), (M, 8192, 128)]
    probs, expect = [], []
    for i, (m, k, n) in enumerate(shapes):
        a, wp = synth(m, k, n, 55 * M + i)
        expect.append(oracle_lib.matmul(a, wp))
        dw = torch.from_numpy(wp).cuda()
        pre = tb.prepack_k4(dw)
        assert tuple(pre.shape) == ((k + 3) // 4, n)
        # the layout itself: word [r][b] holds bytes W[4r..4r+3][b]
        ref = np.zeros(((k + 3) // 4 * 4, n // 4), dtype=np.uint8)
        ref[:k] = wp
        ref = ref.reshape(-1, 4, n // 4).transpose(0, 2, 1).reshape(-1, n)
        assert np.array_equal(pre.cpu().numpy(), ref)
        probs.append((torch.from_numpy(a).cuda(), pre, torch.full((m, n), -999, dtype=torch.int32, device="cuda")))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs, prepacked=True)
    assert group.launches == 1
    for _ in range(2):
        group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, f"prepacked member {tuple(a.shape)}")
    with pytest.raises(ValueError):                                  # prefill-sized members are not taken
        big = torch.zeros((256, 64), dtype=torch.int8, device="cuda")
        tb.ProjectionGroup([(big, tb.prepack_k4(torch.zeros((64, 64), dtype=torch.uint8, device="cuda")),
                             torch.zeros((256, 256), dtype=torch.int32, device="cuda"))], prepacked=True)


def test_python_module_device_arrays():
    """ternix_engine.ternary_matmul on device arrays (__cuda_array_interface__): no host round trip, strided out."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "ternixengine_b200"))
    import ternix_engine as te
    for (m, k, n) in [(1, 2560, 6912), (300, 1040, 832), (7, 129, 4)]:
        a, wp = synth(m, k, n, 5 * m + n)
        expect = oracle_lib.matmul(a, wp)
        da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
        wide = torch.full((m, n + 4), -9, dtype=torch.int32, device="cuda")
        out = wide[:, :n]
        got = te.ternary_matmul(da, dw, "cuda_tiled", out=out, stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert got is out
        assert_same(out.cpu().numpy(), expect, f"device arrays {m}x{k}x{n}")
        assert bool((wide[:, n:] == -9).all())
    with pytest.raises(ValueError):
        te.ternary_matmul(da, dw)                                  # device input without `out`


# ---------------------------------------------------------------- host-pointer call, column-slab pipeline
@pytest.mark.parametrize("slab", ["512", "1024", "r256", "0"])
def test_host_call_pipelined_slabs(option, slab):
    """The host-pointer entry point cuts large products into column slabs on three streams; forced here on a small
    product (ragged last slab included) and switched off, all against the oracle."""
    option("host_slab", slab)
    for (m, k, n) in [(300, 512, 2304), (129, 256, 1088), (5, 64, 1024)]:
        a, wp = synth(m, k, n, 300 + m)
        expect = oracle_lib.matmul(a, wp)
        for _ in range(2):
            assert_same(tb.ternary_matmul_host(a, wp), expect, f"host call, slab {slab}, {m}x{k}x{n}")


def test_host_call_pipelined_default_threshold():
    """Above 64 MB of output the pipeline is on by default: same result as the device-pointer call."""
    import torch
    for (m, k, n) in [(4096, 256, 4608), (1024, 128, 16384 + 64)]:      # row slabs; column slabs
        a, wp = synth(m, k, n, 77)
        dc = tb.matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda())
        got = tb.ternary_matmul_host(a, wp)
        assert_same(got, dc.cpu().numpy(), "pipelined host call vs device call")
        rows = np.arange(0, m, 97)
        assert_same(got[rows], oracle_lib.matmul(a[rows], wp), "pipelined host call vs oracle (row sample)")


# ---------------------------------------------------------------- decode batch: both item widths
@pytest.mark.parametrize("words", ["32", "16"])
@pytest.mark.parametrize("shapes", [
    [(1, 2560, 6912)],
    [(1, 8192, 512), (1, 8192, 64)],                          # deepest K
    [(2, 2560, 640), (1, 4112, 1088), (2, 6912, 2560)],       # two-row groups, K not a multiple of the stage
    [(5, 2560, 1152), (16, 1040, 576), (4, 6912, 512)],       # four-row groups, several row groups per chunk
])
def test_decode_batch_item_widths(option, words, shapes):
    """The persistent decode kernel with 512-column items (128-byte rows, the default) and 256-column items
    (64-byte rows): transposing loads from a stage swizzled to match.  The oracle's bytes, run after run."""
    import torch
    option("group_words", words)
    probs, expect = [], []
    for i, (m, k, n) in enumerate(shapes):
        a, wp = synth(m, k, n, 900 + 7 * i + m)
        expect.append(torch.from_numpy(oracle_lib.matmul(a, wp)).cuda())
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                      torch.empty((m, n), dtype=torch.int32, device="cuda")))
    group = tb.ProjectionGroup(probs)
    rows = [m for (m, _, _) in shapes]          # one launch per kernel in use: dp4a (1 row), mma.sync (2..8, 9..64 rows)
    assert group.launches == any(m == 1 for m in rows) + any(2 <= m <= 8 for m in rows) + any(m > 8 for m in rows)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = 0
    for _ in range(10):
        for p in probs:
            p[2].fill_(-7)
        group.run(status=status)
        bad += sum(int(bool((p[2] != e).any())) for p, e in zip(probs, expect))
    assert int(status.item()) == 0 and bad == 0
    group.close()
