"""Pins the CPU oracle (oracle/ternary_oracle.c): against the committed golden vectors made from the
reference's own sources, against those sources compiled here when present, and against numpy."""
import os

import numpy as np
import pytest

import oracle_lib

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cases.npz"))
CASES = [str(n) for n in GOLDEN["names"]]


def test_pack_known_answer_bytes():
    # src/bitpack.cpp:10-11: {1,0,-1,1} -> 01 | 00<<2 | 11<<4 | 01<<6 = 0x71 ; {-1,0,1,0} -> 0x13
    vec, packed = GOLDEN["bitpack/vec"], GOLDEN["bitpack/packed"]
    assert list(packed) == [0x71, 0x13]
    assert np.array_equal(oracle_lib.pack(vec), packed)
    assert np.array_equal(oracle_lib.unpack(packed), vec)          # tests/test_bitpack.cpp:5-15
    assert np.array_equal(oracle_lib.pack(np.array([0, 0, 0, 0, 1, 1, 1, 1, -1, -1, -1, -1], dtype=np.int8)),
                          np.array([0x00, 0x55, 0xFF], dtype=np.uint8))


def test_pack_drops_tail_and_maps_out_of_domain_to_zero():
    w = np.array([1, -1, 2, -2, 1, 1, 1], dtype=np.int8)           # 7 values: one byte, tail of 3 dropped
    assert list(oracle_lib.pack(w)) == [0x0D]                      # 01 | 11<<2 | 00 | 00
    assert list(oracle_lib.unpack(np.array([0xAA], dtype=np.uint8))) == [0, 0, 0, 0]   # code 10 -> 0


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden(name):
    a, wp, c = GOLDEN[name + "/A"], GOLDEN[name + "/Wp"], GOLDEN[name + "/C"]
    w = oracle_lib.unpack(wp)
    assert np.array_equal(oracle_lib.pack(w), wp)
    assert np.array_equal(oracle_lib.matmul(a, wp, "scalar"), c)
    assert np.array_equal(oracle_lib.matmul(a, wp, "naive"), c)
    assert np.array_equal(oracle_lib.matmul(a, wp, "fast"), c)
    assert np.array_equal(oracle_lib.matmul_unpacked(a, w), c)
    if wp.shape[1] % 2 == 0:
        assert np.array_equal(oracle_lib.matmul(a, wp, "avx2_semantics"), c)
    assert np.array_equal(a.astype(np.int32) @ w.astype(np.int32), c)


def test_oracle_column_slices():
    name = "cuda_37x100x52_s2"
    a, wp, c = GOLDEN[name + "/A"], GOLDEN[name + "/Wp"], GOLDEN[name + "/C"]
    for n0, nc in [(0, 52), (0, 4), (48, 4), (12, 24)]:
        assert np.array_equal(oracle_lib.matmul_columns(a, wp, n0, nc, threads=3), c[:, n0:n0 + nc])


def test_worst_case_magnitude():
    # A == -128, W == -1 (every packed byte 0xFF): every C entry is exactly 128*K
    for (m, k, n) in [(1, 3001, 1028), (7, 129, 4)]:
        a = np.full((m, k), -128, dtype=np.int8)
        wp = np.full((k, n // 4), 0xFF, dtype=np.uint8)
        for variant in ("scalar", "fast"):
            assert (oracle_lib.matmul(a, wp, variant) == 128 * k).all()


needs_ref = pytest.mark.skipif(not oracle_lib.have_ref(), reason="oracle/_ref not built (no reference checkout)")


@needs_ref
@pytest.mark.parametrize("shape", [(1, 8, 8), (5, 33, 24), (13, 100, 40), (37, 129, 52), (64, 256, 128), (3, 70, 4)])
def test_oracle_matches_compiled_reference(shape):
    m, k, n = shape
    rng = np.random.default_rng(sum(shape))
    a = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-1, 2, size=(k, n), dtype=np.int8)
    wp = oracle_lib.pack(w)
    rp = np.empty_like(wp)
    oracle_lib.ref().ref_pack_ternary(oracle_lib._ptr(rp), oracle_lib._ptr(w), w.size)
    assert np.array_equal(wp, rp)
    expect = oracle_lib.ref_matmul(a, wp, "scalar")
    assert np.array_equal(oracle_lib.ref_matmul(a, wp, "naive"), expect)
    for variant in ("scalar", "naive", "fast"):
        assert np.array_equal(oracle_lib.matmul(a, wp, variant), expect)
    if n % 8 == 0:
        for kern in ("avx2", "avx2_blocked"):
            assert np.array_equal(oracle_lib.ref_matmul(a, wp, kern), expect)
        assert np.array_equal(oracle_lib.ref_matmul(a, wp, "avx2_blocked", threads=3), expect)
        assert np.array_equal(oracle_lib.matmul(a, wp, "avx2_semantics"), expect)


@needs_ref
def test_goldens_regenerate_identically():
    """The committed fixtures are what the reference's sources produce today."""
    for name in ("cpu_5x33x24_s3", "cuda_37x100x52_s2"):
        kind, dims, seed = name.split("_")
        m, k, n = map(int, dims.split("x"))
        a, w, wp = oracle_lib.ref_make_problem(m, k, n, int(seed[1:]), -127 if kind == "cpu" else -128)
        assert np.array_equal(a, GOLDEN[name + "/A"]) and np.array_equal(wp, GOLDEN[name + "/Wp"])
        assert np.array_equal(oracle_lib.ref_matmul(a, wp, "scalar"), GOLDEN[name + "/C"])
