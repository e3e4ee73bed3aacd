"""Regenerates tests/golden/reference_cases.npz from the reference's own CPU sources.

Needs oracle/_ref/libternix_ref.so (built by `make -C oracle` where the reference checkout is
present).  Inputs are produced exactly as the reference's tests produce them -- one
std::mt19937(seed) feeding uniform_int_distribution for A and then W, then pack_ternary_weights --
and the expected outputs are computed by the reference's kernels:

  * tests/test_ternary_matmul.cpp:44-46   six shapes, seeds 1..6, A in [-127,127]
  * tests/test_ternary_matmul.cpp:61-69   M=4,K=4096,N=16, seed 99, A == -128
  * tests/test_cuda_matmul.cu:28-39       seven shapes, seeds 1..7, A in [-128,127]
  * tests/test_bitpack.cpp:6              the 8-weight round-trip vector

Stored per case: A, packed W, and C from `scalar`; the script asserts that naive, avx2 and avx2_blocked
(where N % 8 == 0) and a numpy int32 product on the unpacked W give the same C before writing anything.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib  # noqa: E402

CPU_TEST_SHAPES = [(1, 8, 8), (4, 16, 8), (5, 33, 24), (8, 64, 64), (13, 100, 40), (64, 256, 128)]
CUDA_TEST_CASES = [(64, 64, 64, 1), (37, 100, 52, 2), (128, 512, 256, 3),
                   (64, 64, 64, 4), (128, 256, 192, 5), (256, 1024, 512, 6), (64, 4096, 64, 7)]


def main():
    if oracle_lib.ref() is None:
        raise SystemExit("oracle/_ref/libternix_ref.so is missing: run `make -C oracle` next to the reference")
    out = {}
    names = []

    def add(name, a, w, wp):
        c = oracle_lib.ref_matmul(a, wp, "scalar")
        assert np.array_equal(c, oracle_lib.ref_matmul(a, wp, "naive")), name
        if wp.shape[1] % 2 == 0:
            assert np.array_equal(c, oracle_lib.ref_matmul(a, wp, "avx2")), name
            assert np.array_equal(c, oracle_lib.ref_matmul(a, wp, "avx2_blocked")), name
        assert np.array_equal(c, a.astype(np.int32) @ w.astype(np.int32)), name
        names.append(name)
        out[name + "/A"], out[name + "/Wp"], out[name + "/C"] = a, wp, c

    for seed, (m, k, n) in enumerate(CPU_TEST_SHAPES, start=1):
        add(f"cpu_{m}x{k}x{n}_s{seed}", *oracle_lib.ref_make_problem(m, k, n, seed, -127))
    a, w, wp = oracle_lib.ref_make_problem(4, 4096, 16, 99, -127)
    a[:] = -128
    add("cpu_extreme_4x4096x16_s99", a, w, wp)
    for (m, k, n, seed) in CUDA_TEST_CASES:
        add(f"cuda_{m}x{k}x{n}_s{seed}", *oracle_lib.ref_make_problem(m, k, n, seed, -128))

    vec = np.array([1, 0, -1, 1, -1, 0, 1, 0], dtype=np.int8)
    packed = np.empty(2, dtype=np.uint8)
    oracle_lib.ref().ref_pack_ternary(oracle_lib._ptr(packed), oracle_lib._ptr(vec), vec.size)
    out["bitpack/vec"], out["bitpack/packed"] = vec, packed
    out["names"] = np.array(names)
    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(names)} matmul cases, packed test vector = {[hex(b) for b in packed]}")


if __name__ == "__main__":
    main()
