"""Property tests (hypothesis) of the host side: packing, column slicing and the shard plan, against the oracle
and against plain numpy, on arbitrary small shapes."""
import numpy as np
from hypothesis import given, settings, strategies as st

import oracle_lib
import ternixengine_b200 as tb


@settings(max_examples=60, deadline=None)
@given(k=st.integers(1, 40), n4=st.integers(1, 30), seed=st.integers(0, 2**31 - 1))
def test_pack_unpack_roundtrip_and_oracle_bytes(k, n4, seed):
    w = np.random.default_rng(seed).integers(-1, 2, size=(k, 4 * n4), dtype=np.int8)
    p = tb.pack_ternary(w)
    assert p.shape == (k, n4) and np.array_equal(p, oracle_lib.pack(w))
    assert np.array_equal(tb.unpack_ternary(p), w)
    # every byte only uses the codes 00, 01, 11
    fields = (p[..., None] >> np.array([0, 2, 4, 6], dtype=np.uint8)) & 3
    assert not (fields == 2).any()


@settings(max_examples=60, deadline=None)
@given(k=st.integers(1, 20), n4=st.integers(1, 40), a=st.integers(0, 39), b=st.integers(0, 40), seed=st.integers(0, 10**6))
def test_slice_columns_equals_packing_the_slice(k, n4, a, b, seed):
    lo, hi = sorted((min(a, n4), min(b, n4)))
    w = np.random.default_rng(seed).integers(-1, 2, size=(k, 4 * n4), dtype=np.int8)
    got = tb.slice_columns(tb.pack_ternary(w), 4 * lo, 4 * (hi - lo))
    want = tb.pack_ternary(np.ascontiguousarray(w[:, 4 * lo:4 * hi])) if hi > lo else np.empty((k, 0), np.uint8)
    assert np.array_equal(got, want)


@settings(max_examples=200, deadline=None)
@given(n4=st.integers(0, 5000), world=st.integers(1, 8), g4=st.integers(1, 64))
def test_shard_plan_is_a_partition(n4, world, g4):
    N, granule = 4 * n4, 4 * g4
    shards = [tb.shard_columns(N, world, r, granule) for r in range(world)]
    assert shards[0].n0 == 0
    assert sum(s.n_cols for s in shards) == N
    for s0, s1 in zip(shards, shards[1:]):
        assert s0.n0 + s0.n_cols == s1.n0 and s0.n_cols >= s1.n_cols
    assert all(s.n0 % granule == 0 or s.n_cols == 0 for s in shards)
    assert all(s.n_cols <= shards[0].n_pad for s in shards)


@settings(max_examples=30, deadline=None)
@given(m=st.integers(1, 6), k=st.integers(1, 50), n4=st.integers(1, 12), seed=st.integers(0, 10**6))
def test_oracle_variants_agree_with_numpy(m, k, n4, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-1, 2, size=(k, 4 * n4), dtype=np.int8)
    expect = a.astype(np.int32) @ w.astype(np.int32)
    wp = oracle_lib.pack(w).reshape(k, n4)
    for variant in ("scalar", "naive", "fast"):
        assert np.array_equal(oracle_lib.matmul(a, wp, variant), expect)
    if n4 % 2 == 0:
        assert np.array_equal(oracle_lib.matmul(a, wp, "avx2_semantics"), expect)
