"""The allocation-free decode batch (ternix_b200_gemv_batch_noalloc).

Who needs it: callers that cannot let a library call cudaMalloc for them -- a serving process whose device
memory belongs to its own pool allocator, code running under a fixed memory cap or in a latency-critical
section, hosts that forbid allocation after start-up.  The entry point keeps the kernel's tables in a fixed
array inside the library image, so the only device memory it touches besides that array is what the caller
passes in.

This file is collected last on purpose (its name sorts after the other test files): a run that stops at the
first failure has then already run everything else.  The test works both on its own in a fresh process and
after the rest of the suite; it compares the new entry point with the existing grouped entry point (and with
the CPU oracle) on two calls in a row that use different problem lists, bit for bit.
"""
import ctypes

import numpy as np
import pytest

import oracle_lib
import ternixengine_b200 as tb

pytestmark = pytest.mark.gpu

LAYER = [(2560, 2560), (2560, 640), (2560, 640), (2560, 2560), (2560, 6912), (2560, 6912), (6912, 2560)]


def _make(batch_shapes, seed):
    import torch
    probs, expect = [], []
    for i, (m, k, n) in enumerate(batch_shapes):
        a = tb.synth_activations((m, k), seed + i)
        wp = tb.synth_packed_weights(k, n, seed + 100 + i)
        expect.append(oracle_lib.matmul(a, wp))
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()))
    return probs, expect


def _run_noalloc(probs, outs, status):
    import torch
    arr = (tb._Problem * len(probs))()
    for i, ((a, w), out) in enumerate(zip(probs, outs)):
        m, k = a.shape
        n = w.shape[1] * 4
        arr[i] = tb._Problem(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, k, n, max(n, out.stride(0)))
    return tb.lib.ternix_b200_gemv_batch_noalloc(arr, len(probs), status.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)


def test_noalloc_batch_matches_grouped_entry_point_twice():
    import torch
    torch.cuda.set_device(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two calls in a row with different lists: the second must fully replace the tables of the first
    batches = [[(1, k, n) for (k, n) in LAYER] * 2 + [(3, 1040, 320), (16, 4096, 1024)],
               [(2, k, n) for (k, n) in LAYER[:5]] + [(1, 144, 64), (4, 8192, 128)]]
    for call, shapes in enumerate(batches):
        probs, expect = _make(shapes, 900 + 50 * call)
        outs_new = [torch.full((a.shape[0], w.shape[1] * 4), -999, dtype=torch.int32, device="cuda") for a, w in probs]
        outs_old = [torch.full_like(o, -777) for o in outs_new]
        rc = _run_noalloc(probs, outs_new, status)
        assert rc == tb.OK, tb.status_string(rc)
        group = tb.ProjectionGroup([(a, w, o) for (a, w), o in zip(probs, outs_old)])
        group.run(status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for i, (new, old, e) in enumerate(zip(outs_new, outs_old, expect)):
            assert torch.equal(new, old), f"call {call}, problem {i}: differs from the grouped entry point"
            assert np.array_equal(new.cpu().numpy(), e), f"call {call}, problem {i}: differs from the CPU oracle"
        group.close()


def test_noalloc_batch_limits_and_rejections():
    import torch
    torch.cuda.set_device(0)
    mp, mi, nbytes = ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    assert tb.lib.ternix_b200_gemv_batch_noalloc_limits(ctypes.byref(mp), ctypes.byref(mi), ctypes.byref(nbytes)) == 0
    assert (mp.value, mi.value) == (256, 4096) and 0 < nbytes.value <= 128 * 1024
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = torch.zeros((1, 64), dtype=torch.int8, device="cuda")
    w = torch.zeros((64, 16), dtype=torch.uint8, device="cuda")
    outs = [torch.zeros((1, 64), dtype=torch.int32, device="cuda") for _ in range(mp.value + 1)]
    assert _run_noalloc([(a, w)] * (mp.value + 1), outs, status) == tb.ERR_TOO_LARGE          # too many problems
    big = torch.zeros((64, 64), dtype=torch.int8, device="cuda")                                # M = 64: not decode regime
    assert _run_noalloc([(big, w)], [torch.zeros((64, 64), dtype=torch.int32, device="cuda")], status) == tb.ERR_UNSUPPORTED
    wide_w = torch.zeros((64, 8192), dtype=torch.uint8, device="cuda")                          # 64 chunks x 16/4 row groups
    a16 = torch.zeros((16, 64), dtype=torch.int8, device="cuda")
    many = [(a16, wide_w)] * 17                                                                  # 17 * 256 items > 4096
    outs = [torch.zeros((16, 32768), dtype=torch.int32, device="cuda") for _ in many]
    assert _run_noalloc(many, outs, status) == tb.ERR_TOO_LARGE
    assert tb.lib.ternix_b200_gemv_batch_noalloc(None, 0, None, None) == tb.OK
    torch.cuda.synchronize()
    # a member with K == 0 is an empty sum: its C is zeroed, as in the single-product calls
    a0 = torch.zeros((2, 0), dtype=torch.int8, device="cuda")
    w0 = torch.zeros((0, 16), dtype=torch.uint8, device="cuda")
    c0 = torch.full((2, 64), 7, dtype=torch.int32, device="cuda")
    prob = (tb._Problem * 1)(tb._Problem(a0.data_ptr(), w0.data_ptr(), c0.data_ptr(), 2, 0, 64, 64))
    assert tb.lib.ternix_b200_gemv_batch_noalloc(prob, 1, status.data_ptr(), torch.cuda.current_stream().cuda_stream) == tb.OK
    torch.cuda.synchronize()
    assert bool((c0 == 0).all())
    # a stream that is being captured is refused: the tables are uploaded from one fixed host buffer, which a graph
    # would read at replay time, after later calls have rewritten it
    s = torch.cuda.Stream()
    out = torch.zeros((1, 64), dtype=torch.int32, device="cuda")
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            prob = (tb._Problem * 1)(tb._Problem(a.data_ptr(), w.data_ptr(), out.data_ptr(), 1, 64, 64, 64))
            rc = tb.lib.ternix_b200_gemv_batch_noalloc(prob, 1, None, s.cuda_stream)
    assert rc == tb.ERR_UNSUPPORTED
    torch.cuda.synchronize()
