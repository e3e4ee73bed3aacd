"""The tensor-memory decode kernel (1..64 rows), the weight handle, the device-side packer, the bounded-wait
self-test, a second GPU in one process and the C++ boundary harness.  Needs a B200."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import oracle_lib
import ternixengine_b200 as tb
from test_gpu_parity import BITNET_LAYER, assert_same, device_matmul, synth

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("split", ["1", "2", "0"])
def test_skinny_tc_rows_shapes_and_edges(option, split):
    """Every batch class and its edges (1, 16, 17, 32, 33, 64, 65, 128 rows), K that is not a multiple of the 128-row stage,
    column counts that leave the second 128-column block of an item empty or ragged, a padded C, single-stage and
    deep problems; with the default plan (whole-K items unless blocks outnumber SMs), with blocks shared between CTAs
    wherever that evens the load (2: partial sums handed on through C, chains of up to three CTAs) and with whole
    blocks only (0)."""
    option("skinny_split", split)
    for (m, k, n, pad) in [(1, 64, 64, 0), (1, 2560, 6912, 0), (2, 2560, 640, 0), (3, 1040, 320, 1), (7, 4112, 1088, 0),
                           (15, 16, 64, 3), (16, 6912, 2560, 0), (17, 272, 576, 0), (32, 4096, 11008, 0),
                           (33, 8192, 128, 4), (48, 1024, 2112, 0), (64, 2560, 6912, 0), (64, 144, 704, 8),
                           (5, 65536, 256, 0), (65, 272, 576, 0), (100, 2560, 6912, 8), (128, 4096, 2048, 0),
                           (40, 512, 40960, 0)]:                            # the last one: more 256-column blocks than SMs
        a, wp = synth(m, k, n, 90 + m + k)
        assert_same(device_matmul(a, wp, "skinny_tc", pad_cols=pad), oracle_lib.matmul(a, wp),
                    f"skinny_tc split={split} {m}x{k}x{n} pad {pad}")
    for m in (1, 16, 64, 128):                             # largest magnitudes: 64 * 128 * K stays inside int32
        k, n = 8192, 512
        a = np.full((m, k), -128, dtype=np.int8)
        wp = np.full((k, n // 4), 0xFF, dtype=np.uint8)
        assert (device_matmul(a, wp, "skinny_tc") == 128 * k).all()
    with pytest.raises(ValueError):                        # more than 128 rows are the prefill kernels' business
        a, wp = synth(129, 256, 256, 1)
        device_matmul(a, wp, "skinny_tc")


@pytest.mark.parametrize("split", ["1", "2"])
@pytest.mark.parametrize("shape,launches", [((32, 4096, 11008), 200), ((16, 8192, 28672), 40), ((1, 2560, 6912), 200),
                                            ((64, 1024, 1536), 200)])
def test_skinny_tc_repeated_launches(option, shape, launches, split):
    """Races in the rings or in the hand-over of partial sums between CTAs would show as rare, launch-dependent
    errors: every one of many back-to-back launches (flags are reused with a new epoch each time) equals the oracle."""
    import torch
    option("skinny_split", split)
    m, k, n = shape
    a, wp = synth(m, k, n, 3 * m + n)
    expect = torch.from_numpy(oracle_lib.matmul(a, wp)).cuda()
    da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = [torch.empty((m, n), dtype=torch.int32, device="cuda") for _ in range(2)]
    bad = 0
    for i in range(launches):
        c = outs[i & 1]
        c.fill_(-1)
        tb.matmul(da, dw, out=c, kernel="skinny_tc", status=status)
        bad += int(bool((c != expect).any()))
    assert int(status.item()) == 0
    assert bad == 0, f"{bad} of {launches} launches differ from the oracle"
    assert tb.last_launched_kernel() == "ternary_skinny_tc_kernel"


def test_skinny_tc_two_streams_use_two_flag_slots():
    """Launches on different streams may overlap, so each stream has its own flags: interleaved launches of two
    different problems on two streams all equal the oracle."""
    import torch
    tb.set_option("skinny_split", "2")          # shared blocks, so that the flags are in use
    jobs = []
    for i, (m, k, n) in enumerate([(32, 4096, 11008), (8, 4096, 4096)]):
        a, wp = synth(m, k, n, 700 + i)
        jobs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(),
                     torch.from_numpy(oracle_lib.matmul(a, wp)).cuda(), torch.cuda.Stream()))
    torch.cuda.synchronize()
    outs = [[torch.full_like(j[2], -1) for _ in range(20)] for j in jobs]
    for r in range(20):
        for (da, dw, _, s), o in zip(jobs, outs):
            tb.matmul(da, dw, out=o[r], kernel="skinny_tc", stream=s)
    torch.cuda.synchronize()
    tb.set_option("skinny_split", None)
    for (_, _, expect, _), o in zip(jobs, outs):
        assert all(bool((x == expect).all()) for x in o)


@pytest.mark.parametrize("M", [2, 8, 16, 24, 64, 100])
@pytest.mark.parametrize("skinny_from", ["default", "2", "0"])
def test_projection_group_batched_decode(option, M, skinny_from):
    """config 5 at a few rows: one BitNet-shaped layer plus odd members in one group.  Members with several rows run
    on the tensor-memory decode kernel from 17 rows up (default), from 2 rows up, or never (then the mma.sync kernel
    takes them up to 64 rows and larger ones are launched one by one)."""
    import torch
    if skinny_from != "default":
        option("skinny_group_rows", skinny_from)
    lo = {"default": 17, "2": 2, "0": 129}[skinny_from]
    shapes = [(M, k, n) for (_, k, n) in BITNET_LAYER] + [(3, 1040, 320), (40, 144, 64), (1, 2560, 640)]
    probs, expect = [], []
    for i, (m, k, n) in enumerate(shapes):
        a, wp = synth(m, k, n, 31 * M + i)
        expect.append(oracle_lib.matmul(a, wp))
        wide = torch.full((m, n + 8), -999, dtype=torch.int32, device="cuda")
        probs.append((torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(), wide[:, :n]))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = tb.ProjectionGroup(probs)
    rows = [m for (m, _, _) in shapes]
    skinny_classes = {16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128 for m in rows if lo <= m <= 128}
    mma_sizes = {8 if m <= 8 else 16 for m in rows if 2 <= m < lo and m <= 64}
    singles = sum(1 for m in rows if m > 64 and m < lo)          # 65..128 rows without the tensor-memory kernel: one by one
    assert group.launches == 1 + len(skinny_classes) + len(mma_sizes) + singles
    for _ in range(3):
        for p in probs:
            p[2].fill_(-1)
        group.run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (a, w, out), e in zip(probs, expect):
        assert_same(out.cpu().numpy(), e, f"group member {tuple(a.shape)}")
    group.close()


@pytest.mark.parametrize("pdl", ["1", "0", "-1"])
def test_decode_batches_back_to_back_as_programmatic_dependents(option, pdl):
    """Decode batches launched back to back: with gemv_pdl the next grid starts while the previous one finishes and
    prefetches weights early, but reads activations and writes C only after it.  Each run's activations are the previous
    run's outputs (a chain), so an early read or a late write would change the bytes."""
    import torch
    option("gemv_pdl", pdl)
    k = n = 2560
    wps = [tb.synth_packed_weights(k, n, 40 + i) for i in range(3)]
    dws = [torch.from_numpy(w).cuda() for w in wps]
    a0 = tb.synth_activations((1, k), 9)
    acts = [torch.from_numpy(a0).cuda()] + [torch.zeros((1, k), dtype=torch.int8, device="cuda") for _ in range(3)]
    outs = [torch.zeros((1, n), dtype=torch.int32, device="cuda") for _ in range(3)]
    groups = [tb.ProjectionGroup([(acts[i], dws[i], outs[i])]) for i in range(3)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # layer i: out_i = act_i x W_i; act_{i+1} = low byte of out_i (a tiny torch kernel between the batches keeps the
    # chain honest for the first pass; the second pass runs the three batches with nothing in between on fixed inputs)
    expect, a = [], a0
    for i in range(3):
        c = oracle_lib.matmul(a, wps[i], "scalar")
        expect.append(c)
        a = c.astype(np.int8)
    for i in range(3):
        groups[i].run(status=status)
        if i < 2:
            acts[i + 1].copy_(outs[i].to(torch.int8))
    torch.cuda.synchronize()
    for i in range(3):
        assert_same(outs[i].cpu().numpy(), expect[i], f"chained batch {i} (pdl={pdl})")
    for rep in range(20):                      # back to back, same inputs: every run must reproduce the same bytes
        for i in range(3):
            groups[i].run(status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i in range(3):
        assert_same(outs[i].cpu().numpy(), expect[i], f"back-to-back batch {i} (pdl={pdl})")


def test_weight_handle_matches_and_caches():
    """ternix_b200_weights_*: same results as the plain entry point in every regime, across changing activations,
    outputs and row counts (the handle's one-entry descriptor caches must notice each change)."""
    import torch
    for (k, n) in [(4096, 11008), (2560, 640), (129, 4)]:
        wp = tb.synth_packed_weights(k, n, 5 + k)
        dw = torch.from_numpy(wp).cuda()
        handle = tb.TernaryWeights(dw)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        for rep, m in enumerate([32, 32, 1, 300, 300, 7, 64, 64, 48, 65]):
            a = tb.synth_activations((m, k), 1000 + rep)
            da = torch.from_numpy(a).cuda()
            out = torch.full((m, n + 4), -5, dtype=torch.int32, device="cuda")
            for _ in range(2):                               # the second call reuses every cached descriptor
                handle.matmul(da, out=out[:, :n], status=status)
            torch.cuda.synchronize()
            assert_same(out[:, :n].cpu().numpy(), oracle_lib.matmul(a, wp), f"weight handle {m}x{k}x{n}")
            assert bool((out[:, n:] == -5).all())
        assert int(status.item()) == 0
        handle.close()


def test_weight_handle_notices_a_change_of_tile_form(option):
    """The handle's cached activation descriptor is made for one tile form of the prefill kernel; an option that
    changes the form between two calls with the same activations must not be served the old descriptor."""
    import torch
    m, k, n = 300, 1040, 832
    wp = tb.synth_packed_weights(k, n, 9)
    a = tb.synth_activations((m, k), 10)
    expect = oracle_lib.matmul(a, wp)
    dw, da = torch.from_numpy(wp).cuda(), torch.from_numpy(a).cuda()
    handle = tb.TernaryWeights(dw)
    out = torch.empty((m, n), dtype=torch.int32, device="cuda")
    for rows in ("256", "128", "256", ""):
        option("tc_tile_rows", rows)
        out.fill_(-7)
        handle.matmul(da, out=out)
        torch.cuda.synchronize()
        assert_same(out.cpu().numpy(), expect, f"weight handle, tile form {rows!r}")
    handle.close()


def test_weight_handle_host_call():
    """ternix_b200_weights_matmul_host: activations and C in host memory (pinned torch tensors and plain numpy arrays),
    weights resident; one slab, several slabs with a ragged last one, every regime's row counts."""
    import torch
    for (m, k, n) in [(300, 1040, 832), (1, 2560, 6912), (32, 4096, 1024), (2304, 528, 16384)]:
        wp = tb.synth_packed_weights(k, n, 21 + k)
        handle = tb.TernaryWeights(torch.from_numpy(wp).cuda())
        for rep in range(2):
            a = tb.synth_activations((m, k), 40 + rep)
            expect = oracle_lib.matmul(a, wp)
            if rep == 0:
                out = handle.matmul_host(torch.from_numpy(a).pin_memory())
                assert_same(out.numpy(), expect, f"matmul_host pinned {m}x{k}x{n}")
            else:
                out = np.full((m, n), -9, dtype=np.int32)
                handle.matmul_host(a, out)
                assert_same(out, expect, f"matmul_host numpy {m}x{k}x{n}")
        handle.close()


def test_pack_ternary_on_the_device():
    """ternix_b200_pack_ternary_device writes the bytes of the host packer (and of the oracle's), for aligned and
    unaligned buffers and for sizes that are not multiples of 16."""
    import torch
    for (k, n) in [(2560, 6912), (33, 24), (1, 4), (129, 4), (7, 52)]:
        w = tb.synth_weights(k, n, 77 + k)
        expect = tb.pack_ternary(w)
        assert np.array_equal(expect, oracle_lib.pack(w))
        dw = torch.from_numpy(w).cuda()
        assert np.array_equal(tb.pack_ternary_device(dw).cpu().numpy(), expect), (k, n)
    # unaligned source and destination: the byte path
    w = tb.synth_weights(64, 64, 3)
    flat = torch.zeros(w.size + 1, dtype=torch.int8, device="cuda")
    flat[1:] = torch.from_numpy(w.reshape(-1)).cuda()
    out = torch.full((w.size // 4 + 3,), 0xEE, dtype=torch.uint8, device="cuda")
    rc = tb.lib.ternix_b200_pack_ternary_device(out.data_ptr() + 1, flat.data_ptr() + 1, w.size,
                                                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    got = out.cpu().numpy()
    assert np.array_equal(got[1:1 + w.size // 4], tb.pack_ternary(w).reshape(-1))
    assert got[0] == 0xEE and (got[1 + w.size // 4:] == 0xEE).all()


def test_bounded_wait_runs_out_and_the_context_survives():
    """A wait that nobody answers ends after its limit: the CTA takes the abort and drain path of the product kernels,
    reports TERNIX_B200_ERR_TIMEOUT in the status word and returns; the next launches work as usual."""
    import torch
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    limit_ns = 1_000_000
    rc = tb.lib.ternix_b200_selftest_wait_timeout(limit_ns, status.data_ptr(), waited.data_ptr(),
                                                  torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert int(status.item()) == tb.ERR_TIMEOUT
    ns = int(waited.item())
    assert limit_ns <= ns < 100 * limit_ns, f"waited {ns} ns for a {limit_ns} ns limit"
    assert tb.lib.ternix_b200_selftest_wait_timeout(0, None, None, None) == tb.ERR_INVALID_ARG
    assert tb.lib.ternix_b200_selftest_wait_timeout(10**9, None, None, None) == tb.ERR_INVALID_ARG
    # the context is intact: a product right after it is exact and reports no timeout
    a, wp = synth(32, 1024, 512, 4)
    assert_same(device_matmul(a, wp, "auto"), oracle_lib.matmul(a, wp), "product after the timeout self-test")


def test_peer_barrier_signals_waits_and_gives_up():
    """ternix_b200_peer_barrier on one GPU with both ranks' flag arrays local: the signal lands in the peer's array;
    a peer whose epoch is already there lets the barrier pass; a peer that never arrives ends the wait after its
    limit with TERNIX_B200_ERR_TIMEOUT in the status word, and the context stays usable."""
    import ctypes
    import torch
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    arrays = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    flags[0][1] = 1                                       # "rank 1 has arrived at barrier 1"
    assert tb.lib.ternix_b200_peer_barrier(arrays, 2, 0, 1, 0, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(flags[1][0].item()) == 1                   # rank 0's signal, in rank 1's array
    flags[0][1] = 5                                       # a peer that is several barriers ahead does not block either
    assert tb.lib.ternix_b200_peer_barrier(arrays, 2, 0, 2, 0, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(flags[1][0].item()) == 2
    # nobody answers barrier 6: 20 ms, then the status word
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert tb.lib.ternix_b200_peer_barrier(arrays, 2, 0, 6, 20_000_000, status.data_ptr(), stream) == 0
    e1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == tb.ERR_TIMEOUT
    assert 15.0 < e0.elapsed_time(e1) < 500.0
    assert tb.lib.ternix_b200_peer_barrier(arrays, 0, 0, 1, 0, None, None) == tb.ERR_INVALID_ARG
    assert tb.lib.ternix_b200_peer_barrier(arrays, 2, 2, 1, 0, None, None) == tb.ERR_INVALID_ARG
    assert tb.lib.ternix_b200_peer_barrier(arrays, 1, 0, 1, 0, None, None) == 0      # one rank: nothing to wait for
    a, wp = synth(32, 1024, 512, 4)
    assert_same(device_matmul(a, wp, "auto"), oracle_lib.matmul(a, wp), "product after the barrier timeout")


def test_second_gpu_in_the_same_process():
    """Per-device state (shared-memory opt-ins, SM counts, flag and scratch addresses): every kernel family on
    device 1 after device 0 in one process."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    shapes = [(1, 2560, 6912), (32, 4096, 1024), (300, 1040, 832), (7, 129, 4), (100, 1024, 128)]
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            for (m, k, n) in shapes:
                a, wp = synth(m, k, n, 11 * m + n)
                expect = oracle_lib.matmul(a, wp)
                da, dw = torch.from_numpy(a).cuda(dev), torch.from_numpy(wp).cuda(dev)
                for kern in ("auto", "gemv", "decode_mma", "skinny_tc", "gemm_tc"):
                    if kern != "auto" and tb.lib.ternix_b200_select_kernel(da.data_ptr(), dw.data_ptr(), 0, m, k, n, n) < 0:
                        continue
                    try:
                        c = tb.matmul(da, dw, kernel=kern)
                    except ValueError:
                        continue                               # that kernel does not take this shape
                    torch.cuda.synchronize(dev)
                    assert_same(c.cpu().numpy(), expect, f"device {dev} [{kern}] {m}x{k}x{n}")
            # the allocation-free batch on this device
            a, wp = synth(1, 2560, 640, 5)
            da, dw = torch.from_numpy(a).cuda(dev), torch.from_numpy(wp).cuda(dev)
            out = torch.full((1, 640), -1, dtype=torch.int32, device=f"cuda:{dev}")
            prob = (tb._Problem * 1)(tb._Problem(da.data_ptr(), dw.data_ptr(), out.data_ptr(), 1, 2560, 640, 640))
            rc = tb.lib.ternix_b200_gemv_batch_noalloc(prob, 1, None, torch.cuda.current_stream(dev).cuda_stream)
            torch.cuda.synchronize(dev)
            assert rc == 0
            assert_same(out.cpu().numpy(), oracle_lib.matmul(a, wp), f"noalloc batch on device {dev}")


def test_cpp_boundary_harness():
    """tests/cpp/boundary_check.cpp: the ternix:: C++ functions with the reference tests' inputs (built by the csrc
    Makefile, links libternix_b200.so)."""
    exe = os.path.join(ROOT, "tests", "cpp", "_build", "boundary_check")
    if not os.path.exists(exe):
        subprocess.run(["make", "-C", os.path.join(ROOT, "ternixengine_b200", "csrc")], check=True, capture_output=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "boundary_check: PASS" in r.stdout
