#!/usr/bin/env python
"""Benchmark of the ternary matrix product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--sustain SECONDS]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input: the prefill GEMM  C[4096,28672] = A[4096,8192] x W[8192,28672]  (the Llama-3-70B-shaped
FFN up projection of the baseline's config list), W ternary and packed.  At N > 1 the packed weights are
N-column-sharded over the ranks, every rank computes its columns and C is gathered into every rank's memory
over NVLink, so total work is fixed ("strong" scaling).  `value` = dense int8 TOPS = 2*M*K*N*steps / time,
zeros not skipped (the reference's own "effective TOPS" convention, benchmarks/bench_cuda.cu:73).

No number is printed unless EVERY entry of the GPU's C equals the reference's AVX2 kernel on the same bytes
(the reference's benchmark applies the same gate, benchmarks/bench_cuda.cu:69-81).

The same line carries: the roofline of the dominant kernel (burst and sustained), the decode-regime figures
(config 1 GEMV and config 5 at M=1, HBM GB/s), config 2 (M=32) and config 4 (ragged shapes), config 5 at
M=256, the CPU baseline (the reference's AVX2 kernel on the host cores: all cores and one pinned core) and an
end-to-end figure with host buffers.

`--impl reference` times the reference's own CPU kernel (oracle/_ref, or the oracle port when that build is
absent) on a bounded row sample of the same workload; it loads nothing of this package.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, N = 4096, 8192, 28672                 # prefill GEMM (Llama-3-70B-shaped FFN up projection)
GEMV_K, GEMV_N = 2560, 6912                 # decode GEMV (BitNet-b1.58-2B FFN up shape)
CFG2 = (32, 4096, 11008)                    # batched decode (Llama-7B-shaped gate/up projection)
CFG4 = [(1, 3001, 1028), (7, 129, 4), (37, 4099, 2052), (255, 2561, 6916)]
SEED = 20240531
# one BitNet-b1.58-2B-shaped layer: (K, N) of Q, K, V, O, gate, up, down
BITNET_LAYER = [(2560, 2560), (2560, 640), (2560, 640), (2560, 2560), (2560, 6912), (2560, 6912), (6912, 2560)]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------- seeded inputs, numpy only
# The same counter-based generator as ternix_b200_synth_* (splitmix64 of key + index), restated in numpy so that the
# reference arm needs nothing of this package; tests/test_host_api.py checks the two against each other byte for byte.
_U64 = np.uint64


def _mix64(z):
    with np.errstate(over="ignore"):
        z = z + _U64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> _U64(30))) * _U64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> _U64(27))) * _U64(0x94D049BB133111EB)
        return z ^ (z >> _U64(31))


def _stream_key(seed):
    return _mix64(np.array([seed ^ 0xA5A5A5A55A5A5A5A], dtype=np.uint64))[0]


def np_synth_activations(shape, seed):
    """int8 uniform on [-128, 127]: the low byte of the hash."""
    count = int(np.prod(shape))
    out = np.empty(count, dtype=np.int8)
    key = _stream_key(seed)
    step = 1 << 22
    for b in range(0, count, step):
        idx = np.arange(b, min(count, b + step), dtype=np.uint64)
        with np.errstate(over="ignore"):
            h = _mix64(key + idx)
        out[b:b + len(idx)] = (h & _U64(0xFF)).astype(np.uint8).view(np.int8)
    return out.reshape(shape)


def np_synth_packed_weights(k, n, seed):
    """iid ternary, P(-1) = P(+1) = 0.3 by the top 32 bits of the hash, packed four per byte (00 zero, 01 +1, 11 -1)."""
    count = k * n
    out = np.empty(count // 4, dtype=np.uint8)
    key = _stream_key(seed ^ 0x57454947)
    step = 1 << 22
    for b in range(0, count, step):
        idx = np.arange(b, min(count, b + step), dtype=np.uint64)
        with np.errstate(over="ignore"):
            u = _mix64(key + idx) >> _U64(32)
        code = np.where(u < 1288490189, 3, np.where(u < 2576980378, 1, 0)).astype(np.uint8).reshape(-1, 4)
        out[b // 4:b // 4 + len(code)] = code[:, 0] | (code[:, 1] << 2) | (code[:, 2] << 4) | (code[:, 3] << 6)
    return out.reshape(k, n // 4)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.idx)], stdout=f, stderr=subprocess.DEVNULL)
            t_wait = time.time()
            while time.time() - t_wait < 3.0 and os.path.getsize(self.path) == 0:
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the samples taken while the GPU drew the most power are the ones "under load"
        order = np.argsort(power)
        loaded = [sm[i] for i in order[len(order) // 2:]] if len(sm) > 3 else sm
        return {"sm_mhz": float(np.median(loaded)), "sm_mhz_min": float(min(sm)), "sm_max_mhz": float(max(smax)),
                "power_w_max": float(max(power)), "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------- CPU side (the reference's kernel)
def _oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    return oracle_lib


def cpu_product(a, wp, threads):
    """The reference's avx2_blocked over row bands on `threads` host threads (the plain-C port when the compiled
    reference is absent).  Returns (C, seconds, kind)."""
    oracle_lib = _oracle()
    t0 = time.perf_counter()
    if oracle_lib.have_ref():
        c = oracle_lib.ref_matmul(a, wp, "avx2_blocked", threads=threads)
        kind = "reference"
    else:
        c = oracle_lib.matmul(a, wp, "fast", threads=threads)
        kind = "port"
    return c, time.perf_counter() - t0, kind


def cpu_one_core(a, wp, target_s=10.0):
    """avx2_blocked on ONE pinned core, the way the reference benchmarks itself (benchmarks/bench_simd_math.cpp:65-78),
    on as many leading rows as take about target_s."""
    oracle_lib = _oracle()
    old = os.sched_getaffinity(0)
    try:
        os.sched_setaffinity(0, {sorted(old)[0]})
        rows = 4
        _, t, kind = cpu_product(a[:rows], wp, 1)
        rows = int(max(4, min(a.shape[0], (rows * target_s / max(t, 1e-3)) // 4 * 4)))
        _, t, kind = cpu_product(a[:rows], wp, 1)
    finally:
        os.sched_setaffinity(0, old)
    k, n = a.shape[1], wp.shape[1] * 4
    return {"value": 2.0 * rows * k * n / t / 1e12, "unit": "TOPS", "cores": 1, "kind": kind,
            "sample": f"first {rows} of {a.shape[0]} rows, full K and N, {t:.1f} s, one pinned core"}


# ------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    a = np_synth_activations((M, K), SEED)
    wp = np_synth_packed_weights(K, N, SEED + 1)
    threads = os.cpu_count() or 1
    # size one step so that warm-up + steps end within about two minutes, then time exactly `steps` of them
    per_step = min(4.0, max(0.25, 120.0 / (args.steps + args.warmup)))
    rows = min(M, 4 * threads)
    _, t, kind = cpu_product(a[:rows], wp, threads)
    rows = int(min(M, max(rows, (int(rows * per_step / max(t, 1e-3)) // (4 * threads)) * 4 * threads)))
    for _ in range(args.warmup):
        cpu_product(a[:rows], wp, threads)
    t_start = time.perf_counter()
    for _ in range(args.steps):
        cpu_product(a[:rows], wp, threads)
    dt = time.perf_counter() - t_start
    tops = 2.0 * rows * K * N * args.steps / dt / 1e12
    sample = f"first {rows} of {M} rows of A, full K and N, per step"
    line = {
        "impl": "reference", "metric": "prefill_gemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic",
        "config": {"workload": f"config3 prefill GEMM M={M} K={K} N={N} (row sample on CPU)", "sample_rows": rows},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- B200 arm
def timed(fn, steps, warmup, barrier):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1)           # ms on this rank


def run_b200(args):
    import torch
    import torch.distributed as dist
    import ternixengine_b200 as tb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL announces its version on stdout when the first communicator is created; stdout carries the JSON line only
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    oracle_lib = _oracle()
    peaks = load_peaks()
    a_host = tb.synth_activations((M, K), SEED)
    wp_host = tb.synth_packed_weights(K, N, SEED + 1)
    a_pin = torch.from_numpy(a_host).pin_memory()
    da = a_pin.to(dev)
    layer = tb.ShardedTernaryLinear(wp_host, device=dev)          # world > 1: fused peer-store gather
    shard = layer.shard
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- exactness gate: EVERY entry of the (gathered) C on EVERY rank against the reference's AVX2 kernel.
    #      Rank 0 computes the expected C once, on all host cores (that run is also the all-cores CPU baseline), and
    #      hands it to the other ranks through a file in shared memory.
    threads = os.cpu_count() or 1
    shm = os.path.join("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir(),
                       f"ternix_bench_expect_{os.environ.get('MASTER_PORT', '0')}.npy")
    cpu_all = None
    if rank == 0:
        expect, cpu_s, cpu_kind = cpu_product(a_host, wp_host, threads)
        cpu_all = {"value": 2.0 * M * K * N / cpu_s / 1e12, "unit": "TOPS", "cores": threads, "kind": cpu_kind,
                   "sample": f"all {M} rows, full K and N, {cpu_s:.1f} s, avx2_blocked over row bands on {threads} threads"}
        if world > 1:
            np.save(shm, expect)
    barrier()
    if rank != 0:
        expect = np.load(shm, mmap_mode="r")
    c = layer.forward(da, status=status)
    torch.cuda.synchronize()
    if int(status.item()) != 0:
        raise SystemExit(f"rank {rank}: a bounded device-side wait ran out")
    got = c.cpu().numpy()
    if not np.array_equal(got, expect):
        bad = np.argwhere(got != expect)
        raise SystemExit(f"rank {rank}: {len(bad)} entries of C differ from the reference's AVX2 kernel (first at "
                         f"{tuple(bad[0])}); refusing to report a number")
    headline_kernel = tb.last_launched_kernel()
    sample_rows = np.r_[0:4, 2046:2050, 4092:4096]
    expect_rows = np.ascontiguousarray(expect[sample_rows])
    del got
    barrier()
    if rank == 0 and world > 1:
        os.unlink(shm)
    if rank != 0:
        del expect

    # ---- device-resident throughput (the headline)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = max_over_ranks(timed(lambda: layer.forward(da), args.steps, args.warmup, barrier))
    clocks = sampler.stop() if rank == 0 else None
    ops = 2.0 * M * K * N
    tops = ops * args.steps / (ms * 1e-3) / 1e12

    # shard compute alone (no gather): explains the scaling curve
    local_out = torch.empty((M, max(shard.n_cols, 4)), dtype=torch.int32, device=dev)
    ms_local = max_over_ranks(timed(lambda: layer.local(da, out=local_out[:, :shard.n_cols]), args.steps, args.warmup,
                                    barrier))

    # the pieces of a sharded step, each timed alone
    gather_parts = None
    if world > 1:
        ms_store = max_over_ranks(timed(lambda: layer.forward(da, barrier=False), args.steps, args.warmup, barrier))
        ms_bar = max_over_ranks(timed(layer.stream_barrier, args.steps, args.warmup, barrier))
        # what the store path alone sustains: the same output (same M, same shard, same destinations) from a product
        # with K = 256, whose arithmetic is 1/32 of config 3's, so that the launch is all stores
        k_probe = 256
        probe = tb.ShardedTernaryLinear(tb.synth_packed_weights(k_probe, N, SEED + 77), device=dev)
        da_probe = torch.from_numpy(tb.synth_activations((M, k_probe), SEED + 78)).to(dev)
        ms_probe = max_over_ranks(timed(lambda: probe.forward(da_probe, barrier=False), args.steps, args.warmup, barrier))
        ms_probe_local = max_over_ranks(timed(lambda: probe.local(da_probe, out=local_out[:, :shard.n_cols]), args.steps,
                                              args.warmup, barrier))
        out_bytes = 4 * M * shard.n_cols * (world - 1)
        gather_parts = {"gemm_with_peer_stores_ms": ms_store / args.steps, "stream_barrier_ms": ms_bar / args.steps,
                        "shard_gemm_alone_ms": ms_local / args.steps, "nvlink_bytes_out_per_rank": out_bytes,
                        "nvlink_gbs_out_per_rank": out_bytes / (ms_store / args.steps * 1e-3) / 1e9,
                        "store_only_probe": {"what": f"same output from a K={k_probe} product: the launch is all stores",
                                             "ms_with_peer_stores": ms_probe / args.steps,
                                             "ms_local_stores_only": ms_probe_local / args.steps,
                                             "nvlink_gbs_out_per_rank": out_bytes / (ms_probe / args.steps * 1e-3) / 1e9}}
        del probe, da_probe

    # ---- sustained figure: the same launch back to back for seconds, clocks sampled throughout
    sustained = None
    if rank == 0 and world == 1 and args.sustain > 0:
        n_sus = max(50, int(args.sustain / (ms / args.steps * 1e-3)))
        s2 = ClockSampler(local)
        s2.start()
        ms_sus = timed(lambda: layer.forward(da), n_sus, 3, lambda: None)
        clk = s2.stop()
        t_sus = ops * n_sus / (ms_sus * 1e-3) / 1e12
        peak_sus = 2.0 * peaks["bf16_tflops_sustained"]
        sustained = {"launches": n_sus, "seconds": ms_sus * 1e-3, "ms_per_step": ms_sus / n_sus, "achieved": t_sus,
                     "peak": peak_sus, "unit": "TOPS", "frac": t_sus / peak_sus,
                     "peak_source": f"2 x sustained bf16 of {peaks['source']} peaks (dense int8 proxy)",
                     "frac_of_nominal_4500": t_sus / 4500.0, "clocks": clk,
                     "ms_times_median_mhz": (ms_sus / n_sus) * clk["sm_mhz"] if clk.get("sm_mhz") else None}

    # ---- end to end, the same definition at every N: activations from pinned host memory to every rank, the step,
    #      and the WHOLE gathered C back to pinned host memory on rank 0; packed weights resident on the devices
    #      The call a user makes: ShardedTernaryLinear.forward_host (one GPU: ternix_b200_weights_matmul_host), which
    #      cuts the rows into slabs and runs upload, product (+ gather) and download on three streams.
    c_pin = torch.empty((M, N), dtype=torch.int32).pin_memory() if rank == 0 else None
    layer_host = tb.ShardedTernaryLinear(wp_host, device=dev)

    def e2e_step():
        layer_host.forward_host(a_pin, c_pin)

    if rank == 0:
        c_pin.fill_(-1)
    e2e_steps = max(3, min(20, args.steps))
    ms_e2e = max_over_ranks(timed(e2e_step, e2e_steps, 3, barrier))
    if rank == 0 and not np.array_equal(c_pin.numpy(), expect):
        raise SystemExit("end-to-end result differs from the reference")
    e2e = {"value": ops * e2e_steps / (ms_e2e * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms_e2e / e2e_steps,
           "h2d_bytes_per_step": M * K * world, "d2h_bytes_per_step": 4 * M * N,
           "note": "forward_host: pinned host A copied to every rank, the step, the whole C copied back to pinned host memory "
                   "on rank 0, in row slabs on three streams; packed weights resident (the same definition at every N); "
                   "every entry of the returned C checked"}
    del layer_host

    # ---- the reference-facing host-pointer call (what mul_mat_ternary_cuda_host binds): A, packed W and C in host
    #      memory; pool allocation, H2D of A and W, kernel, D2H of C, free and sync inside every call
    host_call = None
    if world == 1:
        w_pin = torch.from_numpy(wp_host).pin_memory()

        def host_step():
            rc = tb.lib.ternix_b200_matmul_host(a_pin.data_ptr(), w_pin.data_ptr(), c_pin.data_ptr(), M, K, N, 0)
            if rc:
                raise SystemExit(f"ternix_b200_matmul_host failed: {tb.status_string(rc)}")

        c_pin.fill_(-1)
        host_step()
        if not np.array_equal(c_pin.numpy(), expect):
            raise SystemExit("host-pointer entry point differs from the reference")
        n_host = max(3, min(10, args.steps))
        t0 = time.perf_counter()
        for _ in range(n_host):
            host_step()
        host_ms = (time.perf_counter() - t0) * 1e3 / n_host        # the call synchronises: wall clock covers copies + kernel
        host_call = {"value": ops / (host_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": host_ms,
                     "h2d_bytes_per_step": M * K + K * N // 4, "d2h_bytes_per_step": 4 * M * N,
                     "note": "ternix_b200_matmul_host: the weights go up with every call, as in the reference's wrapper"}
        del w_pin
    if rank == 0:
        del expect

    # ---- the same job with the dequantising epilogue: bfloat16 C = C_int * row_scale * w_scale on every GPU
    row_scale = torch.full((M,), 0.01, dtype=torch.float32, device=dev)
    y = layer.forward_dequant(da, row_scale, 0.05, status=status)
    torch.cuda.synchronize()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import bitnet_scaling_oracle as scaling
    y_bits = y[torch.from_numpy(sample_rows).to(dev)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    if not np.array_equal(y_bits, scaling.dequant_bf16_bits(expect_rows, np.full(len(sample_rows), 0.01, np.float32), 0.05)):
        raise SystemExit(f"rank {rank}: dequantised output differs from its CPU restatement")
    ms_deq = max_over_ranks(timed(lambda: layer.forward_dequant(da, row_scale, 0.05), args.steps, args.warmup, barrier))
    dequant = {"what": "same product, GEMM epilogue emits bfloat16 = C * row_scale * w_scale (and ships it to the peers)",
               "ms_per_step": ms_deq / args.steps, "tops": ops * args.steps / (ms_deq * 1e-3) / 1e12}

    # ---- config 5 at M=256: the 210 projections of a 30-layer BitNet-2B-shaped model
    cfg5 = bench_config5_m256(tb, dev, world, rank, barrier, max_over_ranks)

    # ---- the NCCL all-gather + unpack baseline for the same job (what the fused epilogue replaces)
    nccl_ms = None
    if world > 1:
        base = tb.ShardedTernaryLinear(wp_host, device=dev, mode="nccl")
        c2 = torch.empty((M, N), dtype=torch.int32, device=dev)
        base.forward(da, out=c2)
        torch.cuda.synchronize()
        if not bool((c2 == layer.forward(da)).all()):
            raise SystemExit(f"rank {rank}: NCCL-gathered C differs from the peer-store C")
        n_base = max(5, args.steps // 4)
        nccl_ms = max_over_ranks(timed(lambda: base.forward(da, out=c2), n_base, 3, barrier)) / n_base
        del base, c2

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- rank 0, one GPU: the decode regime, config 2, config 4
    gemv = bench_gemv(tb, dev, peaks)
    cfg2 = bench_config2(tb, dev, peaks)
    cfg4 = bench_config4(tb, dev)
    cpu_one = cpu_one_core(a_host, wp_host)

    int8_peak = 2.0 * peaks["bf16_tflops"]
    traffic, traffic_src = None, None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath) and world == 1 and headline_kernel == "ternary_gemm_tc3_kernel":
        traffic = json.load(open(tpath)).get("gemm_tc3_config3_dram_bytes_per_launch")
        traffic_src = "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, from profiles/traffic.json (not this run)"
    kernel_ms = ms_local / args.steps
    local_ops = 2.0 * M * K * shard.n_cols
    achieved = local_ops / (kernel_ms * 1e-3) / 1e12
    line = {
        "metric": "prefill_gemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic",
        "config": {"workload": f"config3 prefill GEMM M={M} K={K} N={N}, W ternary packed 2-bit",
                   "parallelism": (f"N-column shards x{world}; every rank's GEMM epilogue stores its columns into all "
                                   f"ranks' C over NVLink (fused gather) + stream barrier") if world > 1 else "single GPU",
                   "l2": "A+W+C = 562 MB per step exceeds the 126 MB L2; C (470 MB) is rewritten every step",
                   "exactness": "every entry of C on every rank equals the reference's avx2_blocked", "seed": SEED},
        "shard_compute": {"ms": kernel_ms, "tops_per_gpu": achieved, "columns_rank0": shard.n_cols},
        "gather_parts": gather_parts,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOPS",
                     "frac": achieved / int8_peak, "traffic": traffic, "traffic_source": traffic_src,
                     "kernel": headline_kernel, "kernel_source": "ternix_b200_last_launched_kernel() after the gated launch",
                     "peak_source": f"2 x bf16 burst of {peaks['source']} peaks (dense int8 proxy)",
                     "frac_of_nominal_4500": achieved / 4500.0},
        "roofline_sustained": sustained,
        "nccl_gather_baseline": None if nccl_ms is None else {
            "ms_per_step": nccl_ms, "tops": ops / (nccl_ms * 1e-3) / 1e12,
            "what": "same shards, local GEMM then ncclAllGather of C blocks then unpack to row-major"},
        "dequant_bf16_output": dequant,
        "config5_m256": cfg5,
        "config2": cfg2,
        "config4": cfg4,
        "gemv": gemv,
        "cpu_baseline": cpu_all,
        "cpu_baseline_one_core": cpu_one,
        "e2e": e2e,
        "e2e_host_call": host_call,
        "gpu_launches": args.steps * (2 if world > 1 else 1),
        "gpu_launches_note": "per timed step and rank: one launch of this library's GEMM and, at N > 1, one of its peer-barrier kernel",
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_config5_m256(tb, dev, world, rank, barrier, max_over_ranks):
    """210 projections (7 per layer x 30 layers) at M=256 in one launch per rank.  A projection is N-column-sharded
    over the ranks only where the model in should_shard() says the gather costs less than the compute it saves; with
    int32 outputs and K = 2560 / 6912 that is nowhere, so every rank computes the whole set (replicas)."""
    import torch
    oracle_lib = _oracle()
    Mb = 256
    weights, acts, ops, byts = [], [], 0.0, 0
    for layer in range(30):
        for i, (k, n) in enumerate(BITNET_LAYER):
            weights.append(tb.synth_packed_weights(k, n, SEED + 9000 + 10 * layer + i))
            acts.append(torch.from_numpy(tb.synth_activations((Mb, k), SEED + 7000 + 10 * layer + i)).to(dev))
            ops += 2.0 * Mb * k * n
            byts += k * n // 4 + Mb * k + 4 * Mb * n
    pset = tb.ShardedProjectionSet(weights, acts, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = pset.run(status=status)
    torch.cuda.synchronize()
    barrier()
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out in the grouped GEMM")
    for idx in range(len(weights)):                  # every entry of all 210 outputs
        expect = oracle_lib.matmul(acts[idx].cpu().numpy(), weights[idx])
        if not np.array_equal(outs[idx].cpu().numpy(), expect):
            raise SystemExit(f"rank {rank}: config 5 projection {idx} differs from the CPU oracle")
    reps = 10
    ms = max_over_ranks(timed(pset.run, reps, 3, barrier)) / reps
    return {"workload": "config5: 30 layers x {Q,K,V,O,gate,up,down} of a BitNet-b1.58-2B-shaped model, M=256",
            "projections": 210, "checked": "all 210 outputs, every entry", "launches_per_rank": pset.launches, "ms": ms,
            "projections_per_s": 210 / (ms * 1e-3), "tops": ops / (ms * 1e-3) / 1e12,
            "gbs_algorithmic": byts / (ms * 1e-3) / 1e9,
            "sharded_projections": pset.sharded_count,
            "note": "per-replica figure; should_shard() keeps a projection whole where the gather would cost more than "
                    "the compute it saves" if world > 1 else "single GPU"}


def _graph_of(fn):
    import torch
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn(s)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            fn(s)
    return g


def bench_config2(tb, dev, peaks):
    """config 2: C[32,11008] = A[32,4096] x W[4096,11008], 12.8 MB per product, HBM-bound.  Timed two ways over 32
    distinct weight copies (361 MB > L2): one launch per product replayed as a CUDA graph (what a caller with one
    projection gets), and all 32 in one group launch."""
    import torch
    oracle_lib = _oracle()
    m, k, n = CFG2
    copies = 32
    a = tb.synth_activations((m, k), SEED + 21, lo=-127)
    ws = [tb.synth_packed_weights(k, n, SEED + 300 + i) for i in range(2)]
    expect = [oracle_lib.matmul(a, w) for w in ws]
    da = torch.from_numpy(a).to(dev)
    dws = [torch.from_numpy(ws[i % 2]).to(dev).clone() for i in range(copies)]
    outs = [torch.full((m, n), -1, dtype=torch.int32, device=dev) for _ in range(copies)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def check(tag):
        torch.cuda.synchronize()
        if int(status.item()) != 0:
            raise SystemExit(f"config 2 ({tag}): a bounded device-side wait ran out")
        for i in range(copies):
            if not np.array_equal(outs[i].cpu().numpy(), expect[i % 2]):
                raise SystemExit(f"config 2 ({tag}) differs from the CPU oracle; refusing to report a number")
            outs[i].fill_(-1)

    handles = [tb.TernaryWeights(w) for w in dws]

    def sweep(s):
        for i in range(copies):
            handles[i].matmul(da, out=outs[i], status=status, stream=s)

    g = _graph_of(sweep)
    g.replay()
    check("graph of single launches")
    kernel = tb.last_launched_kernel()
    us_single = timed(g.replay, 20, 3, lambda: None) * 1e3 / (20 * copies)
    us_stream = timed(lambda: sweep(torch.cuda.current_stream()), 5, 2, lambda: None) * 1e3 / (5 * copies)
    group = tb.ProjectionGroup([(da, dws[i], outs[i]) for i in range(copies)])
    group.run(status=status)
    check("one group launch")
    us_group = timed(group.run, 20, 3, lambda: None) * 1e3 / (20 * copies)
    byts = k * n // 4 + m * k + 4 * m * n
    gbs = lambda us: byts / (us * 1e-6) / 1e9
    return {"workload": f"config2 batched decode M={m} K={k} N={n}; {copies} distinct weight copies (361 MB > L2)",
            "algorithmic_bytes": byts, "kernel_single": kernel, "us_single_launch_in_graph": us_single,
            "gbs_single_launch_in_graph": gbs(us_single), "us_single_launch_from_host": us_stream,
            "us_per_product_grouped": us_group, "gbs_grouped": gbs(us_group), "group_launches": group.launches,
            "roofline": {"bound": "hbm", "achieved": gbs(us_group), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs(us_group) / peaks["hbm_gbs"], "frac_single_launch": gbs(us_single) / peaks["hbm_gbs"],
                         "peak_source": f"{peaks['source']} copy bandwidth"},
            "checked": "every entry of all 32 outputs, both ways"}


def bench_config4(tb, dev):
    """config 4: ragged shapes whose packed rows are not 16-byte multiples (no TMA view): exactness on seeded data
    and on the worst case (A = -128, W = -1, every entry 128 K), and the time of the generic kernel."""
    import torch
    oracle_lib = _oracle()
    out = []
    for (m, k, n) in CFG4:
        a = tb.synth_activations((m, k), SEED + m + k)
        wp = tb.synth_packed_weights(k, n, SEED + n)
        da, dw = torch.from_numpy(a).to(dev), torch.from_numpy(wp).to(dev)
        c = torch.full((m, n), -1, dtype=torch.int32, device=dev)
        tb.matmul(da, dw, out=c)
        kernel = tb.last_launched_kernel()
        torch.cuda.synchronize()
        if not np.array_equal(c.cpu().numpy(), oracle_lib.matmul(a, wp, "scalar")):
            raise SystemExit(f"config 4 {m}x{k}x{n} differs from the reference's scalar kernel")
        da2 = torch.full((m, k), -128, dtype=torch.int8, device=dev)
        dw2 = torch.full((k, n // 4), 0xFF, dtype=torch.uint8, device=dev)
        tb.matmul(da2, dw2, out=c)
        torch.cuda.synchronize()
        if not bool((c == 128 * k).all()):
            raise SystemExit(f"config 4 {m}x{k}x{n}: worst-case accumulation is not 128 K")
        g = _graph_of(lambda s: [tb.matmul(da, dw, out=c, stream=s) for _ in range(10)])
        us = timed(g.replay, 10, 2, lambda: None) * 1e3 / 100
        out.append({"shape": [m, k, n], "kernel": kernel, "us": us, "gmacs": m * k * n / (us * 1e-6) / 1e9})
    return {"workload": "config4 ragged + worst-case exactness sweep", "checked": "every entry, seeded and worst case",
            "shapes": out}


def bench_gemv(tb, dev, peaks):
    """Decode regime, rank 0, one GPU.

    config 1: C[1,6912] = A[1,2560] x W[2560,6912] over 64 distinct weight copies (283 MB > L2), three ways:
      grouped  - all 64 GEMVs in ONE launch of the persistent kernel (ternix_b200_group_run): the throughput figure
      graph    - 64 single-GEMV launches replayed as one CUDA graph
      stream   - 64 single-GEMV launches from Python
    config 5 (M=1): the 210 projections of a 30-layer BitNet-2B-shaped model (521 MB of packed weights) in one launch.
    """
    import torch
    oracle_lib = _oracle()
    copies = 64
    a = tb.synth_activations((1, GEMV_K), SEED + 7)
    ws = [tb.synth_packed_weights(GEMV_K, GEMV_N, SEED + 100 + i) for i in range(4)]
    da = torch.from_numpy(a).to(dev)
    dws = [torch.from_numpy(ws[i % 4]).to(dev).clone() for i in range(copies)]
    outs = [torch.empty((1, GEMV_N), dtype=torch.int32, device=dev) for _ in range(copies)]
    expect = [oracle_lib.matmul(a, ws[i], "scalar") for i in range(4)]
    if oracle_lib.have_ref():
        for i in range(4):
            if not np.array_equal(oracle_lib.ref_matmul(a, ws[i], "avx2_blocked"), expect[i]):
                raise SystemExit("the oracle port and the compiled reference disagree")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    group = tb.ProjectionGroup([(da, dws[i], outs[i]) for i in range(copies)])

    def check(tag):
        torch.cuda.synchronize()
        for i in range(copies):
            if not np.array_equal(outs[i].cpu().numpy(), expect[i % 4]):
                raise SystemExit(f"GEMV ({tag}) differs from the CPU oracle; refusing to report a number")
            outs[i].fill_(-1)

    def sweep(s=None):
        for i in range(copies):
            tb.matmul(da, dws[i], out=outs[i], stream=s)

    group.run(status=status)
    check("grouped")
    sweep()
    check("single launches")
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out in the grouped GEMV")
    bytes_per = GEMV_K * GEMV_N // 4 + GEMV_K + 4 * GEMV_N
    passes = 20
    us_group = timed(group.run, passes, 5, lambda: None) * 1e3 / (passes * copies)
    us_stream = timed(sweep, 5, 3, lambda: None) * 1e3 / (5 * copies)
    g = _graph_of(sweep)
    us_graph = timed(g.replay, passes, 3, lambda: None) * 1e3 / (passes * copies)
    gbs = lambda us: bytes_per / (us * 1e-6) / 1e9
    # the same kernel on four times as many copies (1.13 GB of weights): the ramps of a launch weigh a quarter as much
    many = 4 * copies
    dws_many = dws + [torch.from_numpy(ws[i % 4]).to(dev).clone() for i in range(many - copies)]
    outs_many = outs + [torch.empty((1, GEMV_N), dtype=torch.int32, device=dev) for _ in range(many - copies)]
    group_many = tb.ProjectionGroup([(da, dws_many[i], outs_many[i]) for i in range(many)])
    group_many.run(status=status)
    torch.cuda.synchronize()
    for i in range(many):
        if not np.array_equal(outs_many[i].cpu().numpy(), expect[i % 4]):
            raise SystemExit("GEMV (256 per launch) differs from the CPU oracle; refusing to report a number")
    us_group_many = timed(group_many.run, passes, 5, lambda: None) * 1e3 / (passes * many)
    del group_many, dws_many, outs_many

    # config 5, M = 1
    probs, total_bytes = [], 0
    for layer in range(30):
        for i, (k, n) in enumerate(BITNET_LAYER):
            A = torch.from_numpy(tb.synth_activations((1, k), SEED + 1000 + 10 * layer + i)).to(dev)
            W = torch.from_numpy(tb.synth_packed_weights(k, n, SEED + 5000 + 10 * layer + i)).to(dev)
            probs.append((A, W, torch.empty((1, n), dtype=torch.int32, device=dev)))
            total_bytes += k * n // 4 + k + 4 * n
    g5 = tb.ProjectionGroup(probs)
    g5.run(status=status)
    torch.cuda.synchronize()
    for (A, W, C) in probs:                       # every entry of all 210 outputs
        if not np.array_equal(C.cpu().numpy(), oracle_lib.matmul(A.cpu().numpy(), W.cpu().numpy(), "scalar")):
            raise SystemExit("config 5 projection differs from the CPU oracle; refusing to report a number")
    ms5 = timed(g5.run, passes, 5, lambda: None) / passes

    t_cpu0 = time.perf_counter()
    reps = 5
    for _ in range(reps):
        if oracle_lib.have_ref():
            oracle_lib.ref_matmul(a, ws[0], "avx2_blocked")
        else:
            oracle_lib.matmul(a, ws[0], "scalar")
    cpu_s = (time.perf_counter() - t_cpu0) / reps
    best = gbs(us_group)
    return {"workload": f"config1 GEMV M=1 K={GEMV_K} N={GEMV_N}; {copies} distinct weight copies (283 MB > L2), "
                        f"all {copies} in one launch of the persistent grouped kernel",
            "metric": "gemv_hbm_gbs", "unit": "GB/s", "value": best, "us_per_gemv_grouped": us_group,
            "us_per_gemv_grouped_256_per_launch": us_group_many, "gbs_256_per_launch": gbs(us_group_many),
            "frac_of_nominal_8000_256_per_launch": gbs(us_group_many) / 8000.0,
            "us_per_launch_graph": us_graph, "us_per_launch_stream": us_stream, "gbs_graph": gbs(us_graph),
            "gbs_stream": gbs(us_stream), "algorithmic_bytes_per_gemv": bytes_per,
            "checked": "every entry of all 64 outputs (grouped and single launches) and of all 210 config-5 outputs",
            "roofline": {"bound": "hbm", "achieved": best, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": best / peaks["hbm_gbs"], "traffic": None, "kernel": "ternary_gemv_group_kernel",
                         "peak_source": f"{peaks['source']} copy bandwidth", "frac_of_nominal_8000": best / 8000.0},
            "config5_m1": {"projections": 210, "launches": g5.launches, "ms": ms5, "projections_per_s": 210 / (ms5 * 1e-3),
                           "gbs": total_bytes / (ms5 * 1e-3) / 1e9,
                           "frac_of_measured_hbm": total_bytes / (ms5 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "frac_of_nominal_8000": total_bytes / (ms5 * 1e-3) / 1e9 / 8000.0,
                           "algorithmic_bytes": total_bytes},
            "cpu_baseline": {"value": bytes_per / cpu_s / 1e9, "unit": "GB/s", "cores": 1,
                             "kind": "reference" if oracle_lib.have_ref() else "port",
                             "sample": f"one whole GEMV, mean of {reps}, one thread (the kernel cannot slice M=1)"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sustain", type=float, default=2.0, help="seconds of back-to-back launches for the sustained figure")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
