#!/usr/bin/env python
"""Benchmark of the ternary matrix product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input: the prefill GEMM  C[4096,28672] = A[4096,8192] x W[8192,28672]  (the Llama-3-70B-shaped
FFN up projection of the baseline's config list), W ternary and packed.  At N > 1 the packed weights are
N-column-sharded over the ranks, every rank computes its columns and C is all-gathered over NCCL, so
total work is fixed ("strong" scaling).  `value` = dense int8 TOPS = 2*M*K*N*steps / time, zeros not
skipped (the reference's own "effective TOPS" convention, benchmarks/bench_cuda.cu:73).

The same line carries the decode-regime figure (M=1 BitNet-shaped GEMV, HBM GB/s), the roofline of the
dominant kernel, the CPU baseline (the reference's AVX2 kernel on the host cores) and an end-to-end
figure through the host-pointer entry point.

`--impl reference` times the reference's own CPU kernel (oracle/_ref, or the oracle port when that
build is absent) on a bounded row sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, N = 4096, 8192, 28672                 # prefill GEMM (Llama-3-70B-shaped FFN up projection)
GEMV_K, GEMV_N = 2560, 6912                 # decode GEMV (BitNet-b1.58-2B FFN up shape)
SEED = 20240531
L2_BYTES = 126 * 1024 * 1024
# one BitNet-b1.58-2B-shaped layer: (K, N) of Q, K, V, O, gate, up, down
BITNET_LAYER = [(2560, 2560), (2560, 640), (2560, 640), (2560, 2560), (2560, 6912), (2560, 6912), (6912, 2560)]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
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
        # the busiest half of the samples is "under load"
        load = sorted(sm)[len(sm) // 2:] if len(sm) > 3 else sm
        return {"sm_mhz": float(np.median(sm)), "sm_mhz_min": float(min(sm)), "sm_max_mhz": float(max(smax)),
                "power_w_max": float(max(power)), "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------- CPU baseline
def cpu_reference_sample(a, wp, target_s=12.0, rows0=None):
    """Times the reference's CPU kernel (all host threads, row bands) on the first `rows` rows of A.
    Returns (tops, seconds, rows, threads, kind)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    threads = os.cpu_count() or 1
    use_ref = oracle_lib.have_ref()

    def run(rows):
        t0 = time.perf_counter()
        if use_ref:
            oracle_lib.ref_matmul(a[:rows], wp, "avx2_blocked", threads=threads)
        else:
            oracle_lib.matmul(a[:rows], wp, "fast", threads=threads)
        return time.perf_counter() - t0

    k, n = a.shape[1], wp.shape[1] * 4
    rows = rows0 or min(a.shape[0], 4 * threads)
    t = run(rows)
    if rows0 is None and t < target_s / 4 and rows < a.shape[0]:
        scale = min(a.shape[0] / rows, target_s / max(t, 1e-3))
        rows = int(min(a.shape[0], max(rows, (int(rows * scale) // (4 * threads)) * 4 * threads)))
        t = run(rows)
    return 2.0 * rows * k * n / t / 1e12, t, rows, threads, ("reference" if use_ref else "port")


def make_inputs():
    import ternixengine_b200 as tb
    a = tb.synth_activations((M, K), SEED)
    wp = tb.synth_packed_weights(K, N, SEED + 1)
    return a, wp


# ------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    a, wp = make_inputs()
    # size one step so that warm-up + steps end within about two minutes, then time exactly `steps` of them
    per_step = min(4.0, max(0.25, 120.0 / (args.steps + args.warmup)))
    tops0, t0, rows, threads, kind = cpu_reference_sample(a, wp, target_s=per_step)
    for _ in range(args.warmup):
        cpu_reference_sample(a, wp, rows0=rows)
    t_start = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_sample(a, wp, rows0=rows)
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
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = load_peaks()
    a_host, wp_host = make_inputs()
    a_pin = torch.from_numpy(a_host).pin_memory()
    da = a_pin.to(dev)
    layer = tb.ShardedTernaryLinear(wp_host, device=dev)          # world > 1: fused peer-store gather
    shard = layer.shard
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- exactness gate (the reference's benchmark refuses to report an unverified number,
    #      benchmarks/bench_cuda.cu:69-81): sampled rows of the gathered C against the CPU oracle.
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    c = layer.forward(da, status=status)
    torch.cuda.synchronize()
    if int(status.item()) != 0:
        raise SystemExit(f"rank {rank}: a bounded device-side wait ran out")
    rows = np.r_[0:4, 2046:2050, 4092:4096]
    expect = oracle_lib.matmul(a_host[rows], wp_host)
    got = c[torch.from_numpy(rows).to(dev)].cpu().numpy()
    if not np.array_equal(got, expect):
        raise SystemExit(f"rank {rank}: GPU result differs from the CPU oracle; refusing to report a number")

    # ---- device-resident throughput
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        t_wait = time.time()
        while time.time() - t_wait < 3.0 and (not sampler.path or os.path.getsize(sampler.path) == 0):
            time.sleep(0.05)
    ms = max_over_ranks(timed(lambda: layer.forward(da), args.steps, args.warmup, barrier))
    clocks = sampler.stop() if rank == 0 else None
    ops = 2.0 * M * K * N
    tops = ops * args.steps / (ms * 1e-3) / 1e12

    # shard compute alone (no gather): explains the scaling curve
    local_out = torch.empty((M, max(shard.n_cols, 4)), dtype=torch.int32, device=dev)
    ms_local = max_over_ranks(timed(lambda: layer.local(da, out=local_out[:, :shard.n_cols]), args.steps, args.warmup,
                                    barrier))

    # ---- end to end through the host-pointer entry point: pinned host A in, result columns out, every step
    c_pin = torch.empty((M, max(shard.n_cols, 4)), dtype=torch.int32).pin_memory()

    def e2e_step():
        da.copy_(a_pin, non_blocking=True)
        cc = layer.forward(da)
        c_pin[:, :shard.n_cols].copy_(cc[:, shard.n0:shard.n0 + shard.n_cols], non_blocking=True)

    e2e_steps = max(3, min(20, args.steps))
    ms_e2e = max_over_ranks(timed(e2e_step, e2e_steps, 3, barrier))
    e2e_tops = ops * e2e_steps / (ms_e2e * 1e-3) / 1e12

    # ---- end to end through the reference-facing host-pointer call (what mul_mat_ternary_cuda_host binds):
    #      A, packed W and C all in (pinned) host memory, allocation + H2D + kernel + D2H + free inside the call
    host_call = None
    if world == 1:
        w_pin = torch.from_numpy(wp_host).pin_memory()
        c_host = torch.empty((M, N), dtype=torch.int32).pin_memory()

        def host_step():
            rc = tb.lib.ternix_b200_matmul_host(a_pin.data_ptr(), w_pin.data_ptr(), c_host.data_ptr(), M, K, N, 0)
            if rc:
                raise SystemExit(f"ternix_b200_matmul_host failed: {tb.status_string(rc)}")

        host_step()
        if not np.array_equal(c_host[torch.from_numpy(rows)].numpy(), expect):
            raise SystemExit("host-pointer entry point differs from the CPU oracle")
        n_host = max(3, min(10, args.steps))
        t0 = time.perf_counter()
        for _ in range(n_host):
            host_step()
        host_ms = (time.perf_counter() - t0) * 1e3 / n_host        # the call synchronises: wall clock is the device time + copies
        host_call = {"value": ops / (host_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": host_ms,
                     "h2d_bytes_per_step": M * K + K * N // 4, "d2h_bytes_per_step": 4 * M * N,
                     "note": "ternix_b200_matmul_host (what the reference's mul_mat_ternary_cuda_host binds): pinned host A, "
                             "packed W and C; pool allocation, H2D of A and W, kernel, D2H of C, free, sync inside every call"}

    # the same job with the dequantising epilogue: bfloat16 C = C_int * row_scale * w_scale on every GPU
    row_scale = torch.full((M,), 0.01, dtype=torch.float32, device=dev)
    y = layer.forward_dequant(da, row_scale, 0.05, status=status)
    torch.cuda.synchronize()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import bitnet_scaling_oracle as scaling
    y_bits = y[torch.from_numpy(rows).to(dev)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    if not np.array_equal(y_bits, scaling.dequant_bf16_bits(expect, np.full(len(rows), 0.01, np.float32), 0.05)):
        raise SystemExit(f"rank {rank}: dequantised output differs from its CPU restatement")
    ms_deq = max_over_ranks(timed(lambda: layer.forward_dequant(da, row_scale, 0.05), args.steps, args.warmup, barrier))
    dequant = {"what": "same product, GEMM epilogue emits bfloat16 = C * row_scale * w_scale (and ships it to the peers)",
               "ms_per_step": ms_deq / args.steps, "tops": ops * args.steps / (ms_deq * 1e-3) / 1e12}

    # config 5 at M=256: the 210 projections of a 30-layer BitNet-2B-shaped model, sharded where it pays off
    cfg5 = bench_config5_m256(tb, dev, world, rank, barrier, max_over_ranks)

    # the NCCL all-gather + unpack baseline for the same job (what the fused epilogue replaces)
    nccl_ms = None
    if world > 1:
        base = tb.ShardedTernaryLinear(wp_host, device=dev, mode="nccl")
        c2 = torch.empty((M, N), dtype=torch.int32, device=dev)
        base.forward(da, out=c2)
        torch.cuda.synchronize()
        if not bool((c2 == c).all()):
            bad = (c2 != c)
            rows_bad = bad.any(dim=1).nonzero().flatten()
            cols_bad = bad.any(dim=0).nonzero().flatten()
            truth = tb.matmul(da[rows_bad[:8]].contiguous(), torch.from_numpy(wp_host).to(dev), kernel="generic")
            raise SystemExit(f"rank {rank}: NCCL-gathered C differs from the peer-store C in {int(bad.sum())} entries, "
                             f"rows {rows_bad[:6].tolist()}..{int(rows_bad[-1])} ({rows_bad.numel()}), cols "
                             f"{cols_bad[:6].tolist()}..{int(cols_bad[-1])} ({cols_bad.numel()}); vs generic kernel: "
                             f"peer-store wrong={int((c[rows_bad[:8]] != truth).sum())}, "
                             f"nccl wrong={int((c2[rows_bad[:8]] != truth).sum())}")
        nccl_ms = max_over_ranks(timed(lambda: base.forward(da, out=c2), max(5, args.steps // 4), 3, barrier))
        nccl_ms /= max(5, args.steps // 4)
        del base, c2

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- decode regime: M=1 GEMV over rotating weight copies larger than L2 (rank 0, one GPU)
    gemv = bench_gemv(tb, dev, peaks)

    # ---- CPU baseline on the host cores (bounded sample)
    cpu_tops, cpu_t, cpu_rows, cpu_threads, cpu_kind = cpu_reference_sample(a_host, wp_host, target_s=12.0)

    int8_peak = 2.0 * peaks["bf16_tflops"]
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        # measured for the single-GPU kernel on the whole of config 3; a column shard runs another kernel
        traffic = json.load(open(tpath)).get("gemm_tc3_config3_dram_bytes_per_launch") if world == 1 else None
    kernel_ms = ms_local / args.steps
    local_ops = 2.0 * M * K * shard.n_cols
    line = {
        "metric": "prefill_gemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic",
        "config": {"workload": f"config3 prefill GEMM M={M} K={K} N={N}, W ternary packed 2-bit",
                   "parallelism": (f"N-column shards x{world}; every rank's GEMM epilogue stores its columns into all "
                                   f"ranks' C over NVLink (fused gather) + stream barrier") if world > 1 else "single GPU",
                   "l2": "A+W+C = 562 MB per step exceeds the 126 MB L2; C (470 MB) is rewritten every step",
                   "seed": SEED},
        "shard_compute": {"ms": kernel_ms, "tops_per_gpu": local_ops / (kernel_ms * 1e-3) / 1e12,
                          "columns_rank0": shard.n_cols},
        "roofline": {"bound": "tensor", "achieved": local_ops / (kernel_ms * 1e-3) / 1e12, "peak": int8_peak,
                     "unit": "TOPS", "frac": local_ops / (kernel_ms * 1e-3) / 1e12 / int8_peak, "traffic": traffic,
                     "kernel": "ternary_gemm_tc3_kernel" if world == 1 else "ternary_gemm_tc2_kernel", "peak_source": f"2 x bf16 burst of {peaks['source']} peaks "
                     "(dense int8 proxy)", "frac_of_nominal_4500": local_ops / (kernel_ms * 1e-3) / 1e12 / 4500.0},
        "nccl_gather_baseline": None if nccl_ms is None else {
            "ms_per_step": nccl_ms, "tops": ops / (nccl_ms * 1e-3) / 1e12,
            "what": "same shards, local GEMM then ncclAllGather of C blocks then unpack to row-major"},
        "dequant_bf16_output": dequant,
        "config5_m256": cfg5,
        "gemv": gemv,
        "cpu_baseline": {"value": cpu_tops, "unit": "TOPS", "cores": cpu_threads, "kind": cpu_kind,
                         "sample": f"first {cpu_rows} of {M} rows, full K and N, {cpu_t:.1f} s, avx2_blocked row bands"},
        # N = 1: the reference-facing host-pointer call; N > 1 (no host-pointer multi-GPU entry exists): pinned host
        # activations in, C back out every step, packed weight shards resident
        "e2e": host_call if host_call is not None else {
            "value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": M * K * world, "d2h_bytes_per_step": 4 * M * N,
            "ms_per_step": ms_e2e / e2e_steps,
            "note": "activations copied from pinned host memory and C copied back to pinned host memory every step; "
                    "packed weight shards stay resident"},
        "e2e_weights_resident": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": M * K * world,
                                 "d2h_bytes_per_step": 4 * M * N, "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_config5_m256(tb, dev, world, rank, barrier, max_over_ranks):
    """210 projections (7 per layer x 30 layers) at M=256 in one launch per rank; Q/O/gate/up/down are N-column
    sharded over the ranks with the fused peer-store gather, K/V (N=640) stay whole on every rank."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
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
    for idx in (0, 1, 4, 209):                      # Q, K, gate of layer 0 and `down` of layer 29, every entry
        expect = oracle_lib.matmul(acts[idx].cpu().numpy(), weights[idx])
        if not np.array_equal(outs[idx].cpu().numpy(), expect):
            raise SystemExit(f"rank {rank}: config 5 projection {idx} differs from the CPU oracle")
    reps = 10
    ms = max_over_ranks(timed(pset.run, reps, 3, barrier)) / reps
    return {"workload": "config5: 30 layers x {Q,K,V,O,gate,up,down} of a BitNet-b1.58-2B-shaped model, M=256",
            "projections": 210, "launches_per_rank": pset.launches, "ms": ms, "projections_per_s": 210 / (ms * 1e-3),
            "tops": ops / (ms * 1e-3) / 1e12, "gbs_algorithmic": byts / (ms * 1e-3) / 1e9,
            "sharded": "Q,O,gate,up,down by N columns; K,V whole on every rank" if world > 1 else "single GPU"}


def bench_gemv(tb, dev, peaks):
    """Decode regime, rank 0, one GPU.

    config 1: C[1,6912] = A[1,2560] x W[2560,6912] over 64 distinct weight copies (283 MB > L2), three ways:
      grouped  - all 64 GEMVs in ONE launch of the persistent kernel (ternix_b200_group_run): the throughput figure
      graph    - 64 single-GEMV launches replayed as one CUDA graph
      stream   - 64 single-GEMV launches from Python
    config 5 (M=1): the 210 projections of a 30-layer BitNet-2B-shaped model (521 MB of packed weights) in one launch.
    """
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    copies = 64
    a = tb.synth_activations((1, GEMV_K), SEED + 7)
    ws = [tb.synth_packed_weights(GEMV_K, GEMV_N, SEED + 100 + i) for i in range(4)]
    da = torch.from_numpy(a).to(dev)
    dws = [torch.from_numpy(ws[i % 4]).to(dev).clone() for i in range(copies)]
    outs = [torch.empty((1, GEMV_N), dtype=torch.int32, device=dev) for _ in range(copies)]
    expect = [oracle_lib.matmul(a, ws[i], "scalar") for i in range(4)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    group = tb.ProjectionGroup([(da, dws[i], outs[i]) for i in range(copies)])

    def check(tag):
        torch.cuda.synchronize()
        for i in (0, 1, 2, 3, copies - 1):
            if not np.array_equal(outs[i].cpu().numpy(), expect[i % 4]):
                raise SystemExit(f"GEMV ({tag}) differs from the CPU oracle; refusing to report a number")
            outs[i].fill_(-1)

    def sweep():
        for i in range(copies):
            tb.matmul(da, dws[i], out=outs[i])

    group.run(status=status)
    check("grouped")
    sweep()
    check("single launches")
    if int(status.item()) != 0:
        raise SystemExit("a bounded device-side wait ran out in the grouped GEMV")
    bytes_per = GEMV_K * GEMV_N // 4 + GEMV_K + 4 * GEMV_N
    passes = 20
    us_group = timed(group.run, passes, 5, lambda: None) * 1e3 / (passes * copies)
    # the same 64 GEMVs on prepacked (K-interleaved) copies of the weights: no byte transpose in the kernel
    pre_w = [tb.prepack_k4(w) for w in dws]
    group_pre = tb.ProjectionGroup([(da, pre_w[i], outs[i]) for i in range(copies)], prepacked=True)
    group_pre.run(status=status)
    check("grouped, prepacked")
    us_group_pre = timed(group_pre.run, passes, 5, lambda: None) * 1e3 / (passes * copies)
    del group_pre, pre_w
    us_stream = timed(sweep, 5, 3, lambda: None) * 1e3 / (5 * copies)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        sweep()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            sweep()
    us_graph = timed(g.replay, passes, 3, lambda: None) * 1e3 / (passes * copies)
    gbs = lambda us: bytes_per / (us * 1e-6) / 1e9

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
    for idx in (0, 5, 6, 209):
        A, W, C = probs[idx]
        if not np.array_equal(C.cpu().numpy(), oracle_lib.matmul(A.cpu().numpy(), W.cpu().numpy(), "scalar")):
            raise SystemExit("config 5 projection differs from the CPU oracle; refusing to report a number")
    ms5 = timed(g5.run, passes, 5, lambda: None) / passes
    pre5 = [(A, tb.prepack_k4(W), torch.empty_like(C)) for (A, W, C) in probs]
    g5p = tb.ProjectionGroup(pre5, prepacked=True)
    g5p.run(status=status)
    torch.cuda.synchronize()
    for (A, W, C), (Ap, Wp_, Cp) in zip(probs, pre5):
        if not torch.equal(C, Cp):
            raise SystemExit("config 5: prepacked result differs from the packed-format result")
    ms5p = timed(g5p.run, passes, 5, lambda: None) / passes

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
            "us_per_launch_graph": us_graph, "us_per_launch_stream": us_stream, "gbs_graph": gbs(us_graph),
            "gbs_stream": gbs(us_stream), "algorithmic_bytes_per_gemv": bytes_per,
            "roofline": {"bound": "hbm", "achieved": best, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": best / peaks["hbm_gbs"], "traffic": None, "kernel": "ternary_gemv_group_kernel",
                         "peak_source": f"{peaks['source']} copy bandwidth", "frac_of_nominal_8000": best / 8000.0},
            "config5_m1": {"projections": 210, "launches": g5.launches, "ms": ms5, "projections_per_s": 210 / (ms5 * 1e-3),
                           "gbs": total_bytes / (ms5 * 1e-3) / 1e9, "frac_of_measured_hbm": total_bytes / (ms5 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "algorithmic_bytes": total_bytes},
            "prepacked_weights": {
                "what": "same kernels on ternix_b200_prepack_k4 copies of the weights (same size, four k-rows interleaved per "
                        "packed byte column); the packed format above stays the headline",
                "config1_x64_us_per_gemv": us_group_pre, "config1_x64_gbs": gbs(us_group_pre),
                "config5_m1_ms": ms5p, "config5_m1_gbs": total_bytes / (ms5p * 1e-3) / 1e9,
                "config5_m1_frac_of_measured_hbm": total_bytes / (ms5p * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "config5_m1_frac_of_nominal_8000": total_bytes / (ms5p * 1e-3) / 1e9 / 8000.0},
            "cpu_baseline": {"value": bytes_per / cpu_s / 1e9, "unit": "GB/s", "cores": 1,
                             "kind": "reference" if oracle_lib.have_ref() else "port",
                             "sample": f"one whole GEMV, mean of {reps}, one thread (the kernel cannot slice M=1)"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
