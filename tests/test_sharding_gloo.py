"""The N > 1 host path on CPU: two gloo ranks shard the packed weights by columns, each computes its
columns (with the CPU oracle standing in for the GPU kernel), the equal-sized blocks are all-gathered and
unpacked to row-major C.  Checks shard bounds, padding and gather offsets against the unsharded product."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, shape, granule, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    import ternixengine_b200 as tb

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = shape
        a = tb.synth_activations((M, K), 5)
        wp = tb.synth_packed_weights(K, N, 6)                       # every rank regenerates the same bytes
        sh = tb.shard_columns(N, world, rank, granule)
        local_w = tb.slice_columns(wp, sh.n0, sh.n_cols)            # this rank's packed shard
        block = np.zeros((M, sh.n_pad), dtype=np.int32)
        if sh.n_cols:
            block[:, :sh.n_cols] = oracle_lib.matmul(a, local_w)    # stand-in for the GPU kernel
            # the shard is a valid packed matrix: same result as slicing the full product
            assert np.array_equal(block[:, :sh.n_cols], oracle_lib.matmul_columns(a, wp, sh.n0, sh.n_cols))
        blocks = [torch.empty((M, sh.n_pad), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(blocks, torch.from_numpy(block))
        gathered = torch.stack(blocks).numpy()
        c = tb.gathered_to_row_major(gathered, N, granule)
        assert np.array_equal(c, oracle_lib.matmul(a, wp)), f"rank {rank}: gathered C differs"
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape,granule", [(2, (5, 96, 640), 64), (2, (3, 64, 192), 64), (3, (4, 40, 1028), 4),
                                                 (2, (2, 32, 64), 64)])
def test_column_sharded_product_over_gloo(world, shape, granule, tmp_path):
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, shape, granule, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_should_shard_policy():
    sys.path.insert(0, ROOT)
    import ternixengine_b200 as tb
    # config 3 (K = 8192, int32 C on every rank): the gather hides under the compute at 2 and 4 GPUs, not at 8
    assert tb.should_shard(4096, 8192, 28672, 2)
    assert not tb.should_shard(4096, 8192, 28672, 4)               # the gather (0.59 ms) outweighs one GPU's 0.55 ms
    assert not tb.should_shard(4096, 8192, 28672, 8)
    assert tb.should_shard(4096, 8192, 28672, 8, out_bytes=2)      # bfloat16 outputs halve the gather
    assert tb.should_shard(4096, 32768, 8192, 8)                   # deep K: compute dominates
    # BitNet-2B projections (K = 2560 / 6912): shipping int32 C costs more than the compute it saves
    assert not tb.should_shard(256, 2560, 6912, 8)
    assert not tb.should_shard(256, 6912, 2560, 2)
    assert not tb.should_shard(256, 2560, 640, 8)        # K/V projections: 80 columns per rank
    assert not tb.should_shard(1, 2560, 6912, 8)         # decode regime is never sharded
    assert not tb.should_shard(4096, 8192, 28672, 1)


def _protocol_rank(rank, world, port, tmp):
    """The two-buffer gather protocol of ShardedTernaryLinear with CPU ranks: memory-mapped files stand in for the
    peer-mapped C buffers, the oracle for the GPU kernel, a gloo barrier for the stream barrier.  The activations
    change every step and one rank reads its result late, while the others are already storing the next step."""
    import time
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    import ternixengine_b200 as tb

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 6, 64, 384
        wp = tb.synth_packed_weights(K, N, 3)
        sh = tb.shard_columns(N, world, rank, 64)
        local_w = tb.slice_columns(wp, sh.n0, sh.n_cols)
        for b in range(2):                                   # this rank's two C buffers
            np.lib.format.open_memmap(os.path.join(tmp, f"c{rank}_{b}.npy"), mode="w+", dtype=np.int32, shape=(M, N))[:] = -1
        dist.barrier()
        bufs = [[np.load(os.path.join(tmp, f"c{r}_{b}.npy"), mmap_mode="r+") for b in range(2)] for r in range(world)]
        for step in range(8):
            a = tb.synth_activations((M, K), 100 + step)     # new activations every step
            b = tb.gather_buffer_index(step)
            mine = oracle_lib.matmul(a, local_w)
            for r in range(world):                           # the epilogue's stores into every rank's C
                bufs[r][b][:, sh.n0:sh.n0 + sh.n_cols] = mine
                bufs[r][b].flush()
            dist.barrier()                                   # all stores of this step have landed
            if rank == 0:
                time.sleep(0.05)                             # a slow reader: the other ranks run ahead into the next step
            got = np.array(bufs[rank][b])
            assert np.array_equal(got, oracle_lib.matmul(a, wp)), f"rank {rank} step {step}: torn or stale C"
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_buffer_gather_protocol_over_gloo(tmp_path):
    world = 2
    mp.spawn(_protocol_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
