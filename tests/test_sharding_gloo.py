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


def test_host_slab_plan():
    """forward_host's slab extent: about 64 MB of C per slab, whole 256-row tiles, at most 16 slabs, never above M."""
    sys.path.insert(0, ROOT)
    import ternixengine_b200 as tb
    assert tb.host_slab_rows(4096, 28672) == 768                   # config 3: 470 MB of C in 6 slabs
    assert tb.host_slab_rows(100, 1024) == 100                     # small products are one slab
    assert tb.host_slab_rows(1, 6912) == 1
    assert tb.host_slab_rows(0, 64) == 0
    for (m, n) in [(4096, 28672), (65536, 8192), (300, 832), (1 << 20, 4096), (5000, 100000)]:
        rows = tb.host_slab_rows(m, n)
        assert 0 < rows <= m and (rows % 256 == 0 or rows == m)
        assert -(-m // rows) <= 16


def test_should_shard_policy():
    sys.path.insert(0, ROOT)
    import ternixengine_b200 as tb
    # config 3 (K = 8192, int32 C on every rank): sharding pays at 2 GPUs, not at 4 or 8
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


class _FlagBarrier:
    """ternix_b200_peer_barrier restated on memory-mapped files: rank r's flag array has one slot per rank; arriving
    means writing the epoch into slot `rank` of every peer's array, then waiting (with a limit) until every peer's
    epoch shows in the own array.  Epochs only grow, so `>=` is the test."""

    def __init__(self, tmp, rank, world):
        self.rank, self.world, self.epoch = rank, world, 0
        self.flags = [np.load(os.path.join(tmp, f"flags{r}.npy"), mmap_mode="r+") for r in range(world)]

    @staticmethod
    def create(tmp, rank, world):
        np.lib.format.open_memmap(os.path.join(tmp, f"flags{rank}.npy"), mode="w+", dtype=np.uint32, shape=(world,))[:] = 0

    def __call__(self, limit_s=20.0):
        import time
        self.epoch += 1
        for t in range(self.world):
            if t != self.rank:
                self.flags[t][self.rank] = self.epoch
                self.flags[t].flush()
        t0 = time.monotonic()
        for t in range(self.world):
            while t != self.rank and int(self.flags[self.rank][t]) < self.epoch:
                if time.monotonic() - t0 > limit_s:
                    return False                      # the status word's timeout code; nothing hangs
                time.sleep(0.0005)
        return True


def _protocol_rank(rank, world, port, tmp, barrier_kind="gloo"):
    """The two-buffer gather protocol of ShardedTernaryLinear with CPU ranks: memory-mapped files stand in for the
    peer-mapped C buffers, the oracle for the GPU kernel, and either a gloo barrier or the flag protocol of
    ternix_b200_peer_barrier (restated above) for the stream barrier.  The activations
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
        _FlagBarrier.create(tmp, rank, world)
        dist.barrier()
        flag_barrier = _FlagBarrier(tmp, rank, world)
        bufs = [[np.load(os.path.join(tmp, f"c{r}_{b}.npy"), mmap_mode="r+") for b in range(2)] for r in range(world)]
        for step in range(8):
            a = tb.synth_activations((M, K), 100 + step)     # new activations every step
            b = tb.gather_buffer_index(step)
            mine = oracle_lib.matmul(a, local_w)
            for r in range(world):                           # the epilogue's stores into every rank's C
                bufs[r][b][:, sh.n0:sh.n0 + sh.n_cols] = mine
                bufs[r][b].flush()
            if barrier_kind == "gloo":
                dist.barrier()                               # all stores of this step have landed
            else:
                assert flag_barrier(), f"rank {rank} step {step}: a peer did not arrive"
            if rank == 0:
                time.sleep(0.05)                             # a slow reader: the other ranks run ahead into the next step
            got = np.array(bufs[rank][b])
            assert np.array_equal(got, oracle_lib.matmul(a, wp)), f"rank {rank} step {step}: torn or stale C"
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,barrier_kind", [(2, "gloo"), (2, "flags"), (3, "flags")])
def test_two_buffer_gather_protocol_over_gloo(world, barrier_kind, tmp_path):
    mp.spawn(_protocol_rank, args=(world, _free_port(), str(tmp_path), barrier_kind), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_flag_barrier_gives_up_on_an_absent_peer(tmp_path):
    """A peer that never arrives: the wait runs out and reports it, as the kernel does through the status word."""
    for r in range(2):
        _FlagBarrier.create(str(tmp_path), r, 2)
    assert _FlagBarrier(str(tmp_path), 0, 2)(limit_s=0.2) is False
