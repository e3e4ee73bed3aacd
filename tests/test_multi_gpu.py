"""N-column sharding on real GPUs: one process per GPU over NCCL.  Skipped when fewer than two GPUs are
visible.  The gathered C of every rank must equal the single-GPU C and the CPU oracle, bit for bit, for
the fused peer-store gather, the NCCL all-gather baseline and the sharded projection set."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle_lib
    import ternixengine_b200 as tb

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        for (m, k, n) in [(512, 1024, 2048), (300, 2064, 1856), (1024, 4096, 4096)]:
            a = tb.synth_activations((m, k), 11 + m)
            wp = tb.synth_packed_weights(k, n, 12 + n)
            expect = oracle_lib.matmul(a, wp)
            da = torch.from_numpy(a).to(dev)
            for mode in ("peer", "nccl"):
                layer = tb.ShardedTernaryLinear(wp, device=dev, mode=mode)
                for _ in range(3):
                    c = layer.forward(da, status=status)
                torch.cuda.synchronize()
                dist.barrier()
                assert int(status.item()) == 0
                assert np.array_equal(c.cpu().numpy(), expect), f"rank {rank}: {mode} gather differs ({m},{k},{n})"
        # activations that change every step, a reader that is late on one rank: the result of step i must not be
        # overwritten by a peer that is already storing step i + 1 (two alternating C buffers)
        m, k, n = 1024, 2048, 4096
        wp = tb.synth_packed_weights(k, n, 5)
        layer = tb.ShardedTernaryLinear(wp, device=dev, mode="peer")
        steps = 6
        acts = [tb.synth_activations((m, k), 200 + i) for i in range(steps)]
        d_acts = [torch.from_numpy(x).to(dev) for x in acts]
        busy = torch.randn((4096, 4096), device=dev)
        kept = []
        for i in range(steps):
            c = layer.forward(d_acts[i], status=status)
            if rank == 0:
                for _ in range(8):
                    busy = busy @ busy * 1e-3               # this rank's reader comes late, on the same stream
            kept.append(c.clone())
        torch.cuda.synchronize()
        dist.barrier()
        assert int(status.item()) == 0
        for i in range(steps):
            assert np.array_equal(kept[i].cpu().numpy(), oracle_lib.matmul(acts[i], wp)), f"rank {rank}: step {i} torn"
        # a small projection set, sharding forced where the shape allows it: two sharded members, one kept whole
        # (N = 640), one decode-regime member; then the automatic plan (BitNet-sized members stay whole)
        shapes = [(256, 2560, 2560), (256, 2560, 640), (256, 2560, 6912), (1, 2560, 2560)]
        weights = [tb.synth_packed_weights(k, n, 70 + i) for i, (m, k, n) in enumerate(shapes)]
        for shard in (True, "auto"):
            for rep in range(3):
                acts_h = [tb.synth_activations((m, k), 80 + i + 10 * rep) for i, (m, k, n) in enumerate(shapes)]
                d_in = [torch.from_numpy(x).to(dev) for x in acts_h]
                if rep == 0:
                    inputs = d_in
                    pset = tb.ShardedProjectionSet(weights, inputs, device=dev, shard=shard)
                    # forced: every member with more than 16 rows and at least 256 columns per rank; automatic: the
                    # gather of a BitNet-sized projection costs more than the compute it saves, so none
                    forced = sum(1 for (m, k, n) in shapes if m > 16 and n // world >= 256)
                    assert pset.sharded_count == (forced if shard is True else 0)
                else:
                    for dst, src in zip(inputs, d_in):
                        dst.copy_(src)                       # same buffers, new activations
                outs = pset.run(status=status)
                torch.cuda.synchronize()
                dist.barrier()
                assert int(status.item()) == 0
                for i, out in enumerate(outs):
                    assert np.array_equal(out.cpu().numpy(), oracle_lib.matmul(acts_h[i], weights[i])), \
                        f"rank {rank}: member {i} (shard={shard}, rep {rep})"
        # the step with host operands: row slabs on three streams; a ragged last slab; C wanted on rank 0 only,
        # then on every rank; new activations on every call
        m, k, n = 1664, 1040, 4096
        wp = tb.synth_packed_weights(k, n, 31)
        layer = tb.ShardedTernaryLinear(wp, device=dev, mode="peer")
        for rep in range(3):
            a = tb.synth_activations((m, k), 300 + rep)
            a_host = torch.from_numpy(a).pin_memory()
            want = rank == 0 or rep == 2
            out_host = torch.full((m, n), -3, dtype=torch.int32).pin_memory() if want else None
            layer.forward_host(a_host, out_host, slab_rows=512, status=status)
            dist.barrier()
            assert int(status.item()) == 0
            if want:
                assert np.array_equal(out_host.numpy(), oracle_lib.matmul(a, wp)), f"rank {rank}: forward_host rep {rep}"
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_sharded_gather_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
