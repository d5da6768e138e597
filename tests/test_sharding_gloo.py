"""world_size-2 gloo test of the data-parallel plumbing (CPU): the loss is a sum
over utterances, so shard losses all-reduced over ranks must equal the
full-batch loss.  The CPU oracle stands in for the CUDA kernels here."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fast_rnnt_b200 import sharding
    from oracle import rnnt_oracle as orc
    from tests import workloads
    wl = workloads.pipeline_workload("small", seed=3)
    keys = ("am", "lm", "symbols", "boundary")
    mine = sharding.shard_batch(wl, keys, rank, world)
    loss = orc.loss_simple(mine["lm"], mine["am"], mine["symbols"], 0, mine["boundary"],
                           reduction="sum")
    total = sharding.allreduce_loss(loss.detach().clone())
    lo, hi = sharding.shard_range(wl["am"].shape[0], rank, world)
    out.put((rank, float(total), lo, hi))
    dist.destroy_process_group()


def test_sharded_loss_equals_full_batch_loss():
    from oracle import rnnt_oracle as orc
    from tests import workloads
    wl = workloads.pipeline_workload("small", seed=3)
    full = float(orc.loss_simple(wl["lm"], wl["am"], wl["symbols"], 0, wl["boundary"],
                                 reduction="sum"))
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[2:] for r in res] == [(0, 3), (3, 6)]
    for r in res:
        assert abs(r[1] - full) <= 1e-5 * abs(full)


def test_shard_ranges_cover_the_batch():
    from fast_rnnt_b200 import sharding
    for batch in (1, 7, 64, 513):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
