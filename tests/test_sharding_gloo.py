"""world_size-2 CPU test (gloo) of the multi-GPU plumbing: contiguous shards of independent
signals, no collective on the data path, optional final gather, max-over-ranks timing.  The
per-rank compute here is the CPU port (there is no GPU in this test); on GPUs each rank runs the
CUDA path on its own shard in exactly this arrangement."""
import os
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from metalaudio_b200.sharding import gather_rows, max_over_ranks, shard_range
    from oracle import configs, reference_path as rp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_signals, length, n, hop = 5, 4096, 256, 64
    lo, hi = shard_range(n_signals, rank, world)
    x = configs.c2_signals(hi - lo, length, first_signal=lo)      # this rank's signals only
    w = rp.window("hann", n)
    mags = np.stack([rp.magnitude(*rp.stft(s, n, hop, w)) for s in x]) if hi > lo else np.zeros((0, 1, 1), np.float32)
    full = gather_rows(torch.from_numpy(mags), n_signals)
    worst = max_over_ranks(float(rank + 1))
    if rank == 0:
        q.put((full.numpy(), worst))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_and_gather():
    sys.path.insert(0, ROOT)
    from oracle import configs, reference_path as rp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    full, worst = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = configs.c2_signals(5, 4096)
    w = rp.window("hann", 256)
    ref = np.stack([rp.magnitude(*rp.stft(s, 256, 64, w)) for s in x])
    assert full.shape == ref.shape and np.array_equal(full, ref)
    assert worst == 2.0
