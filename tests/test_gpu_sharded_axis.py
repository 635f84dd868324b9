"""Reduction along the sharded axis on real GPUs: each rank reduces its k block with the CUDA kernel,
NCCL combines the partials. Needs at least two GPUs in the box; skipped otherwise (the combine logic
itself is covered on CPU over gloo in test_shard_gloo.py)."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import binding as O
        from tcacomp_b200.shard import block
        from tcacomp_b200.sharded import reduce_outer_sharded_k
        rng = np.random.default_rng(77)                       # the same tensor on every rank
        t = rng.uniform(-100, 100, (8, 600, 260)).astype(np.float32)
        t[0, 10, :] = 500.0
        t[0, 450, :] = 500.0                                   # a tie across shards
        lo, hi = block(t.shape[1], world, rank)
        res = reduce_outer_sharded_k(torch.from_numpy(np.ascontiguousarray(t[:, lo:hi])).to(dev), lo)
        torch.cuda.synchronize()
        if rank == 0:
            s, m, a = O.reduce_outer(t)
            ok = (np.array_equal(res["argmax"].cpu().numpy(), a) and np.array_equal(res["max"].cpu().numpy(), m)
                  and bool((np.abs(res["sum"].cpu().numpy() - s) <= 1e-5 * np.abs(t).sum(1)).all()))
            q.put(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_axis_reduce_with_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=300)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ok
