"""The multi-rank host logic on CPU: world_size-2 gloo processes partition the
independent axis, each 'computes' its block (here with the oracle standing in
for a device), and the union equals the single-rank result. No data-path
collective is involved; gloo only carries the check."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_blocks_cover_exactly_once():
    from tcacomp_b200.shard import block, blocks
    for n in (0, 1, 7, 8, 16384, 65537):
        for w in (1, 2, 3, 4, 8):
            bl = blocks(n, w)
            assert bl[0][0] == 0 and bl[-1][1] == n
            assert all(bl[i][1] == bl[i + 1][0] for i in range(w - 1))
            sizes = [hi - lo for lo, hi in bl]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        block(4, 2, 2)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import binding as O
        from tcacomp_b200.shard import block
        rng = np.random.default_rng(123)  # identical seeded input on every rank
        x = (4 * rng.normal(0, 1, (101, 64))).astype(np.float32)
        lo, hi = block(x.shape[0], world, rank)
        mine = O.softmax_rows(np.ascontiguousarray(x[lo:hi]))
        # gather only to verify; the timed path never exchanges data
        parts = [None] * world
        dist.all_gather_object(parts, (lo, hi, mine))
        # max-over-ranks timing reduction, as the benchmark does it
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            full = np.concatenate([p[2] for p in sorted(parts, key=lambda p: p[0])])
            q.put((np.array_equal(full, O.softmax_rows(x)), float(t.item())))
    finally:
        dist.destroy_process_group()


def test_two_rank_partition_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok, tmax = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert ok and tmax == 2.0


def _sharded_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import binding as O
        from tcacomp_b200.shard import block
        from tcacomp_b200.sharded import combine_partials
        rng = np.random.default_rng(5)
        t = rng.integers(-4, 5, (3, 40, 17)).astype(np.float32)   # many equal maxima across the two shards
        t[0, :, 0] = 2.0                 # a tie spanning both shards: global index 0 must win
        t[1, 25:, 1] = 9.0               # the maximum lives only in the second shard
        t[2, :, 2] = -np.inf             # -inf everywhere: index 0
        t[2, 3, 3] = np.nan              # a NaN never wins
        lo, hi = block(t.shape[1], world, rank)
        s, m, a = O.reduce_outer(np.ascontiguousarray(t[:, lo:hi]))   # the oracle stands in for the device kernel
        part = {"sum": torch.from_numpy(s), "max": torch.from_numpy(m), "argmax": torch.from_numpy(a)}
        out = combine_partials(part, lo)
        if rank == 0:
            fs, fm, fa = O.reduce_outer(t)
            ok_idx = np.array_equal(out["argmax"].numpy(), fa)
            ok_max = np.array_equal(out["max"].numpy(), fm)
            both = np.isfinite(fs)
            ok_sum = np.array_equal(out["sum"].numpy()[both], fs[both])   # small integers: exact in any order
            q.put((ok_idx, ok_max, ok_sum))
    finally:
        dist.destroy_process_group()


def test_reduction_along_the_sharded_axis_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert res == (True, True, True)


def test_run_block_queues_exactly_this_ranks_slices():
    """multi.run_block: every rank queues its own contiguous block of the GLOBAL host buffers through its pipeline,
    a rank whose block is empty queues nothing, and the blocks of all ranks tile the problem (fake pipeline: the
    host logic needs no device)."""
    from tcacomp_b200 import multi

    class FakePipeline:
        def __init__(self):
            self.calls = []

        def run(self, ins, outs, n):
            self.calls.append((ins, outs, n))
            for i, o in zip(ins, outs):
                o.copy_(i * 2)

    for units in (0, 1, 3, 16, 17):
        for world in (1, 2, 3, 4):
            x = torch.arange(units * 5, dtype=torch.float32).view(units, 5)
            y = torch.full_like(x, -1.0)
            total = 0
            for rank in range(world):
                pipe = FakePipeline()
                n = multi.run_block(pipe, [x], [y], units, world, rank)
                views, m = multi.block_views([x], units, world, rank)
                assert m == n == views[0].shape[0]
                assert len(pipe.calls) == (1 if n > 0 else 0)
                if n:
                    assert pipe.calls[0][0][0].data_ptr() == views[0].data_ptr()   # a view of the global buffer, no copy
                total += n
            assert total == units and torch.equal(y, x * 2)
