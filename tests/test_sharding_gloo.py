"""Multi-rank host logic on CPU (gloo, world size 2): request sharding and the max-time / summed-work
reduction the benchmark uses.  No GPU, no data-path collective."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kestrel_b200.sharding import combine_step_stats, gather_rank_stats, owner_of, shard_bounds, whole_job_rate


def test_shard_bounds_cover_everything_once():
    for n in (0, 1, 7, 2048, 2049):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = shard_bounds(n, world, r)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
                for i in (lo, hi - 1):
                    if lo < hi:
                        assert owner_of(i, n, world) == r
            assert seen == list(range(n))
            sizes = [shard_bounds(n, world, r)[1] - shard_bounds(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    assert shard_bounds(2048, 8, 3) == (768, 1024)
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_combine_without_process_group_is_identity():
    assert combine_step_stats(3.5, 10.0) == (3.5, 10.0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = shard_bounds(2048, world, rank)
        # every rank "runs" its shard: time and work depend on the rank
        elapsed, units = combine_step_stats(10.0 + rank, float(hi - lo))
        # what the benchmark does after its timed region: every rank's (time, bytes) side by side
        per = gather_rank_stats([10.0 + rank, 1000.0 * (hi - lo)])
        # page tables are rank-local: the same page index on two ranks names two different pages
        from kestrel_b200.kv_cache import PageTable
        pt = PageTable(n_pages=16, page_size=16, max_batch_size=4, device="cpu")
        row = pt.allocate()
        pt.reserve(row, 40 + rank)
        pages = torch.tensor(pt.page_table_cpu[row][:3])
        gathered = [torch.zeros_like(pages) for _ in range(world)]
        dist.all_gather(gathered, pages)
        out.put((rank, elapsed, units, [g.tolist() for g in gathered], per.tolist()))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_combine():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    results = sorted(q.get(timeout=120) for _ in range(world))
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    for rank, elapsed, units, gathered, per in results:
        assert elapsed == 11.0          # max over ranks
        assert units == 2048.0          # sum over ranks
        assert gathered[0] == gathered[1] == [3, 2, 1]   # identical local numbering, independent pools
        assert per == [[10.0, 1024000.0], [11.0, 1024000.0]]      # the same table on every rank, row = rank
        t, rate, own = whole_job_rate(torch.tensor(per)[:, 0], torch.tensor(per)[:, 1])
        assert t == 11.0 and rate == pytest.approx(2048000.0 / 11e-3)      # everybody's work over the slowest rank
        assert own == pytest.approx([1024000.0 / 10e-3, 1024000.0 / 11e-3])


def test_whole_job_rate_of_one_rank_is_its_own_rate():
    per = gather_rank_stats([4.0, 8e9])
    assert per.shape == (1, 2)
    t, rate, own = whole_job_rate(per[:, 0], per[:, 1])
    assert t == 4.0 and rate == pytest.approx(2e12) and own == pytest.approx([2e12])
