"""The N>1 host logic on CPU: two gloo ranks shard batch x heads without exchanging data and
reproduce the unsharded answer; the benchmark's max-over-ranks reduction."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from based_b200.sharding import max_over_ranks, shard_range, sum_over_ranks
    from oracle import based_oracle as O
    g = torch.Generator().manual_seed(0)
    B, H, dv = 5, 2, 16
    kv = torch.randn(B, H, 1, dv, 273, generator=g, dtype=torch.float64)
    ks = torch.rand(B, H, 1, 1, 273, generator=g, dtype=torch.float64) + 1
    qq, kk = torch.randn(B, H, 1, 16, generator=g, dtype=torch.float64), torch.randn(B, H, 1, 16, generator=g, dtype=torch.float64)
    vv = torch.randn(B, H, 1, dv, generator=g, dtype=torch.float64)
    s, e = shard_range(B, rank, world)
    y = O.linattn_recurrent_step(kv[s:e].clone(), ks[s:e].clone(), qq[s:e], kk[s:e], vv[s:e])
    full = O.linattn_recurrent_step(kv.clone(), ks.clone(), qq, kk, vv)
    ok = torch.equal(y, full[s:e])  # shards are bit-identical to the unsharded run: no cross-unit arithmetic
    mx = max_over_ranks([1.0 + rank, 5.0 - rank], "cpu")
    sm = sum_over_ranks([e - s], "cpu")
    q.put((rank, ok, mx, sm, (s, e)))
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[4] for r in res] == [(0, 3), (3, 5)]
    for rank, ok, mx, sm, _ in res:
        assert ok
        assert mx == [2.0, 5.0]
        assert sm == [5.0]


def test_shard_range_covers_everything():
    from based_b200.sharding import shard_range
    for total in (0, 1, 7, 256, 4096):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
