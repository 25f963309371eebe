"""Multi-GPU host logic on CPU: how configs shard over ranks, and the world-size-2 gather that
validates shards against the unsharded oracle (gloo; the GPU run uses NCCL for the same step)."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sdpa_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_never_splits_a_gqa_group():
    c3 = O.CONFIGS["C3"]
    for world in (1, 2, 4, 8):
        s = O.shard(c3, 0, world)
        assert s.Hq // s.Hkv == c3.Hq // c3.Hkv
        assert s.B * s.Hkv * world == c3.B * c3.Hkv
    c4 = O.shard(O.CONFIGS["C4"], 3, 8)
    assert (c4.B, c4.Hq, c4.Hkv) == (1, 4, 4)
    c5 = O.shard(O.CONFIGS["C5"], 0, 8)
    assert (c5.B, c5.Hq) == (8, 16)
    c2 = O.shard(O.CONFIGS["C2"], 0, 8)
    assert c2.B == 1 and c2.Hq == 12
    with pytest.raises(ValueError):
        O.shard(O.CONFIGS["C3"], 0, 3)


def test_bench_shard_slices_tile_the_problem_and_agree_with_the_config_shards():
    """bench.py's strong-scaling split: the ranks' (batch, head) slices are disjoint, cover the
    problem, never cut a GQA group and have the shape oracle.shard() names."""
    sys.path.insert(0, ROOT)
    import bench

    for name, worlds in (("C4", (2, 4, 8)), ("C5", (2, 4, 8)), ("C3", (2, 4, 8, 16, 32)), ("C2", (2, 4, 8))):
        cfg = O.CONFIGS[name]
        group = cfg.Hq // cfg.Hkv
        for world in worlds:
            seen_q = torch.zeros(cfg.B, cfg.Hq, dtype=torch.int32)
            seen_k = torch.zeros(cfg.B, cfg.Hkv, dtype=torch.int32)
            for rank in range(world):
                bs, qs, ks = bench.shard_slices(cfg, rank, world)
                seen_q[bs, qs] += 1
                seen_k[bs, ks] += 1
                part = O.shard(cfg, rank, world)
                assert seen_q[bs, qs].shape == (part.B, part.Hq) and seen_k[bs, ks].shape == (part.B, part.Hkv)
                q_heads = torch.arange(cfg.Hq)[qs]
                k_heads = torch.arange(cfg.Hkv)[ks]
                assert torch.equal(q_heads // group, k_heads.repeat_interleave(group))
            assert torch.all(seen_q == 1) and torch.all(seen_k == 1)
    with pytest.raises(ValueError):
        bench.shard_slices(O.CONFIGS["C3"], 0, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank derives the full problem from the seed and takes its (batch) slice: shards are
    # bit-identical to the corresponding rows of the single-process run
    B, H, S, D = 4, 2, 64, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
    per = B // world
    sl = slice(rank * per, (rank + 1) * per)
    out, lse = O.sdpa_forward(q[sl], k[sl], v[sl], True, 0.125)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        full, _ = O.sdpa_forward(q, k, v, True, 0.125)
        torch.save({"err": (torch.cat(gathered) - full).abs().max().item(), "max": t.item()}, result_path)
    dist.destroy_process_group()


def test_world_size_two_gather_matches_unsharded(tmp_path):
    path = str(tmp_path / "result.pt")
    mp.spawn(_worker, args=(2, _free_port(), path), nprocs=2, join=True)
    res = torch.load(path)
    assert res["err"] < 1e-6 and res["max"] == 2.0


def _leaver_worker(rank, world, port, result_path):
    """Rank 1 leaves between steps (after a completed gather, before the next one); rank 0 must
    learn of it from a bounded collective, on the host, and report instead of waiting forever."""
    import datetime

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)   # step 0 completes on every rank
    if rank == 1:
        os._exit(0)                             # gone before step 1, nothing of its own in flight
    detected = ""
    try:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    except Exception as exc:  # gloo reports a closed connection or its timeout
        detected = type(exc).__name__
    torch.save({"first": t.item(), "detected": detected}, result_path)
    os._exit(0)                                 # the group is broken; skip its teardown


def test_rank_that_leaves_before_the_gather_is_detected_on_the_host(tmp_path):
    path = str(tmp_path / "leaver.pt")
    ctx = mp.spawn(_leaver_worker, args=(2, _free_port(), path), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(60)
        assert not p.is_alive(), "a rank is still waiting on a peer that left"
    res = torch.load(path)
    assert res["first"] == 1.0
    assert res["detected"], "the surviving rank did not notice the missing peer"
