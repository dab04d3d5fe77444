"""Multi-GPU host logic on CPU: two gloo ranks each derive their shard of a
workload the way `bench.py --gpus 2` does; together the shards must tile the
global problem exactly (no unit dropped or duplicated) and no collective is
needed to agree on the split."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = {}
        for name in ("target", "gqa", "varlen", "skewed"):
            wl = bench.describe(name, rank, world)
            acct = bench.accounting(wl)
            mine[name] = dict(seqlens=wl["seqlens"], hq=wl["hq"], hkv=wl["hkv"], flops=acct["f_step"],
                              scaling=wl["scaling"], seed=wl["seed"])
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        # max-over-ranks timing, as the benchmark reduces it
        t = torch.tensor([1.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            out.put((gathered, float(t)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_tile_every_workload():
    world, port = 2, 29511 + (os.getpid() % 200)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    gathered, tmax = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tmax == 2.0
    # head-sharded strong scaling: the KV heads of all ranks add up to 8, 4 query heads each
    for name in ("gqa", "skewed"):
        assert sum(g[name]["hkv"] for g in gathered) == 8
        assert all(g[name]["hq"] == 4 * g[name]["hkv"] for g in gathered)
        one = bench.accounting(bench.describe(name, 0, 1))["f_step"]
        assert abs(sum(g[name]["flops"] for g in gathered) - one) < 1e-6 * one
    # sequence-sharded: every sequence exactly once, token counts balanced by LPT
    lens = sorted(bench.varlen_lengths())
    assert sorted(sum((g["varlen"]["seqlens"] for g in gathered), [])) == lens
    assert sum(lens) == 262144 and len(lens) == 32
    loads = [sum(g["varlen"]["seqlens"]) for g in gathered]
    assert max(loads) <= 1.01 * sum(loads) / world
    # weak scaling: identical per-rank work, different seeds
    assert gathered[0]["target"]["flops"] == gathered[1]["target"]["flops"]
    assert gathered[0]["target"]["seed"] != gathered[1]["target"]["seed"]
    assert gathered[0]["target"]["scaling"] == "weak" and gathered[0]["gqa"]["scaling"] == "strong"


def test_pair_counts_of_the_accounting_match_the_oracle_closed_forms():
    from oracle import moba_oracle as orc
    for s in (128, 1000, 4096, 29312):
        assert bench.attended_pairs(s) == orc.attended_pairs(s, 128, 8)
        assert bench.selected_pairs(s) == orc.selected_pairs(s, 128, 8)
    wl = bench.describe("target", 0, 1)
    acct = bench.accounting(wl)
    assert acct["pairs"] == 4179968 and round(acct["f_fwd"] / 1e9, 2) == 128.45
