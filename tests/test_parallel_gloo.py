"""The (batch, kv-head) partition on two CPU ranks over gloo: shards cover the problem exactly once, each
rank's oracle result equals its rows of the unsharded result bit for bit (no statistic crosses a unit), and
the timing reduction returns the slowest rank's figure."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fa4b_oracle as O
from fa4b import parallel


def test_unit_ranges_cover_everything_once():
    for n, world in ((16, 8), (16, 3), (5, 8), (1, 2)):
        seen = [u for r in range(world) for u in parallel.unit_range(n, world, r)]
        assert seen == list(range(n))
        sizes = [len(parallel.unit_range(n, world, r)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    assert parallel.shard_units(2, 8, 8, 3) == [(0, 6), (0, 7)]
    with pytest.raises(ValueError):
        parallel.unit_range(4, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        B, Hq, Hkv, S, D = 1, 4, 2, 256, 64
        q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=5, rope=False, do_std=0.01)
        qs, ks, vs, dos = parallel.shard_attention_inputs(q, k, v, rank, world, do)
        fwd = O.attn_forward(qs, ks, vs)
        dq, dk, dv = O.attn_backward(qs, ks, vs, fwd.o, fwd.lse, dos)
        gathered = {}
        for name, t in (("o", fwd.o), ("lse", fwd.lse), ("dq", dq), ("dk", dk), ("dv", dv)):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())  # checking only: the data path itself has no collective
            gathered[name] = parts
        slowest = parallel.max_over_ranks(10.0 + rank)
        if rank == 0:
            full = O.attn_forward(q, k, v)
            fdq, fdk, fdv = O.attn_backward(q, k, v, full.o, full.lse, do)
            ok = (torch.equal(parallel.unshard_q_like(gathered["o"], B, Hq), full.o)
                  and torch.equal(parallel.unshard_q_like(gathered["lse"], B, Hq), full.lse)
                  and torch.equal(parallel.unshard_q_like(gathered["dq"], B, Hq), fdq)
                  and torch.equal(parallel.unshard_kv_like(gathered["dk"], B, Hkv), fdk)
                  and torch.equal(parallel.unshard_kv_like(gathered["dv"], B, Hkv), fdv))
            out.put((ok, slowest))
    finally:
        dist.destroy_process_group()


def test_two_rank_partition_reproduces_the_unsharded_result():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    ok, slowest = out.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
    assert slowest == 11.0
