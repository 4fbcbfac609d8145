"""The N > 1 path on CPU: two gloo ranks shard a decode by KV-head group, take
identical allocator decisions, compute their heads (the oracle stands in for
the GPU kernels here) and gather; the result equals the single-rank result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_oracle as co
from oracle import paged_oracle as po


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_case():
    rng, lens, tables, n_pool = po.make_decode_case(77, 6, 1, 90, 8, 4, head_dim=32, block_size=16, spare_blocks=2)
    k = rng.standard_normal((n_pool, 4, 16, 32), dtype=np.float32)
    v = rng.standard_normal((n_pool, 4, 16, 32), dtype=np.float32)
    q = rng.standard_normal((6, 8, 32), dtype=np.float32)
    return q, k, v, tables, lens


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import pagedattentionmetal_b200 as pam
    from pagedattentionmetal_b200 import sharding

    q, k, v, tables, lens = _make_case()
    q_lo, q_hi, kv_lo, kv_hi = sharding.head_range(rank, world, 8, 4)
    assert (q_hi - q_lo, kv_hi - kv_lo) == (8 // world, 4 // world)
    # every rank replays the same allocator calls on its own (bookkeeping) manager
    m = pam.KVCacheManager(None, 64, 16)
    for sid, L in enumerate(lens):
        m.allocateSequence(sid)
        m.appendTokens(sid, int(L), [100 + sid] if sid % 2 == 0 else None)
    m.freeSequence(1)
    m.allocateSequence(9)
    m.appendTokens(9, 40)
    mine = torch.tensor(sum((m.getBlockTable(s) for s in (0, 2, 3, 4, 5, 9)), []), dtype=torch.int64)
    other = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(other, mine)
    assert all(torch.equal(o, mine) for o in other), "block tables differ between ranks"
    # its heads only: pools sliced on the kv-head axis, queries on the head axis
    k_loc = np.ascontiguousarray(sharding.shard_heads(k, rank, world, 1))
    v_loc = np.ascontiguousarray(sharding.shard_heads(v, rank, world, 1))
    q_loc = np.ascontiguousarray(sharding.shard_heads(q, rank, world, 1))
    assert q_loc.shape[1] == q_hi - q_lo and k_loc.shape[1] == kv_hi - kv_lo
    out_loc = co.decode(q_loc, k_loc, v_loc, tables, lens, kv_hi - kv_lo, 16, po.DT_F32, window=33)
    full = sharding.gather_heads(torch.from_numpy(out_loc))
    # timing reduction used by the benchmark: max over ranks
    tmax = torch.tensor([float(rank + 1)])
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    assert tmax.item() == world
    if rank == 0:
        results.put(full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_kv_head_sharding_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    full = results.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    q, k, v, tables, lens = _make_case()
    ref = co.decode(q, k, v, tables, lens, 4, 16, po.DT_F32, window=33)
    assert full.shape == ref.shape
    assert np.array_equal(full, ref)          # same arithmetic per head: bit-identical


def test_head_range_rules():
    from pagedattentionmetal_b200 import sharding
    assert sharding.head_range(3, 8, 32, 8) == (12, 16, 3, 4)
    assert sharding.head_range(0, 1, 32, 8) == (0, 32, 0, 8)
    with pytest.raises(ValueError):
        sharding.head_range(0, 3, 32, 8)
