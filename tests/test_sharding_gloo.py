"""Host logic of the multi-GPU path, exercised with world_size-2 gloo ranks on the CPU: document sharding covers
every document exactly once, the packed layout obeys the kernels' contract, and the timing reduction used by
bench.py (max over ranks) behaves."""
import os
import random

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from xlstm_b200.ops import prepare_cu_seqlens
from xlstm_b200.sharding import SlotPool, pack_documents, shard_documents


def _lengths(n=64, seed=0):
    rnd = random.Random(seed)
    return [max(16, min(16384, int(rnd.lognormvariate(6.93, 1.0)))) for _ in range(n)]


def test_packing_obeys_kernel_contract():
    lens = _lengths(100)
    pk = pack_documents(lens, 32768)
    cu, nd = prepare_cu_seqlens(pk.cu_seqlens, pk.rows, pk.row_len, "cpu")   # raises if a document straddles a row
    assert nd == len(pk.doc_ids)
    real = [d for d in pk.doc_ids if d >= 0]
    assert sorted(real) == list(range(len(lens)))
    for i, d in enumerate(pk.doc_ids):
        if d >= 0:
            assert pk.cu_seqlens[i + 1] - pk.cu_seqlens[i] == lens[d]
    with pytest.raises(ValueError):
        pack_documents([40000], 32768)


def test_slot_pool_reuses_slots():
    pool = SlotPool(2)
    a, b = pool.acquire("x"), pool.acquire("y")
    with pytest.raises(RuntimeError):
        pool.acquire("z")
    pool.release(a)
    assert pool.acquire("z") == a and {a, b} == {0, 1}
    with pytest.raises(KeyError):
        pool.release(7)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lens = _lengths(64, seed=1)
    mine = shard_documents(lens, world)[rank]
    # every rank reports its documents; together they must be a partition
    got = [None] * world
    dist.all_gather_object(got, mine)
    tokens = torch.tensor([float(sum(lens[i] for i in mine))])
    t = torch.tensor([10.0 + rank], dtype=torch.float64)   # stand-in for a per-rank device time
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total = tokens.clone()
    dist.all_reduce(total)
    if rank == 0:
        q.put((got, float(t), float(total), float(tokens)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_partition_and_max_reduce():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + random.randint(0, 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got, tmax, total, tok0 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    lens = _lengths(64, seed=1)
    assert sorted(got[0] + got[1]) == list(range(64)) and not set(got[0]) & set(got[1])
    assert tmax == 11.0 and total == float(sum(lens))
    assert abs(tok0 - total / 2) <= max(lens)     # balanced to within one document
