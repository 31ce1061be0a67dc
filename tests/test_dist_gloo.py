"""The multi-rank path on CPU: two gloo ranks shard a decode workload by kv head, each computes its
heads (the oracle stands in for the GPU kernels here), the outputs are all-gathered and must equal
the unsharded result bit for bit; a rank that never joins is detected on the host by a short
process-group timeout."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from attention_rs_b200 import sharding, workloads
from oracle import oracle as O
from tests.helpers import make_case


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_rank_output(c, rank, world):
    nh, nkv = c.q.shape[1], c.key_cache.shape[1]
    kv_lo, kv_hi, q_lo, q_hi = sharding.head_ranges(rank, world, nh, nkv)
    slopes = None if c.alibi_slopes is None else c.alibi_slopes[q_lo:q_hi]
    return O.paged_attention(np.ascontiguousarray(c.q[:, q_lo:q_hi]), np.ascontiguousarray(c.key_cache[:, kv_lo:kv_hi]),
                             np.ascontiguousarray(c.value_cache[:, kv_lo:kv_hi]), c.block_tables, c.context_lens, c.scale,
                             c.dtype, alibi_slopes=slopes)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        c = make_case([5, 300, 77], 8, 4, 64, 16, "bf16", seed=5, alibi=True)
        local = torch.from_numpy(_oracle_rank_output(c, rank, world))
        full = sharding.gather_heads(local)
        slowest = sharding.max_over_ranks(float(rank + 1), torch.device("cpu"))
        if rank == 0:
            want = c.expected()
            ret["equal"] = bool(np.array_equal(full.numpy(), want))
            ret["slowest"] = slowest
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_by_kv_head_and_gather():
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret["equal"] is True
        assert ret["slowest"] == 2.0


def test_head_ranges_and_workload_shard():
    assert sharding.head_ranges(1, 2, 32, 8) == (4, 8, 16, 32)
    assert sharding.head_ranges(7, 8, 64, 8) == (7, 8, 56, 64)
    with pytest.raises(ValueError):
        sharding.head_ranges(0, 3, 32, 8)
    w = workloads.decode_workload(5, num_seqs=2, ctx_range=(100, 200))
    parts = [w.shard(r, 4) for r in range(4)]
    assert all(p.num_kv_heads == 2 and p.num_heads == 8 for p in parts)
    assert np.array_equal(np.concatenate([p.alibi_slopes for p in parts]), w.alibi_slopes)
    assert sum(p.kv_bytes() for p in parts) == w.kv_bytes()
    q = torch.zeros((3, 32, 16))
    assert sharding.shard_query(q, 1, 4, 8).shape == (3, 8, 16) and sharding.shard_query(q, 1, 4, 8).stride(0) == 512
    cache = torch.arange(2 * 8 * 4).reshape(2, 8, 4)
    assert torch.equal(sharding.shard_cache(cache, 3, 4), cache[:, 6:8])


def _absent_peer(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            return            # leaves between steps, with nothing in flight, and never joins the gather
        try:
            sharding.gather_heads(torch.zeros((1, 2, 4)))
            ret["error"] = None
        except Exception as exc:      # the short timeout turns the missing peer into a host-side error
            ret["error"] = type(exc).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_surfaces_as_host_error():
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_absent_peer, args=(2, port, ret), nprocs=2, join=True)
        assert ret.get("error") is not None
