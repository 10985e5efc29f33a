"""Multi-rank host logic on CPU (gloo, world_size 2): the two partitionings the
decode path supports — KV heads per rank and sequences per rank with local block
pools — reproduce the unsharded result when the rank outputs are all-gathered.
The compute on each rank is the CPU oracle (the product itself has no CPU path);
what is under test is the sharding plan and the gather layout."""
import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle(w):
    from oracle import paged_oracle as O
    return O.paged_attention(w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                             w.block_tables, w.seq_lens, w.alibi_slopes, w.kv_cache_dtype,
                             float(w.k_scale), float(w.v_scale), mode="ref", partition_size=512)


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from vllm_b200 import workloads as W
        # every rank derives the same full plan from the same seed
        full = W.small("cpu", seed=21, num_seqs=6, num_heads=8, num_kv_heads=4, head_size=64,
                       max_len=700, num_blocks=256)
        want = _oracle(full)

        # (i) KV heads per rank: outputs concatenate along the head dimension
        mine = W.shard_kv_heads(full, world, rank)
        assert mine.key_cache.shape[1] == 4 // world and mine.query.shape[1] == 8 // world
        out = _oracle(mine).contiguous()
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)
        ok_heads = torch.equal(torch.cat(parts, dim=1), want)

        # (ii) sequences per rank with local block pools: outputs concatenate along the batch
        mine = W.shard_sequences(full, world, rank)
        assert mine.key_cache.shape[0] <= full.key_cache.shape[0]
        assert int(mine.block_tables.max()) < mine.key_cache.shape[0]
        out = _oracle(mine).contiguous()
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)
        ok_seqs = torch.equal(torch.cat(parts, dim=0), want)

        # timing aggregation used by bench.py: max over ranks
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q.put((rank, ok_heads, ok_seqs, float(t)))
    finally:
        dist.destroy_process_group()


def test_two_rank_partitionings_reassemble_the_unsharded_result():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_heads, ok_seqs, tmax in res:
        assert ok_heads, f"rank {rank}: kv-head sharding does not reassemble"
        assert ok_seqs, f"rank {rank}: sequence sharding does not reassemble"
        assert tmax == float(world)
