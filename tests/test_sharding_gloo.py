"""Multi-rank host logic on CPU (gloo, world_size 2): the partitionings the decode path
supports — KV heads per rank, sequences per rank with local block pools, and the tokens of
every sequence per rank (merged through their log-sum-exps) — reproduce the unsharded result
when the rank outputs are all-gathered.
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
        import workloads as W
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

        # (iii) tokens of every sequence per rank: partial outputs and their log-sum-exps are
        # all-gathered and combined with the merge_attn_states formula
        from oracle import paged_oracle as O
        mine = W.shard_tokens(full, world, rank)
        assert int(mine.seq_lens.sum()) < int(full.seq_lens.sum())
        o, l = O.paged_attention(mine.query, mine.key_cache, mine.value_cache, mine.num_kv_heads,
                                 mine.scale, mine.block_tables, mine.seq_lens, None,
                                 mine.kv_cache_dtype, float(mine.k_scale), float(mine.v_scale),
                                 mode="f64", return_lse=True)
        outs = [torch.empty_like(o) for _ in range(world)]
        lses = [torch.empty_like(l) for _ in range(world)]
        dist.all_gather(outs, o.contiguous())
        dist.all_gather(lses, l.contiguous())
        acc_o, acc_l = outs[0], lses[0]
        for o2, l2 in zip(outs[1:], lses[1:]):
            acc_o, acc_l = O.merge_attn_states(acc_o, acc_l, o2, l2)
        want64 = O.paged_attention(full.query, full.key_cache, full.value_cache, full.num_kv_heads,
                                   full.scale, full.block_tables, full.seq_lens, None,
                                   full.kv_cache_dtype, float(full.k_scale), float(full.v_scale),
                                   mode="f64")
        ok_tokens = bool(torch.allclose(acc_o.double(), want64, atol=1e-5, rtol=1e-5))

        # timing aggregation used by bench.py: max over ranks
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q.put((rank, ok_heads, ok_seqs and ok_tokens, float(t)))
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
