"""CUDA-graph capture of the ops (the reference captures them in its decode graphs,
benchmarks/kernels/benchmark_reshape_and_cache.py:83-88) and the multi-GPU verification path:
outputs of head-, sequence- or token-sharded ranks, all-gathered over NCCL (and, for token
shards, merged through their log-sum-exps), equal the unsharded result."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

from vllm_b200 import _custom_ops as ops
import workloads as W

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_ops_capture_into_a_cuda_graph_and_replay():
    dev = "cuda"
    w = W.config3(dev, num_seqs=6, seq_len=2048, new_tokens=16)
    scratch = w.scratch()
    out = torch.empty_like(w.query)

    def decode_step():
        ops.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping,
                              "fp8", w.k_scale, w.v_scale)
        W.run_attention(w, out=out, version="v2", scratch=scratch)
        W.run_attention(w, out=out1, version="v1")

    out1 = torch.empty_like(w.query)
    # warm-up outside capture (first calls resolve device symbols and opt in to large shared memory)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        decode_step()
    torch.cuda.current_stream().wait_stream(s)
    want2, want1 = out.clone(), out1.clone()
    kc_want = w.key_cache.clone()

    B = w.block_size
    blk, off = w.slot_mapping // B, w.slot_mapping % B
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        decode_step()
    for _ in range(3):
        out.zero_()
        out1.zero_()
        w.key_cache[blk, :, :, off, :] = 0  # the replayed write must restore the new tokens
        w.value_cache[blk, :, :, off] = 0
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(w.key_cache, kc_want)
    assert torch.equal(out, want2)
    assert torch.equal(out1, want1)


def _free_port():
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        return sck.getsockname()[1]


def _rank_main(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import workloads as Wl
        full = Wl.small(dev, seed=51, num_seqs=8, num_heads=32, num_kv_heads=8, max_len=2500, num_blocks=2048)
        full.query.mul_(10.0)
        want = Wl.run_attention(full, version="v2")
        ok = []
        for shard, dim in ((Wl.shard_kv_heads, 1), (Wl.shard_sequences, 0)):
            mine = shard(full, world, rank)
            out = Wl.run_attention(mine, version="v2").contiguous()
            if dim == 1:
                # all_gather_into_tensor concatenates along dim 0: gather [W, S, H/W, D] and fold
                buf = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
                dist.all_gather_into_tensor(buf, out)
                got = buf.permute(1, 0, 2, 3).reshape(want.shape)
            else:
                got = torch.empty_like(want)
                dist.all_gather_into_tensor(got, out)
            # a shard is cut into different pieces than the whole problem (the kernel balances
            # cache blocks per warp), so the partial sums round differently: close, not equal
            ok.append(bool(torch.allclose(got.float(), want.float(), atol=2e-3, rtol=1e-2)))
        # tokens of every sequence per rank: partial outputs + log-sum-exps, two all-gathers, merge
        from vllm_b200 import context_parallel
        got = context_parallel.decode(Wl.shard_tokens(full, world, rank))
        ok.append(bool(torch.allclose(got.float(), want.float(), atol=1e-2, rtol=1e-2)))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_sharded_ranks_reassemble_over_nccl():
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok in res:
        assert ok == [True, True, True], f"rank {rank}: kv-head / sequence / token sharding mismatch {ok}"
