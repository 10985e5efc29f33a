"""The optional log-sum-exp output of the attention entry points and what it is for:
combining attention over disjoint token ranges of a sequence with merge_attn_states."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200 import _custom_ops as ops
from vllm_b200 import capi, context_parallel
import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _oracle(w):
    return O.paged_attention(w.query.cpu(), w.key_cache.cpu(), w.value_cache.cpu(), w.num_kv_heads,
                             w.scale, w.block_tables.cpu(), w.seq_lens.cpu(), None, w.kv_cache_dtype,
                             float(w.k_scale), float(w.v_scale), mode="f64", return_lse=True)


def _check(w, out, lse):
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    want_out, want_lse = _oracle(w)
    tol = 2e-2 if w.kv_cache_dtype != "auto" else 1e-2
    torch.testing.assert_close(out.cpu().double(), want_out, atol=tol, rtol=tol)
    got = lse.cpu().double()
    empty = torch.isinf(want_lse)
    assert torch.equal(torch.isinf(got) & (got < 0), empty)
    # the logits come from 16-bit products accumulated in fp32: a few 1e-3 at most
    torch.testing.assert_close(got[~empty], want_lse[~empty], atol=5e-3, rtol=1e-4)


@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("case", [
    (8, 2, 128, [0, 1, 17, 300, 513, 2500, 64, 4000]),   # direct writes and merged partitions
    (16, 1, 256, [3000, 5]),                              # two n-tiles per item
    (4, 4, 120, [700, 40]),                               # generic kernel
    (1, 1, 64, [4096]),                                   # 64 fine partitions of one head
])
def test_lse_matches_oracle(kv, case):
    hq, hkv, d, lens = case
    if kv == "fp8" and d % 16:
        pytest.skip("an fp8 cache packs 16 elements per chunk")
    rng = np.random.default_rng(3)
    w = W.make_decode("lse", num_seqs=len(lens), num_heads=hq, num_kv_heads=hkv, head_size=d,
                      block_size=16, lens=np.array(lens), dtype=torch.bfloat16, kv_cache_dtype=kv,
                      device=DEV, seed=3, rng=rng)
    w.query.mul_(6.0)
    out, lse = context_parallel.local_attention(w)
    _check(w, out, lse)


@pytest.mark.parametrize("head_size", [128, 120])
def test_lse_through_the_c_abi_v2_entry(head_size):
    """v2 with the caller's scratch (head size 120: generic kernel + separate reduce kernel)."""
    rng = np.random.default_rng(4)
    lens = np.array([1500, 3, 513, 0, 2049])
    w = W.make_decode("lse2", num_seqs=len(lens), num_heads=8, num_kv_heads=2, head_size=head_size,
                      block_size=16, lens=lens, dtype=torch.bfloat16, kv_cache_dtype="auto", device=DEV,
                      seed=4, rng=rng)
    out = torch.empty_like(w.query)
    lse = torch.full((w.num_heads, w.num_seqs), 7.0, dtype=torch.float32, device=DEV)
    e, m, t = w.scratch()
    a = capi.AttnArgs()
    a.out, a.query, a.key_cache, a.value_cache = (out.data_ptr(), w.query.data_ptr(),
                                                  w.key_cache.data_ptr(), w.value_cache.data_ptr())
    a.block_tables, a.seq_lens = w.block_tables.data_ptr(), w.seq_lens.data_ptr()
    a.exp_sums, a.max_logits, a.tmp_out = e.data_ptr(), m.data_ptr(), t.data_ptr()
    a.out_lse = lse.data_ptr()
    a.q_stride = w.query.stride(0)
    a.kv_block_stride, a.kv_head_stride = w.key_cache.stride(0), w.key_cache.stride(1)
    a.num_seqs, a.num_heads, a.num_kv_heads, a.head_size = w.num_seqs, w.num_heads, w.num_kv_heads, head_size
    a.block_size, a.max_seq_len = w.block_size, w.max_seq_len
    a.max_num_blocks_per_seq, a.max_num_partitions = w.block_tables.shape[1], e.shape[2]
    a.scale, a.q_dtype, a.kv_dtype = w.scale, capi.BF16, capi.KV_AUTO
    a.blocksparse_block_size = 64
    capi.paged_attention_v2(a, torch.cuda.current_stream().cuda_stream)
    _check(w, out, lse)


@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("world", [2, 3])
def test_token_shards_merge_to_full_attention(kv, world):
    """Every sequence's tokens cut into `world` block-aligned ranges (one per would-be rank),
    attended separately and merged: equals attention over the whole sequence."""
    rng = np.random.default_rng(8)
    lens = np.array([2500, 1, 16, 17, 700, 4096, 33])
    w = W.make_decode("cp", num_seqs=len(lens), num_heads=16, num_kv_heads=4, head_size=128,
                      block_size=16, lens=lens, dtype=torch.bfloat16, kv_cache_dtype=kv, device=DEV,
                      seed=8, rng=rng)
    w.query.mul_(6.0)
    full = W.run_attention(w, version="v2")
    parts = [context_parallel.local_attention(W.shard_tokens(w, world, r)) for r in range(world)]
    got = context_parallel.merge_partials([p[0] for p in parts], [p[1] for p in parts])
    torch.testing.assert_close(got.float(), full.float(), atol=1e-2, rtol=1e-2)
    want, _ = _oracle(w)
    tol = 2e-2 if kv != "auto" else 1e-2
    torch.testing.assert_close(got.cpu().double(), want, atol=tol, rtol=tol)
