"""b200pa_paged_attention_v2_noalloc: the split-KV decode for callers that have no
device memory to lend (a bare C host without an allocator; a server whose HBM is
already committed to the KV pool).  It must produce the oracle's result - and what
b200pa_paged_attention_v2 produces with caller-owned scratch - call after call,
although every call reuses the same built-in buffer and finds the previous call's
partials in it.

Collected last on purpose (file name), so a failure here cannot hide other tests
from a run that stops at the first failure.  Both entry points are called through
the C ABI with raw device pointers.
"""
import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200 import capi
import workloads as W

DEV = "cuda"


def _args(w, out, scratch=None):
    a = capi.AttnArgs()
    a.out, a.query = out.data_ptr(), w.query.data_ptr()
    a.key_cache, a.value_cache = w.key_cache.data_ptr(), w.value_cache.data_ptr()
    a.block_tables, a.seq_lens = w.block_tables.data_ptr(), w.seq_lens.data_ptr()
    a.k_scale, a.v_scale = w.k_scale.data_ptr(), w.v_scale.data_ptr()
    a.q_stride = w.query.stride(0)
    a.kv_block_stride, a.kv_head_stride = w.key_cache.stride(0), w.key_cache.stride(1)
    a.num_seqs, a.num_heads, a.head_size = w.query.shape
    a.num_kv_heads, a.block_size, a.max_seq_len = w.num_kv_heads, w.block_size, w.max_seq_len
    a.max_num_blocks_per_seq = w.block_tables.shape[1]
    a.scale = w.scale
    a.q_dtype = {torch.bfloat16: capi.BF16, torch.float16: capi.F16, torch.float32: capi.F32}[w.query.dtype]
    a.kv_dtype = capi.kv_dtype_from_string(w.kv_cache_dtype)
    if scratch is not None:
        e, m, t = scratch
        a.exp_sums, a.max_logits, a.tmp_out = e.data_ptr(), m.data_ptr(), t.data_ptr()
        a.max_num_partitions = e.shape[2]
    return a


def _oracle(w, seqs):
    """float64 oracle on the sequences `seqs`, with only their cache blocks brought to the host."""
    idx = torch.tensor(seqs, device=DEV)
    lens = w.seq_lens[idx].cpu()
    need = max(1, int(np.ceil(lens.numpy() / w.block_size).max()))
    bt = w.block_tables[idx, :need].cpu()
    uniq, inv = torch.unique(bt.flatten(), return_inverse=True)
    kc = w.key_cache[uniq.to(DEV).long()].cpu()
    vc = w.value_cache[uniq.to(DEV).long()].cpu()
    return O.paged_attention(w.query[idx].cpu(), kc, vc, w.num_kv_heads, w.scale,
                             inv.view(bt.shape).int(), lens, None, w.kv_cache_dtype,
                             float(w.k_scale), float(w.v_scale), mode="f64")


@pytest.mark.gpu
def test_noalloc_matches_the_oracle_on_consecutive_calls():
    stream = torch.cuda.current_stream().cuda_stream
    # Different batches back to back: each finds the previous one's partials in the shared
    # array and must not be affected by them.  Every case keeps its partials in the built-in
    # array (this entry point uses nothing else): a small bf16 batch (many slots per sequence),
    # an fp8 one with block size 32, an fp32 one (generic kernel + separate reduce kernel, 4-byte
    # partials) and a batch of 256 sequences whose partials fill a third of the array.
    cases = [
        W.small(DEV, seed=31, num_seqs=12, num_heads=32, num_kv_heads=8, max_len=2300, num_blocks=2048),
        W.small(DEV, seed=32, num_seqs=9, num_heads=64, num_kv_heads=8, block_size=32, max_len=1700,
                kv_cache_dtype="fp8", num_blocks=700),
        W.small(DEV, seed=34, num_seqs=5, num_heads=8, num_kv_heads=2, max_len=1900, dtype=torch.float32,
                num_blocks=700),
        W.small(DEV, seed=35, num_seqs=256, num_heads=32, num_kv_heads=8, max_len=2300, num_blocks=40000),
    ]
    for rounds in range(2):
        for w in cases:
            if rounds == 0:
                w.query.mul_(8.0)
            got = torch.full_like(w.query, float("nan"))
            capi.paged_attention_v2_noalloc(_args(w, got), stream)
            torch.cuda.synchronize()
            assert capi.device_status() == 0
            assert torch.isfinite(got.float()).all()
            tol = 2e-2 if w.kv_cache_dtype != "auto" else 1e-2
            seqs = list(range(w.num_seqs)) if w.num_seqs <= 16 else [0, 1, 100, 254, 255]
            want = _oracle(w, seqs)
            torch.testing.assert_close(got[torch.tensor(seqs, device=DEV)].cpu().double(), want,
                                       atol=tol, rtol=tol)
            # and, on every sequence, what v2 gives with scratch that the caller owns
            ref = torch.empty_like(w.query)
            capi.paged_attention_v2(_args(w, ref, w.scratch()), stream)
            torch.testing.assert_close(got.float(), ref.float(), atol=tol, rtol=tol)


@pytest.mark.gpu
def test_noalloc_rejects_problems_beyond_the_built_in_buffer():
    w = W.small(DEV, seed=33, num_seqs=4, num_heads=8, num_kv_heads=2, max_len=600, num_blocks=256)
    out = torch.zeros_like(w.query)
    a = _args(w, out)
    # 4096 sequences x 64 heads x 64 partitions of 128-wide bf16 partials is ~4.4 GB of scratch
    a.num_seqs, a.num_heads, a.num_kv_heads, a.max_seq_len = 4096, 64, 8, 32768
    with pytest.raises(RuntimeError, match="built-in buffer holds"):
        capi.paged_attention_v2_noalloc(a, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.count_nonzero(out) == 0  # nothing was launched
