"""Decode attention with the KV tokens of every sequence partitioned across ranks.

Each rank attends over the tokens it holds and gets, besides its partial output, the
log-sum-exp of its logits (``paged_attention_with_lse``); the partial results of all ranks
are exchanged with one NCCL all-gather each and combined with ``merge_attn_states``.  This
is the arithmetic of the reference's decode context parallelism
(``vllm/attention/ops/common.py:172-205``, ``cp_lse_ag_out_rs``: all-gather of the LSEs,
correction of the outputs) on top of the paged-attention ops, which in the reference
cannot take part in it because they return no LSE.

The query is replicated, the caches are private to each rank.  ALiBi is not supported (the
bias needs the global token position)."""
from __future__ import annotations

import torch

from vllm_b200 import _custom_ops as ops


def local_attention(w, out: torch.Tensor | None = None, lse: torch.Tensor | None = None):
    """Attention of this rank's workload shard; returns (out [S, H, D], lse [H, S] float32)."""
    if out is None:
        out = torch.empty_like(w.query)
    if lse is None:
        lse = torch.empty((w.num_heads, w.num_seqs), dtype=torch.float32, device=w.query.device)
    ops.paged_attention_with_lse(out, lse, w.query, w.key_cache, w.value_cache, w.num_kv_heads,
                                 w.scale, w.block_tables, w.seq_lens, w.block_size, w.max_seq_len,
                                 None, w.kv_cache_dtype, w.k_scale, w.v_scale)
    return out, lse


def merge_partials(outs: list[torch.Tensor], lses: list[torch.Tensor]) -> torch.Tensor:
    """Combines per-rank (out, lse) pairs, left to right, with merge_attn_states."""
    acc_out, acc_lse = outs[0], lses[0]
    for o, l in zip(outs[1:], lses[1:]):
        new_out = torch.empty_like(acc_out)
        new_lse = torch.empty_like(acc_lse)
        ops.merge_attn_states(new_out, acc_out, acc_lse, o, l, new_lse)
        acc_out, acc_lse = new_out, new_lse
    return acc_out


def decode(w, group=None) -> torch.Tensor:
    """Full attention output on every rank of `group` (default: the world group); `w` is this
    rank's token shard.  Two all-gathers (outputs, LSEs), then world_size - 1 merges."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    out, lse = local_attention(w)
    outs = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=out.device)
    lses = torch.empty((world,) + tuple(lse.shape), dtype=lse.dtype, device=lse.device)
    dist.all_gather_into_tensor(outs, out.contiguous(), group=group)
    dist.all_gather_into_tensor(lses, lse, group=group)
    return merge_partials(list(outs.unbind(0)), list(lses.unbind(0)))
