"""Operator wrappers with the reference's names, argument order and error behaviour.

Mirror of ``vllm/_custom_ops.py:29-120`` (``paged_attention_v1/v2``) and
``:2121-2199`` (``reshape_and_cache``, ``reshape_and_cache_flash``,
``convert_fp8``) of the reference.  Each function is a pass-through to a torch
custom op whose CUDA implementation lives in ``libb200pa.so``; loading this
module loads the native libraries and raises if they are missing.
"""
from __future__ import annotations

from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_SHIM = _PKG / "_C_b200.so"


def _load() -> None:
    if not _SHIM.exists() or not (_PKG / "libb200pa.so").exists():
        raise RuntimeError(
            f"native libraries are missing under {_PKG}: run `python -m vllm_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)")
    torch.ops.load_library(str(_SHIM))


_load()

# Always-present private namespaces.
_ops = torch.ops._C_b200
_cache_ops = torch.ops._C_b200_cache_ops


def claim_reference_names() -> int:
    """Registers the kernels under the reference's own operator names as well
    (``torch.ops._C.paged_attention_v1/v2``, ``merge_attn_states``,
    ``torch.ops._C_cache_ops.reshape_and_cache/_flash``, ``convert_fp8``, ``copy_blocks``,
    ``swap_blocks``), for code written against ``torch.ops._C`` that runs WITHOUT vLLM's own
    extension - the reference's kernel tests and benchmarks, for instance.

    Not done at import time on purpose: had this package defined those names first, importing
    ``vllm._C`` afterwards would fail on the duplicate definitions.  Names that another
    library has defined already are left to it; beside an installed vLLM use
    ``vllm_b200.plugin.register()`` instead.  Returns the number of names claimed by this call
    (0 when called again).
    """
    import ctypes

    fn = ctypes.CDLL(str(_SHIM)).b200_claim_reference_names
    fn.argtypes = [ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_int
    buf = ctypes.create_string_buffer(1024)
    n = fn(buf, len(buf))
    if n < 0:
        raise RuntimeError("could not register the reference operator names: " + buf.value.decode())
    return n


def paged_attention_v1(
    out: torch.Tensor,
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    num_kv_heads: int,
    scale: float,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    block_size: int,
    max_seq_len: int,
    alibi_slopes: torch.Tensor | None,
    kv_cache_dtype: str,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    tp_rank: int = 0,
    blocksparse_local_blocks: int = 0,
    blocksparse_vert_stride: int = 0,
    blocksparse_block_size: int = 64,
    blocksparse_head_sliding_step: int = 0,
) -> None:
    _ops.paged_attention_v1(
        out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
        block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale, tp_rank,
        blocksparse_local_blocks, blocksparse_vert_stride, blocksparse_block_size,
        blocksparse_head_sliding_step)


def paged_attention_v2(
    out: torch.Tensor,
    exp_sum: torch.Tensor,
    max_logits: torch.Tensor,
    tmp_out: torch.Tensor,
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    num_kv_heads: int,
    scale: float,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    block_size: int,
    max_seq_len: int,
    alibi_slopes: torch.Tensor | None,
    kv_cache_dtype: str,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    tp_rank: int = 0,
    blocksparse_local_blocks: int = 0,
    blocksparse_vert_stride: int = 0,
    blocksparse_block_size: int = 64,
    blocksparse_head_sliding_step: int = 0,
) -> None:
    _ops.paged_attention_v2(
        out, exp_sum, max_logits, tmp_out, query, key_cache, value_cache, num_kv_heads, scale,
        block_tables, seq_lens, block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale,
        v_scale, tp_rank, blocksparse_local_blocks, blocksparse_vert_stride,
        blocksparse_block_size, blocksparse_head_sliding_step)


def reshape_and_cache(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    kv_cache_dtype: str,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
) -> None:
    _cache_ops.reshape_and_cache(
        key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale)


def reshape_and_cache_flash(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    kv_cache_dtype: str,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
) -> None:
    _cache_ops.reshape_and_cache_flash(
        key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale)


def convert_fp8(
    output: torch.Tensor, input: torch.Tensor, scale: float = 1.0, kv_dtype: str = "fp8"
) -> None:
    _cache_ops.convert_fp8(output, input, scale, kv_dtype)


def paged_attention_with_lse(
    out: torch.Tensor,
    lse: torch.Tensor,
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    num_kv_heads: int,
    scale: float,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    block_size: int,
    max_seq_len: int,
    alibi_slopes: torch.Tensor | None,
    kv_cache_dtype: str,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
) -> None:
    """``paged_attention_v1`` that also fills ``lse`` [num_heads, num_seqs] (float32) with the
    natural log-sum-exp of each sequence's scaled logits, in the layout ``merge_attn_states``
    takes.  The reference's paged-attention ops have no such output; its decode context
    parallelism gets the LSE from other backends (vllm/attention/ops/common.py:172-205)."""
    torch.ops._C_b200.paged_attention_with_lse(
        out, lse, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
        block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale)


def merge_attn_states(
    output: torch.Tensor,
    prefix_output: torch.Tensor,
    prefix_lse: torch.Tensor,
    suffix_output: torch.Tensor,
    suffix_lse: torch.Tensor,
    output_lse: torch.Tensor | None = None,
) -> None:
    """Same argument order as the reference wrapper (vllm/_custom_ops.py ``merge_attn_states``)."""
    _ops.merge_attn_states(output, output_lse, prefix_output, prefix_lse, suffix_output, suffix_lse)


def copy_blocks(
    key_caches: list[torch.Tensor],
    value_caches: list[torch.Tensor],
    block_mapping: torch.Tensor,
) -> None:
    _cache_ops.copy_blocks(key_caches, value_caches, block_mapping)


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, block_mapping: torch.Tensor) -> None:
    _cache_ops.swap_blocks(src, dst, block_mapping)
