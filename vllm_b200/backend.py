"""A V1-style attention backend that drives the B200 paged-attention ops.

Shape of the classes follows the reference's paged-attention backend for its
x-layout cache (``vllm/v1/attention/backends/rocm_attn.py:153-362``): a backend
class with the static queries the engine makes (name, impl class, KV-cache shape,
metadata builder), per-step metadata, and an ``Impl.forward`` that first writes
the step's new K/V into the paged cache (``PagedAttention.write_to_paged_cache``)
and then attends.  The classes are duck-typed to
``vllm/attention/backends/abstract.py:41,257,303`` and do not import vLLM, so the
module also works stand-alone; inside vLLM it is registered with::

    from vllm.attention.backends.registry import register_backend, AttentionBackendEnum
    register_backend(AttentionBackendEnum.CUSTOM, "vllm_b200.backend.B200PagedAttentionBackend")

Decode steps (one query token per sequence) go straight to
``PagedAttention.forward_decode``.  Steps that contain prefill or chunked-prefill
tokens are served by the same decode kernels: after the KV write every query
token is presented as its own single-token "sequence" that shares its request's
block-table row and sees the cache up to its own position (causal).  That reads
the cache once per query token - fine for short prompts and for correctness; a
dedicated prefill kernel is outside this path.
"""
from __future__ import annotations

import dataclasses

import torch

from vllm_b200.paged_attn import PagedAttention


@dataclasses.dataclass
class B200PagedAttentionMetadata:
    """Per-step metadata, the fields the reference's builders provide
    (``vllm/v1/attention/backends/utils.py`` CommonAttentionMetadata)."""

    num_actual_tokens: int          # query tokens in this step (excluding padding)
    max_query_len: int              # longest query of the step (1 = pure decode)
    query_start_loc: torch.Tensor   # [num_reqs + 1] int32, token offsets of each request
    max_seq_len: int                # longest sequence including this step's tokens
    seq_lens: torch.Tensor          # [num_reqs] int32, sequence lengths including this step
    block_table: torch.Tensor       # [num_reqs, max_blocks] int32
    slot_mapping: torch.Tensor      # [num_tokens] int64, cache slot of every new token
    use_cascade: bool = False


def expand_to_token_sequences(query_start_loc: torch.Tensor, seq_lens: torch.Tensor,
                              block_table: torch.Tensor, num_tokens: int):
    """Maps a step with multi-token queries onto single-token "sequences".

    Query token t of request r (the i-th of its q_r tokens this step) attends to
    the first ``seq_len_r - q_r + i + 1`` cached tokens.  Returns
    ``(token_seq_lens [num_tokens] int32, token_block_table [num_tokens, max_blocks])``.
    """
    qsl = query_start_loc.to(torch.int64)
    q_lens = qsl[1:] - qsl[:-1]
    req_of_token = torch.repeat_interleave(
        torch.arange(q_lens.numel(), device=qsl.device), q_lens, output_size=num_tokens)
    pos_in_query = torch.arange(num_tokens, device=qsl.device) - qsl[req_of_token]
    ctx = seq_lens.to(torch.int64)[req_of_token] - q_lens[req_of_token] + pos_in_query + 1
    return ctx.to(torch.int32), block_table.index_select(0, req_of_token)


class B200PagedAttentionMetadataBuilder:
    """Builds ``B200PagedAttentionMetadata`` from the engine's per-step
    ``CommonAttentionMetadata``.  Same constructor and ``build`` signature as the
    reference's builders (``AttentionMetadataBuilder``,
    ``vllm/v1/attention/backends/utils.py:245-330``; ``RocmAttentionMetadataBuilder``,
    ``rocm_attn.py:65-150``), so the engine can construct and call it unchanged.  The
    arguments are read by attribute only: any object with the fields of
    ``CommonAttentionMetadata`` (``utils.py:53-95``) does.
    """

    # the ops neither allocate nor synchronise, so decode steps may be captured in full graphs
    # (the reference spells this AttentionCGSupport.ALWAYS; the name is kept as a string so that
    # this module does not have to import vLLM)
    _cudagraph_support = "ALWAYS"
    reorder_batch_threshold = None

    def __init__(self, kv_cache_spec, layer_names=None, vllm_config=None, device=None):
        # `kv_cache_spec` is the engine's AttentionSpec (block_size attribute); a bare block
        # size is accepted for stand-alone use
        self.kv_cache_spec = kv_cache_spec
        self.layer_names = list(layer_names) if layer_names is not None else []
        self.vllm_config = vllm_config
        self.device = device
        self.block_size = int(getattr(kv_cache_spec, "block_size", kv_cache_spec))

    @classmethod
    def get_cudagraph_support(cls, vllm_config=None, kv_cache_spec=None):
        return cls._cudagraph_support

    def build(self, common_prefix_len: int, common_attn_metadata,
              fast_build: bool = False) -> B200PagedAttentionMetadata:
        if common_prefix_len > 0:
            raise NotImplementedError("cascade attention is not supported by the paged-attention ops "
                                      "(use_cascade_attention() returns False)")
        m = common_attn_metadata
        return B200PagedAttentionMetadata(
            num_actual_tokens=m.num_actual_tokens, max_query_len=m.max_query_len,
            query_start_loc=m.query_start_loc, max_seq_len=m.max_seq_len, seq_lens=m.seq_lens,
            block_table=m.block_table_tensor, slot_mapping=m.slot_mapping)

    def build_for_cudagraph_capture(self, common_attn_metadata) -> B200PagedAttentionMetadata:
        """Metadata for a capture run: real shapes, every sequence one token long so that the
        captured launch is cheap (rocm_attn.py:84-99 does the same)."""
        md = self.build(0, common_attn_metadata)
        md.seq_lens.fill_(1)
        return md


class B200PagedAttentionImpl:
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 alibi_slopes: list[float] | None = None, sliding_window: int | None = None,
                 kv_cache_dtype: str = "auto", logits_soft_cap: float | None = None,
                 attn_type: str = "decoder", kv_sharing_target_layer_name: str | None = None,
                 sinks: torch.Tensor | None = None) -> None:
        B200PagedAttentionBackend.validate_head_size(head_size)
        if sliding_window is not None:
            raise NotImplementedError("sliding window is not supported by the paged-attention ops")
        if logits_soft_cap:
            raise NotImplementedError("logits soft cap is not supported by the paged-attention ops")
        if sinks is not None:
            raise NotImplementedError("attention sinks are not supported by the paged-attention ops")
        if attn_type != "decoder":
            raise NotImplementedError("only decoder self-attention is implemented")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        self.alibi_slopes = (None if alibi_slopes is None
                             else torch.tensor(alibi_slopes, dtype=torch.float32))
        self.kv_cache_dtype = kv_cache_dtype
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
        self.num_queries_per_kv = num_heads // num_kv_heads

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                kv_cache: torch.Tensor, attn_metadata: B200PagedAttentionMetadata | None,
                output: torch.Tensor | None = None, output_scale=None,
                output_block_scale=None) -> torch.Tensor:
        """query [num_tokens, num_heads, head_size]; key/value [num_tokens, num_kv_heads,
        head_size]; kv_cache [2, num_blocks, block_size * num_kv_heads * head_size];
        `layer` carries `_k_scale` / `_v_scale` float32 tensors.  Returns `output`."""
        assert output is not None, "Output tensor must be provided."
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not supported")
        if attn_metadata is None:  # profiling run
            return output.fill_(0)
        assert attn_metadata.use_cascade is False
        n = attn_metadata.num_actual_tokens
        key_cache, value_cache = PagedAttention.split_kv_cache(kv_cache, self.num_kv_heads,
                                                               self.head_size)
        if self.kv_sharing_target_layer_name is None:
            PagedAttention.write_to_paged_cache(key[:n], value[:n], key_cache, value_cache,
                                                attn_metadata.slot_mapping[:n], self.kv_cache_dtype,
                                                layer._k_scale, layer._v_scale)
        alibi = self.alibi_slopes
        if alibi is not None and alibi.device != query.device:
            alibi = self.alibi_slopes = alibi.to(query.device)
        q = query[:n].view(n, self.num_heads, self.head_size)
        if attn_metadata.max_query_len == 1:
            seq_lens, block_table = attn_metadata.seq_lens, attn_metadata.block_table
        else:
            seq_lens, block_table = expand_to_token_sequences(
                attn_metadata.query_start_loc, attn_metadata.seq_lens, attn_metadata.block_table, n)
        out = PagedAttention.forward_decode(
            q, key_cache, value_cache, block_table, seq_lens, attn_metadata.max_seq_len,
            self.kv_cache_dtype, self.num_kv_heads, self.scale, alibi, layer._k_scale,
            layer._v_scale)
        output[:n].view(n, self.num_heads, self.head_size).copy_(out)
        return output


class B200PagedAttentionBackend:
    accept_output_buffer: bool = True
    supported_dtypes = [torch.float16, torch.bfloat16, torch.float32]

    @classmethod
    def get_supported_head_sizes(cls) -> list[int]:
        return PagedAttention.get_supported_head_sizes()

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size in cls.get_supported_head_sizes()

    @classmethod
    def validate_head_size(cls, head_size: int) -> None:
        if not cls.supports_head_size(head_size):
            raise ValueError(f"Head size {head_size} is not supported by B200PagedAttention. "
                             f"Supported head sizes are: {cls.get_supported_head_sizes()}.")

    @staticmethod
    def get_name() -> str:
        return "B200_PAGED_ATTN"

    @staticmethod
    def get_impl_cls() -> type[B200PagedAttentionImpl]:
        return B200PagedAttentionImpl

    @staticmethod
    def get_builder_cls() -> type[B200PagedAttentionMetadataBuilder]:
        return B200PagedAttentionMetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if block_size not in (8, 16, 32):
            raise ValueError("Block size must be 8, 16 or 32.")
        return PagedAttention.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size,
                                                 cache_dtype_str)

    @staticmethod
    def use_cascade_attention(*args, **kwargs) -> bool:
        return False
