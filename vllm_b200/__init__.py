"""B200-native PagedAttention decode path behind the reference's operator surface.

Public modules
--------------
``vllm_b200._custom_ops``  same functions and argument order as the reference's
                           ``vllm/_custom_ops.py`` (``paged_attention_v1``,
                           ``paged_attention_v2``, ``reshape_and_cache``,
                           ``reshape_and_cache_flash``, ``convert_fp8``).
``vllm_b200.paged_attn``   mirror of ``vllm/attention/ops/paged_attn.py``
                           (``PagedAttention`` cache-shape helpers and
                           ``forward_decode``).
``vllm_b200.capi``         ctypes binding of the C ABI declared in
                           ``include/b200pa.h`` (raw device pointers).
``vllm_b200.plugin``       ``register()``: the ``vllm.general_plugins`` entry point that makes
                           an installed vLLM call these kernels.
``vllm_b200.backend``      a V1-style attention backend on top of the ops.

There is no CPU or PyTorch fallback: every op fails loudly when the native
libraries are missing.
"""

__version__ = "0.1.0"


def claim_reference_names() -> int:
    """See ``vllm_b200._custom_ops.claim_reference_names`` (loads the native libraries)."""
    from vllm_b200 import _custom_ops

    return _custom_ops.claim_reference_names()
