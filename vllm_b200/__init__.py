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

There is no CPU or PyTorch fallback: every op fails loudly when the native
libraries are missing.
"""

__version__ = "0.1.0"
