"""vLLM plugin entry point: makes an installed vLLM call the B200 kernels.

vLLM loads every entry point of the group ``vllm.general_plugins`` in each of its processes
and calls it (``vllm/plugins/__init__.py:25-78`` of the reference).  Declare

    [project.entry-points."vllm.general_plugins"]
    b200pa = "vllm_b200.plugin:register"

in the packaging metadata of this package, or call ``register()`` by hand before the engine
starts.  ``register()`` may run more than once per process (the loader says plugins must
tolerate that) and is idempotent.

What it does
------------
* Re-points the wrappers in ``vllm._custom_ops`` that belong to this path
  (``paged_attention_v1/v2``, ``reshape_and_cache``, ``reshape_and_cache_flash``,
  ``convert_fp8``, ``merge_attn_states``, ``copy_blocks``, ``swap_blocks``;
  ``vllm/_custom_ops.py:29-120, 2121-2199``) at the functions of the same name and signature in
  ``vllm_b200._custom_ops``.  Those dispatch to ``torch.ops._C_b200.*``, which this package
  always registers, so it does not matter whether vLLM's own ``_C`` extension has been loaded
  before or after (both namespaces can live side by side).
* Registers ``vllm_b200.backend.B200PagedAttentionBackend`` as the ``CUSTOM`` attention backend
  (``vllm/attention/backends/registry.py:124-163``) when that registry can be imported.
"""
from __future__ import annotations

import importlib

OPS = ("paged_attention_v1", "paged_attention_v2", "reshape_and_cache", "reshape_and_cache_flash",
       "convert_fp8", "merge_attn_states", "copy_blocks", "swap_blocks")

BACKEND = "vllm_b200.backend.B200PagedAttentionBackend"


def register(custom_ops_module: str = "vllm._custom_ops",
             registry_module: str = "vllm.attention.backends.registry") -> dict:
    """Patches the op wrappers and registers the backend.  Returns what was done:
    ``{"ops": [names re-pointed], "backend": bool}``."""
    from vllm_b200 import _custom_ops as b200  # raises if the native libraries are missing

    done = {"ops": [], "backend": False}
    ref = importlib.import_module(custom_ops_module)
    for name in OPS:
        if not hasattr(b200, name):
            continue
        fn = getattr(b200, name)
        if getattr(ref, name, None) is not fn:
            if not hasattr(ref, "_b200_replaced"):
                ref._b200_replaced = {}
            ref._b200_replaced.setdefault(name, getattr(ref, name, None))
            setattr(ref, name, fn)
        done["ops"].append(name)
    try:
        reg = importlib.import_module(registry_module)
    except ImportError:
        return done
    reg.register_backend(reg.AttentionBackendEnum.CUSTOM, BACKEND)
    done["backend"] = True
    return done


def unregister(custom_ops_module: str = "vllm._custom_ops") -> None:
    """Puts the original wrappers back (tests, A/B comparisons)."""
    ref = importlib.import_module(custom_ops_module)
    for name, fn in getattr(ref, "_b200_replaced", {}).items():
        if fn is None:
            delattr(ref, name)
        else:
            setattr(ref, name, fn)
    ref._b200_replaced = {}
