"""Driver for the reference project's CPU decode attention.  TEST / BASELINE ONLY.

Loads ``oracle/_ref/_C_ref_cpu.so`` (the reference's csrc/cpu/cpu_attn.cpp built
unmodified by ``oracle/build_ref.py``) and runs one decode step the way the
reference's CPU backend does (vllm/v1/attention/backends/cpu_attn.py:176-191,
:351; tests/kernels/attention/test_cpu_attn.py:220-270): repack the cache with
``cpu_attn_reshape_and_cache``, build scheduler metadata once, call
``cpu_attention_with_kv_cache``.  The reference has no CPU build of
``paged_attention_v1/v2`` itself; this is its CPU code for the same computation.

Used to pin ``paged_oracle`` (tests/golden/make_cpu_attn_golden.py) and as the
timed CPU baseline of ``bench.py``.  The product never imports this module.
"""
from __future__ import annotations

from pathlib import Path

import torch

SO = Path(__file__).resolve().parent / "_ref" / "_C_ref_cpu.so"
_loaded = False


def available() -> bool:
    return SO.exists()


def load() -> None:
    global _loaded
    if not _loaded:
        if not SO.exists():
            raise RuntimeError(f"{SO} not built (run python oracle/build_ref.py where the reference is mounted)")
        torch.ops.load_library(str(SO))
        _loaded = True


def isa_for(block_size: int) -> str:
    # vec needs block_size % 32 == 0, vec16 needs % 16 (cpu_attn_vec.hpp:125, cpu_attn_vec16.hpp:130)
    return "vec" if block_size % 32 == 0 else "vec16"


def x_layout_to_flash(key_cache: torch.Tensor, value_cache: torch.Tensor):
    """[NB,H,D/x,B,x] / [NB,H,D,B]  ->  logical [NB,B,H,D] tensors (CPU)."""
    nb, h, dx, b, x = key_cache.shape
    k = key_cache.permute(0, 3, 1, 2, 4).reshape(nb, b, h, dx * x).contiguous()
    v = value_cache.permute(0, 3, 1, 2).contiguous()
    return k, v


class RefCpuDecode:
    """Holds the repacked cache and metadata; ``run()`` is the timed part."""

    def __init__(self, query, key_flash, value_flash, block_tables, seq_lens, scale,
                 alibi_slopes=None, kv_split=True):
        load()
        ops = torch.ops._C_ref_cpu
        nb, b, hkv, d = key_flash.shape
        s, hq, _ = query.shape
        self.isa = isa_for(b)
        self.query = query.contiguous()
        self.kc = torch.empty(nb, hkv, b, d, dtype=key_flash.dtype)
        self.vc = torch.empty_like(self.kc)
        slots = torch.arange(0, nb * b, dtype=torch.int64)
        ops.cpu_attn_reshape_and_cache(key_flash.reshape(-1, hkv, d), value_flash.reshape(-1, hkv, d),
                                       self.kc, self.vc, slots, self.isa)
        self.cu = torch.arange(0, s + 1, dtype=torch.int32)
        self.lens = seq_lens.to(torch.int32).contiguous()
        self.bt = block_tables.to(torch.int32).contiguous()
        self.scale = float(scale)
        self.alibi = alibi_slopes
        self.meta = ops.get_scheduler_metadata(s, hq, hkv, d, self.lens, query.dtype, self.cu, True,
                                               -1, self.isa, kv_split)
        self.out = torch.empty_like(self.query)

    def run(self) -> torch.Tensor:
        torch.ops._C_ref_cpu.cpu_attention_with_kv_cache(
            self.query, self.kc, self.vc, self.out, self.cu, self.lens, self.scale, True,
            self.alibi, -1, -1, self.bt, 0.0, self.meta, None)
        return self.out
