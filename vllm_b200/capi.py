"""ctypes binding of ``include/b200pa.h`` (the C ABI of ``libb200pa.so``).

The structures below mirror ``b200pa_attn_args`` / ``b200pa_cache_args`` field by
field.  Pointers are raw device addresses (``tensor.data_ptr()``); the caller is
responsible for keeping the tensors alive and for making the owning device
current.  Every wrapper raises ``RuntimeError`` with ``b200pa_last_error()`` when
the library returns a non-zero code.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200pa.so"

F32, F16, BF16 = 0, 1, 2
KV_AUTO, KV_FP8_E4M3, KV_FP8_E5M2 = 0, 1, 2

EXPORTS = (
    "b200pa_kv_dtype_from_string",
    "b200pa_paged_attention_v1",
    "b200pa_paged_attention_v2",
    "b200pa_paged_attention_v2_noalloc",
    "b200pa_reshape_and_cache",
    "b200pa_reshape_and_cache_flash",
    "b200pa_convert_fp8",
    "b200pa_merge_attn_states",
    "b200pa_copy_blocks",
    "b200pa_swap_blocks",
    "b200pa_last_error",
    "b200pa_version",
    "b200pa_device_status",
    "b200pa_launch_count",
)


class AttnArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p), ("query", C.c_void_p), ("key_cache", C.c_void_p),
        ("value_cache", C.c_void_p), ("block_tables", C.c_void_p), ("seq_lens", C.c_void_p),
        ("alibi_slopes", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("exp_sums", C.c_void_p), ("max_logits", C.c_void_p), ("tmp_out", C.c_void_p),
        ("q_stride", C.c_int64), ("kv_block_stride", C.c_int64), ("kv_head_stride", C.c_int64),
        ("num_seqs", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_size", C.c_int32), ("block_size", C.c_int32), ("max_seq_len", C.c_int32),
        ("max_num_blocks_per_seq", C.c_int32), ("max_num_partitions", C.c_int32),
        ("scale", C.c_float), ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32),
        ("tp_rank", C.c_int32), ("blocksparse_local_blocks", C.c_int32),
        ("blocksparse_vert_stride", C.c_int32), ("blocksparse_block_size", C.c_int32),
        ("blocksparse_head_sliding_step", C.c_int32),
        ("out_lse", C.c_void_p),
    ]


class CacheArgs(C.Structure):
    _fields_ = [
        ("key", C.c_void_p), ("value", C.c_void_p), ("key_cache", C.c_void_p),
        ("value_cache", C.c_void_p), ("slot_mapping", C.c_void_p), ("k_scale", C.c_void_p),
        ("v_scale", C.c_void_p),
        ("key_stride", C.c_int64), ("value_stride", C.c_int64), ("block_stride", C.c_int64),
        ("page_stride", C.c_int64), ("head_stride", C.c_int64),
        ("num_tokens", C.c_int32), ("num_heads", C.c_int32), ("head_size", C.c_int32),
        ("block_size", C.c_int32), ("x", C.c_int32), ("in_dtype", C.c_int32),
        ("kv_dtype", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """Loads ``libb200pa.so`` (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vllm_b200.build` "
                "(there is no CPU fallback)")
        l = C.CDLL(str(LIB_PATH))
        l.b200pa_last_error.restype = C.c_char_p
        l.b200pa_kv_dtype_from_string.argtypes = [C.c_char_p]
        l.b200pa_launch_count.restype = C.c_int64
        l.b200pa_launch_count.argtypes = [C.c_int]
        for name in ("b200pa_paged_attention_v1", "b200pa_paged_attention_v2",
                     "b200pa_paged_attention_v2_noalloc"):
            getattr(l, name).argtypes = [C.POINTER(AttnArgs), C.c_void_p]
        for name in ("b200pa_reshape_and_cache", "b200pa_reshape_and_cache_flash"):
            getattr(l, name).argtypes = [C.POINTER(CacheArgs), C.c_void_p]
        l.b200pa_convert_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_void_p]
        l.b200pa_device_status.argtypes = [C.POINTER(C.c_int32)]
        _lib = l
    return _lib


def last_error() -> str:
    return lib().b200pa_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"b200pa error {rc}: {last_error()}")


def kv_dtype_from_string(s: str) -> int:
    return lib().b200pa_kv_dtype_from_string(s.encode())


def paged_attention_v1(args: AttnArgs, stream: int = 0) -> None:
    check(lib().b200pa_paged_attention_v1(C.byref(args), C.c_void_p(stream)))


def paged_attention_v2(args: AttnArgs, stream: int = 0) -> None:
    check(lib().b200pa_paged_attention_v2(C.byref(args), C.c_void_p(stream)))


def paged_attention_v2_noalloc(args: AttnArgs, stream: int = 0) -> None:
    """v2 with the split-KV scratch taken from a 32 MiB array built into the library (allocates
    nothing; limits and sharing rules in b200pa.h)."""
    check(lib().b200pa_paged_attention_v2_noalloc(C.byref(args), C.c_void_p(stream)))


def reshape_and_cache(args: CacheArgs, stream: int = 0) -> None:
    check(lib().b200pa_reshape_and_cache(C.byref(args), C.c_void_p(stream)))


def reshape_and_cache_flash(args: CacheArgs, stream: int = 0) -> None:
    check(lib().b200pa_reshape_and_cache_flash(C.byref(args), C.c_void_p(stream)))


def device_status() -> int:
    v = C.c_int32(0)
    check(lib().b200pa_device_status(C.byref(v)))
    return v.value


def reset_device_state(stream: int = 0) -> None:
    """Zeroes the decode kernel's device-side bookkeeping (see b200pa.h); only needed after a
    launch reported a non-zero device status."""
    check(lib().b200pa_reset_device_state(C.c_void_p(stream)))


def launch_count(reset: bool = False) -> int:
    return int(lib().b200pa_launch_count(1 if reset else 0))
