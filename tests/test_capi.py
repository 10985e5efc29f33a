"""The C-ABI library loads, exports every symbol that include/b200pa.h declares,
and validates its arguments before any CUDA call (no GPU needed)."""
import ctypes as C
import re
from pathlib import Path

import pytest

from vllm_b200 import capi

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "b200pa.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200pa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    names = _declared()
    assert set(capi.EXPORTS) <= set(names)
    lib = capi.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200pa.h but not exported by libb200pa.so"


def test_struct_sizes_match_header_layout():
    # 12 pointers + 3 int64 + 8 int32 + float + 2 int32 + 5 int32 + out_lse = 96+24+64+8 = 192
    assert C.sizeof(capi.AttnArgs) == 12 * 8 + 3 * 8 + 16 * 4 + 8
    assert capi.AttnArgs.out_lse.offset == 184
    assert C.sizeof(capi.CacheArgs) == 7 * 8 + 5 * 8 + 7 * 4 + 4  # tail padding to 8


def test_version_and_kv_dtype_strings():
    assert capi.lib().b200pa_version() == 2
    assert capi.kv_dtype_from_string("auto") == capi.KV_AUTO
    for s in ("fp8", "fp8_e4m3", "fp8_ds_mla"):
        assert capi.kv_dtype_from_string(s) == capi.KV_FP8_E4M3
    assert capi.kv_dtype_from_string("fp8_e5m2") == capi.KV_FP8_E5M2
    assert capi.kv_dtype_from_string("int4") == -1


def _attn(**kw):
    a = capi.AttnArgs()
    a.num_seqs, a.num_heads, a.num_kv_heads, a.head_size = 4, 8, 2, 128
    a.block_size, a.max_seq_len, a.max_num_blocks_per_seq, a.max_num_partitions = 16, 100, 7, 1
    a.q_dtype, a.kv_dtype, a.scale = capi.BF16, capi.KV_AUTO, 0.088
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw,msg", [
    (dict(head_size=48), "Unsupported head size"),
    (dict(block_size=64), "Unsupported block size"),
    (dict(q_dtype=7), "Unsupported input type"),
    (dict(kv_dtype=9), "Unsupported data type of kv cache"),
    (dict(num_heads=7), "not a multiple"),
    # an fp8 cache keeps 16 head dimensions together (x = 16): head size 120 cannot exist in it
    (dict(head_size=120, kv_dtype=capi.KV_FP8_E4M3), "not a multiple of x = 16"),
    (dict(head_size=120, kv_dtype=capi.KV_FP8_E5M2), "not a multiple of x = 16"),
    (dict(blocksparse_vert_stride=2, blocksparse_block_size=24), "blocksparse_block_size"),
    (dict(), "null tensor pointer"),
])
def test_attention_argument_errors_are_reported_not_thrown(kw, msg):
    lib = capi.lib()
    rc = lib.b200pa_paged_attention_v1(C.byref(_attn(**kw)), None)
    assert rc < 0
    assert msg in capi.last_error()
    with pytest.raises(RuntimeError, match=msg):
        capi.paged_attention_v2(_attn(**kw))


def test_null_args_and_empty_batches():
    lib = capi.lib()
    assert lib.b200pa_paged_attention_v1(None, None) == -1
    assert lib.b200pa_reshape_and_cache(None, None) == -1
    # an empty batch / zero tokens is a successful no-op, with no pointer needed
    assert lib.b200pa_paged_attention_v1(C.byref(_attn(num_seqs=0)), None) == 0
    c = capi.CacheArgs()
    c.num_tokens, c.num_heads, c.head_size, c.block_size, c.x = 0, 8, 128, 16, 8
    assert lib.b200pa_reshape_and_cache(C.byref(c), None) == 0
    assert lib.b200pa_reshape_and_cache_flash(C.byref(c), None) == 0
    c.num_tokens = 3
    assert lib.b200pa_reshape_and_cache(C.byref(c), None) == -1
    assert "null tensor pointer" in capi.last_error()
    assert lib.b200pa_convert_fp8(None, None, 0, 1.0, capi.BF16, capi.KV_FP8_E4M3, 1, None) == 0
    assert lib.b200pa_convert_fp8(None, None, 5, 1.0, capi.BF16, capi.KV_FP8_E4M3, 1, None) == -1
