"""torch.library.opcheck on the registered ops, as the reference's kernel tests do
(tests/kernels/utils.py:1062-1080 with the checks of :33-38)."""
import pytest
import torch

from vllm_b200 import _custom_ops
import workloads as W

pytestmark = pytest.mark.gpu
_custom_ops.claim_reference_names()  # the checks below address the ops by the reference's names
CHECKS = ("test_schema", "test_autograd_registration", "test_faketensor")


def _opcheck(op, args):
    torch.library.opcheck(op, args, test_utils=CHECKS, raise_exception=True)


def test_opcheck_attention_ops():
    w = W.small("cuda", seed=40, num_seqs=3, num_heads=8, num_kv_heads=2, max_len=700, num_blocks=128)
    out = torch.empty_like(w.query)
    tail = (w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale, w.block_tables, w.seq_lens,
            w.block_size, w.max_seq_len, None, "auto", w.k_scale, w.v_scale, 0, 0, 0, 64, 0)
    _opcheck(torch.ops._C.paged_attention_v1, (out,) + tail)
    e, m, t = w.scratch()
    _opcheck(torch.ops._C.paged_attention_v2, (out, e, m, t) + tail)


def test_opcheck_cache_ops():
    T, H, D, B, NB = 20, 4, 64, 16, 8
    key = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    val = torch.randn_like(key)
    slots = torch.randperm(NB * B, device="cuda")[:T]
    one = torch.tensor(1.0, device="cuda")
    kc = torch.zeros(NB, H, D // 8, B, 8, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros(NB, H, D, B, device="cuda", dtype=torch.bfloat16)
    _opcheck(torch.ops._C_cache_ops.reshape_and_cache, (key, val, kc, vc, slots, "auto", one, one))
    kf = torch.zeros(NB, B, H, D, device="cuda", dtype=torch.bfloat16)
    vf = torch.zeros_like(kf)
    _opcheck(torch.ops._C_cache_ops.reshape_and_cache_flash, (key, val, kf, vf, slots, "auto", one, one))
    q8 = torch.empty(T, H, D, device="cuda", dtype=torch.uint8)
    _opcheck(torch.ops._C_cache_ops.convert_fp8, (q8, key, 1.0, "fp8"))
