"""The attention backend built on the ops: metadata expansion on CPU, and on a GPU a
small prefill + chunked prefill + decode session checked against dense causal attention."""
import types

import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200.backend import (B200PagedAttentionBackend, B200PagedAttentionImpl,
                               B200PagedAttentionMetadataBuilder, expand_to_token_sequences)


def test_expand_to_token_sequences():
    # request 0: 3 new tokens, 10 cached afterwards; request 1: decode, 7 cached; request 2: 2 new of 2
    qsl = torch.tensor([0, 3, 4, 6], dtype=torch.int32)
    lens = torch.tensor([10, 7, 2], dtype=torch.int32)
    bt = torch.tensor([[5, 6], [7, 8], [9, 0]], dtype=torch.int32)
    ctx, tbt = expand_to_token_sequences(qsl, lens, bt, 6)
    assert ctx.tolist() == [8, 9, 10, 7, 1, 2]
    assert tbt.tolist() == [[5, 6]] * 3 + [[7, 8]] + [[9, 0]] * 2
    assert ctx.dtype == torch.int32


def test_backend_static_interface():
    B = B200PagedAttentionBackend
    assert B.get_name() == "B200_PAGED_ATTN"
    assert B.get_impl_cls() is B200PagedAttentionImpl
    assert B.get_builder_cls() is B200PagedAttentionMetadataBuilder
    assert B.get_kv_cache_shape(10, 16, 8, 128) == (2, 10, 16 * 8 * 128)
    assert B.use_cascade_attention() is False
    with pytest.raises(ValueError):
        B.validate_head_size(48)
    with pytest.raises(ValueError):
        B.get_kv_cache_shape(10, 64, 8, 128)
    with pytest.raises(NotImplementedError):
        B200PagedAttentionImpl(8, 128, 0.1, 2, sliding_window=128)


def test_metadata_builder_has_the_engine_facing_signature():
    """The engine constructs builders as Builder(kv_cache_spec, layer_names, vllm_config, device)
    and calls build(common_prefix_len, common_attn_metadata, fast_build)
    (vllm/v1/attention/backends/utils.py:255-330, rocm_attn.py:65-150)."""
    import inspect
    assert list(inspect.signature(B200PagedAttentionMetadataBuilder.__init__).parameters) == [
        "self", "kv_cache_spec", "layer_names", "vllm_config", "device"]
    assert list(inspect.signature(B200PagedAttentionMetadataBuilder.build).parameters) == [
        "self", "common_prefix_len", "common_attn_metadata", "fast_build"]
    b = B200PagedAttentionMetadataBuilder(types.SimpleNamespace(block_size=32), ["l0", "l1"], None, "cpu")
    assert b.block_size == 32 and b.layer_names == ["l0", "l1"]
    assert B200PagedAttentionMetadataBuilder.get_cudagraph_support(None, None) == "ALWAYS"
    common = types.SimpleNamespace(
        query_start_loc=torch.tensor([0, 1, 2], dtype=torch.int32), seq_lens=torch.tensor([7, 9], dtype=torch.int32),
        num_reqs=2, num_actual_tokens=2, max_query_len=1, max_seq_len=9,
        block_table_tensor=torch.zeros(2, 1, dtype=torch.int32), slot_mapping=torch.tensor([6, 40]))
    md = b.build(0, common, fast_build=True)
    assert md.block_table is common.block_table_tensor and md.max_seq_len == 9 and md.use_cascade is False
    cap = b.build_for_cudagraph_capture(common)
    assert cap.seq_lens.tolist() == [1, 1]
    with pytest.raises(NotImplementedError):
        b.build(16, common)


def test_plugin_repoints_the_wrappers_of_a_custom_ops_module():
    """vllm_b200.plugin.register() against a stand-in for vllm._custom_ops and for the backend
    registry: the wrappers of this path are replaced by functions of the same name, everything
    else is left alone, the backend is registered as CUSTOM, and a second call changes nothing."""
    import sys

    from vllm_b200 import _custom_ops as b200
    from vllm_b200 import plugin

    def _orig(*a, **k):
        raise AssertionError("the reference wrapper was called")

    fake_ops = types.ModuleType("fake_vllm_custom_ops")
    for name in plugin.OPS:
        setattr(fake_ops, name, _orig)
    fake_ops.rms_norm = _orig  # not on this path
    registered = []
    fake_reg = types.ModuleType("fake_vllm_registry")
    fake_reg.AttentionBackendEnum = types.SimpleNamespace(CUSTOM="CUSTOM")
    fake_reg.register_backend = lambda which, path: registered.append((which, path))
    sys.modules["fake_vllm_custom_ops"], sys.modules["fake_vllm_registry"] = fake_ops, fake_reg
    try:
        for _ in range(2):
            done = plugin.register("fake_vllm_custom_ops", "fake_vllm_registry")
            assert set(done["ops"]) == set(plugin.OPS) and done["backend"] is True
            for name in ("paged_attention_v1", "paged_attention_v2", "reshape_and_cache",
                         "reshape_and_cache_flash", "convert_fp8"):
                assert getattr(fake_ops, name) is getattr(b200, name)
            assert fake_ops.rms_norm is _orig
        assert registered[0] == ("CUSTOM", "vllm_b200.backend.B200PagedAttentionBackend")
        import importlib
        mod, cls = registered[0][1].rsplit(".", 1)
        assert getattr(importlib.import_module(mod), cls) is B200PagedAttentionBackend
        plugin.unregister("fake_vllm_custom_ops")
        assert fake_ops.paged_attention_v1 is _orig
        # without a registry module only the wrappers are patched
        assert plugin.register("fake_vllm_custom_ops", "no_such_registry_module")["backend"] is False
    finally:
        del sys.modules["fake_vllm_custom_ops"], sys.modules["fake_vllm_registry"]


def _dense_causal(q, k, v, scale, g):
    """q [n, Hq, D] are the last n positions of a sequence whose keys are k [L, Hkv, D]."""
    L, n = k.shape[0], q.shape[0]
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    logits = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    pos_q = torch.arange(L - n, L, device=q.device).view(1, n, 1)
    mask = torch.arange(L, device=q.device).view(1, 1, L) > pos_q
    logits = logits.masked_fill(mask, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(logits, dim=-1), vv)


@pytest.mark.gpu
@pytest.mark.parametrize("kv_cache_dtype", ["auto", "fp8"])
def test_prefill_chunk_and_decode_session(kv_cache_dtype):
    dev = "cuda"
    Hq, Hkv, D, B, NB = 8, 2, 128, 16, 64
    g = Hq // Hkv
    dtype = torch.bfloat16
    impl = B200PagedAttentionImpl(Hq, D, D ** -0.5, Hkv, kv_cache_dtype=kv_cache_dtype)
    shape = B200PagedAttentionBackend.get_kv_cache_shape(NB, B, Hkv, D, kv_cache_dtype)
    kv_cache = torch.zeros(shape, dtype=torch.uint8 if kv_cache_dtype == "fp8" else dtype, device=dev)
    layer = types.SimpleNamespace(_k_scale=torch.tensor(0.05 if kv_cache_dtype == "fp8" else 1.0, device=dev),
                                  _v_scale=torch.tensor(0.04 if kv_cache_dtype == "fp8" else 1.0, device=dev))
    builder = B200PagedAttentionMetadataBuilder(types.SimpleNamespace(block_size=B), ["layer.0"], None, dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    rng = np.random.default_rng(0)
    nreq = 3
    perm = rng.permutation(NB).astype(np.int32)
    bt = torch.from_numpy(perm[:nreq * 8].reshape(nreq, 8)).to(dev)  # 8 blocks = 128 tokens per request
    hist_k = [torch.zeros(0, Hkv, D, device=dev, dtype=dtype) for _ in range(nreq)]
    hist_v = [torch.zeros(0, Hkv, D, device=dev, dtype=dtype) for _ in range(nreq)]
    # steps: (new tokens per request): prefill, a mixed chunked-prefill/decode step, then decode steps
    for step_lens in ([37, 20, 5], [9, 1, 30], [1, 1, 1], [1, 1, 1]):
        n = sum(step_lens)
        q = torch.randn(n, Hq, D, device=dev, generator=gen).to(dtype)
        k = torch.randn(n, Hkv, D, device=dev, generator=gen).to(dtype)
        v = torch.randn(n, Hkv, D, device=dev, generator=gen).to(dtype)
        qsl = torch.tensor([0] + list(np.cumsum(step_lens)), dtype=torch.int32, device=dev)
        slots, off = [], 0
        for r, ln in enumerate(step_lens):
            start = hist_k[r].shape[0]
            pos = torch.arange(start, start + ln, device=dev)
            slots.append(bt[r, pos // B].long() * B + pos % B)
            kk, vv = k[off:off + ln], v[off:off + ln]
            if kv_cache_dtype == "fp8":
                # the dense reference sees what the cache holds: quantised then dequantised values
                ks, vs = float(layer._k_scale), float(layer._v_scale)
                kk = O.dequantize_fp8(O.quantize_fp8(kk.cpu(), ks), ks, torch.float32).to(dev)
                vv = O.dequantize_fp8(O.quantize_fp8(vv.cpu(), vs), vs, torch.float32).to(dev)
            hist_k[r] = torch.cat([hist_k[r].to(kk.dtype), kk])
            hist_v[r] = torch.cat([hist_v[r].to(vv.dtype), vv])
            off += ln
        lens = torch.tensor([h.shape[0] for h in hist_k], dtype=torch.int32, device=dev)
        # what the engine hands every builder (CommonAttentionMetadata, utils.py:53-95)
        common = types.SimpleNamespace(
            query_start_loc=qsl, query_start_loc_cpu=qsl.cpu(), seq_lens=lens, seq_lens_cpu=lens.cpu(),
            num_computed_tokens_cpu=(lens.cpu() - torch.tensor(step_lens)), num_reqs=nreq,
            num_actual_tokens=n, max_query_len=max(step_lens), max_seq_len=int(lens.max()),
            block_table_tensor=bt, slot_mapping=torch.cat(slots), causal=True)
        md = builder.build(0, common)
        out = torch.empty(n + 3, Hq * D, device=dev, dtype=dtype)  # padded like a CUDA-graph batch
        impl.forward(layer, torch.cat([q, q[:3]]), torch.cat([k, k[:3]]), torch.cat([v, v[:3]]),
                     kv_cache, md, output=out)
        off = 0
        for r, ln in enumerate(step_lens):
            want = _dense_causal(q[off:off + ln], hist_k[r], hist_v[r], D ** -0.5, g)
            got = out[off:off + ln].view(ln, Hq, D).float()
            tol = dict(atol=2e-2, rtol=2e-2) if kv_cache_dtype == "fp8" else dict(atol=1e-2, rtol=1e-2)
            torch.testing.assert_close(got, want, **tol)
            off += ln
