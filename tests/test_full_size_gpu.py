"""Parity at the full benchmark sizes, through properties that do not need the CPU
oracle on gigabytes of cache: agreement of the two partitionings (v1 / v2), exact
linearity in V, invariance under relocation of the physical blocks, the oracle on a
subsample of sequences, and KV write -> read-back round trips."""
import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200 import _custom_ops as ops
from vllm_b200 import capi
import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _oracle_subsample(w, out, seqs, tol):
    idx = torch.tensor(seqs, device=DEV)
    lens = w.seq_lens[idx].cpu()
    need = int(np.ceil(lens.numpy() / w.block_size).max())
    bt = w.block_tables[idx, :need].cpu()
    uniq, inv = torch.unique(bt.flatten(), return_inverse=True)
    kc = w.key_cache[uniq.to(DEV).long()].cpu()
    vc = w.value_cache[uniq.to(DEV).long()].cpu()
    want = O.paged_attention(w.query[idx].cpu(), kc, vc, w.num_kv_heads, w.scale,
                             inv.view(bt.shape).int(), lens, None, w.kv_cache_dtype,
                             float(w.k_scale), float(w.v_scale), mode="f64")
    torch.testing.assert_close(out[idx].cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("cfg", ["cfg2", "cfg3", "cfg4"])
def test_full_size_properties(cfg):
    w = {"cfg2": W.config2, "cfg3": W.config3, "cfg4": W.config4}[cfg](DEV)
    w.query.mul_(16.0)  # away from the uniform-softmax regime
    tol = 2e-2 if w.kv_cache_dtype != "auto" else 1e-2
    out2 = W.run_attention(w, version="v2").clone()
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.isfinite(out2.float()).all()

    # (1) v1 partitions sequences differently (or not at all): same answer within tolerance
    out1 = W.run_attention(w, version="v1")
    torch.testing.assert_close(out1.float(), out2.float(), atol=tol, rtol=tol)

    # (2) the oracle on a few sequences (shortest, longest, first, last)
    lens = w.seq_lens.cpu().numpy()
    seqs = sorted({0, len(lens) - 1, int(lens.argmin()), int(lens.argmax())})
    _oracle_subsample(w, out2, seqs, tol)

    # (3) exact linearity in V: doubling V (exact in bf16; for fp8 doubling v_scale) doubles
    #     the output bit for bit
    if w.kv_cache_dtype == "auto":
        w.value_cache.mul_(2.0)
    else:
        w.v_scale.mul_(2.0)
    out_lin = W.run_attention(w, version="v2")
    assert torch.equal(out_lin.float(), out2.float() * 2.0)
    if w.kv_cache_dtype == "auto":
        w.value_cache.mul_(0.5)
    else:
        w.v_scale.mul_(0.5)

    # (4) relocating the physical blocks (same contents, new block ids) changes nothing
    nb = w.key_cache.shape[0]
    perm = torch.randperm(nb, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb, device=DEV)
    kc2 = torch.empty_like(w.key_cache)
    vc2 = torch.empty_like(w.value_cache)
    kc2[inv] = w.key_cache   # block b moves to position inv[b]
    vc2[inv] = w.value_cache
    old_k, old_v, old_bt = w.key_cache, w.value_cache, w.block_tables
    w.key_cache, w.value_cache = kc2, vc2
    w.block_tables = inv[old_bt.long()].int()
    out_perm = W.run_attention(w, version="v2")
    assert torch.equal(out_perm, out2)
    w.key_cache, w.value_cache, w.block_tables = old_k, old_v, old_bt


def test_full_size_kv_write_round_trip():
    """config 3: 16 384 new tokens quantised into the fp8 cache; reading the written slots
    back gives exactly the oracle's codes, everything else is untouched, and writing twice is
    idempotent."""
    w = W.config3(DEV)
    before_k = w.key_cache.clone()
    ops.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping, "fp8",
                          w.k_scale, w.v_scale)
    B = w.block_size
    slots = w.slot_mapping
    blk, off = slots // B, slots % B
    got_k = w.key_cache[blk, :, :, off, :].reshape(slots.numel(), 8, 128)
    got_v = w.value_cache[blk, :, :, off]
    want_k = O.quantize_fp8(w.new_key.cpu(), float(w.k_scale), "fp8")
    want_v = O.quantize_fp8(w.new_value.cpu(), float(w.v_scale), "fp8")
    assert torch.equal(got_k.cpu(), want_k)
    assert torch.equal(got_v.cpu(), want_v)
    # untouched positions keep their bytes: positions before the last 128 of each sequence
    mask = torch.ones(w.key_cache.shape[0], B, dtype=torch.bool, device=DEV)
    mask[blk, off] = False
    same = (w.key_cache == before_k).all(dim=(1, 2, 4))  # [NB, B]
    assert bool(same[mask].all())
    snap_k, snap_v = w.key_cache.clone(), w.value_cache.clone()
    ops.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping, "fp8",
                          w.k_scale, w.v_scale)
    assert torch.equal(w.key_cache, snap_k) and torch.equal(w.value_cache, snap_v)


def test_config5_full_batch():
    """config 5 as stated: 2048 sequences, 64 query / 8 KV heads, block size 32, fp8-e4m3,
    lengths U{1024..8192} (about 19 GB of cache).  The oracle on a subsample of sequences,
    agreement of v1 (library workspace) and v2 (caller scratch), exact linearity in v_scale."""
    w = W.config5(DEV)
    assert w.num_seqs == 2048 and w.block_size == 32 and w.kv_cache_dtype == "fp8"
    w.query.mul_(16.0)
    scratch = w.scratch()
    out2 = W.run_attention(w, version="v2", scratch=scratch).clone()
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    assert torch.isfinite(out2.float()).all()
    out1 = W.run_attention(w, version="v1")
    torch.testing.assert_close(out1.float(), out2.float(), atol=2e-2, rtol=2e-2)
    lens = w.seq_lens.cpu().numpy()
    rng = np.random.default_rng(5)
    seqs = sorted({0, 2047, int(lens.argmin()), int(lens.argmax())} | set(rng.integers(0, 2048, size=4).tolist()))
    _oracle_subsample(w, out2, seqs, 2e-2)
    w.v_scale.mul_(2.0)
    out_lin = W.run_attention(w, version="v2", scratch=scratch)
    assert torch.equal(out_lin.float(), out2.float() * 2.0)
    w.v_scale.mul_(0.5)


def test_config5_shape_subsample():
    """config 5 shape (fp8, block size 32, 64/8 heads) at a quarter of the batch: oracle on
    four sequences, v1/v2 agreement."""
    w = W.config5(DEV, num_seqs=512)
    w.query.mul_(16.0)
    out2 = W.run_attention(w, version="v2").clone()
    out1 = W.run_attention(w, version="v1")
    torch.testing.assert_close(out1.float(), out2.float(), atol=2e-2, rtol=2e-2)
    lens = w.seq_lens.cpu().numpy()
    _oracle_subsample(w, out2, sorted({0, 511, int(lens.argmin()), int(lens.argmax())}), 2e-2)
