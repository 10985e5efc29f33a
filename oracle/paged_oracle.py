"""CPU oracle for the PagedAttention decode path.  TEST INFRASTRUCTURE ONLY.

A PyTorch-on-CPU restatement of what the reference's CUDA kernels compute, used
as the checker in ``tests/``, in ``__graft_entry__.smoke()`` and as the "port"
CPU baseline of ``bench.py``.  The product never imports this module.

What each function follows in the reference:

``quantize_fp8`` / ``dequantize_fp8``
    ``fp8::scaled_convert`` — csrc/quantization/w8a8/fp8/nvidia/quant_utils.cuh:469-502
    (quantise: IEEE fp32 division, cvt round-to-nearest-even, saturate-to-finite,
    NaN -> 0x7F) and :360-372 (dequantise: fp8 -> half -> float * scale -> T).
``reshape_and_cache`` / ``reshape_and_cache_flash``
    csrc/cache_kernels.cu:225-283 and :285-358 (index formulas, ``slot < 0`` skipped).
``paged_attention`` (mode="ref")
    csrc/attention/attention_kernels.cuh:81-491 with its rounding points: fp32
    logits, ``exp`` softmax with ``1/(sum + 1e-6)``, P rounded to the value dtype,
    the P*V product formed in that dtype, fp32 accumulation; with
    ``partition_size`` the v2 split (:106-131, :344-352) and the reduce kernel
    (:559-664) including the rounding of the partial outputs to T.
``paged_attention`` (mode="f64")
    the same mathematics in float64 without intermediate rounding
    (tests/kernels/attention/test_attention.py:47-114 is the PyTorch statement).

Pinning: the quantiser is checked bit-for-bit against golden vectors produced by
NVIDIA's host ``__nv_cvt_float_to_fp8`` (tests/golden/fp8_*.npz); attention is
checked against outputs of the reference's own CPU attention kernel
(tests/golden/cpu_attn_*.npz) and, on a GPU box, against the reference's CUDA
kernels compiled from its sources (oracle/_ref/_C_ref.so).
"""
from __future__ import annotations

import math

import torch

FP8_FORMATS = {
    "fp8": (torch.float8_e4m3fn, 448.0),
    "fp8_e4m3": (torch.float8_e4m3fn, 448.0),
    "fp8_ds_mla": (torch.float8_e4m3fn, 448.0),
    "fp8_e5m2": (torch.float8_e5m2, 57344.0),
}


def is_fp8(kv_cache_dtype: str) -> bool:
    if kv_cache_dtype == "auto":
        return False
    if kv_cache_dtype not in FP8_FORMATS:
        raise RuntimeError(f"Unsupported data type of kv cache: {kv_cache_dtype}")
    return True


def quantize_fp8(x: torch.Tensor, scale: float, kv_cache_dtype: str = "fp8") -> torch.Tensor:
    """bits = cvt_rn_satfinite(float(x) / scale) as uint8 (NaN -> 0x7F)."""
    dt, fmax = FP8_FORMATS[kv_cache_dtype]
    q = x.to(torch.float32) / torch.tensor(scale, dtype=torch.float32)
    bits = q.clamp(-fmax, fmax).to(dt).view(torch.uint8).clone()
    bits[q.isnan()] = 0x7F
    return bits


def dequantize_fp8(bits: torch.Tensor, scale: float, out_dtype: torch.dtype,
                   kv_cache_dtype: str = "fp8") -> torch.Tensor:
    """T(float(half(fp8)) * scale): every fp8 value is exact in half."""
    dt, _ = FP8_FORMATS[kv_cache_dtype]
    f = bits.view(dt).to(torch.float32) * torch.tensor(scale, dtype=torch.float32)
    return f.to(out_dtype)


def _scalar(t) -> float:
    return float(t.item()) if isinstance(t, torch.Tensor) else float(t)


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
                      k_scale, v_scale) -> None:
    """x-layout KV write: K -> [b, h, d/x, t, d%x], V -> [b, h, d, t] (in place)."""
    num_tokens = slot_mapping.shape[0]
    block_size = key_cache.shape[3]
    x = key_cache.shape[4]
    H, D = key.shape[1], key.shape[2]
    slots = slot_mapping.to(torch.int64)
    keep = slots >= 0
    idx = torch.nonzero(keep).flatten()
    if idx.numel() == 0:
        return
    k = key[:num_tokens][idx]
    v = value[:num_tokens][idx]
    if is_fp8(kv_cache_dtype):
        k = quantize_fp8(k, _scalar(k_scale), kv_cache_dtype)
        v = quantize_fp8(v, _scalar(v_scale), kv_cache_dtype)
        kc = key_cache.view(torch.uint8)
        vc = value_cache.view(torch.uint8)
    else:
        kc, vc = key_cache, value_cache
    b = torch.div(slots[idx], block_size, rounding_mode="floor")
    t = slots[idx] % block_size
    kc[b, :, :, t, :] = k.reshape(-1, H, D // x, x)
    vc[b, :, :, t] = v


def reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
                            k_scale, v_scale) -> None:
    """flash-layout KV write into [num_blocks, block_size, H, D] views (any strides)."""
    num_tokens = slot_mapping.shape[0]
    block_size = key_cache.shape[1]
    slots = slot_mapping.to(torch.int64)
    idx = torch.nonzero(slots >= 0).flatten()
    if idx.numel() == 0:
        return
    k = key[:num_tokens][idx]
    v = value[:num_tokens][idx]
    if is_fp8(kv_cache_dtype):
        k = quantize_fp8(k, _scalar(k_scale), kv_cache_dtype)
        v = quantize_fp8(v, _scalar(v_scale), kv_cache_dtype)
        kc = key_cache.view(torch.uint8)
        vc = value_cache.view(torch.uint8)
    else:
        kc, vc = key_cache, value_cache
    b = torch.div(slots[idx], block_size, rounding_mode="floor")
    t = slots[idx] % block_size
    kc[b, t] = k
    vc[b, t] = v


def gather_kv(key_cache, value_cache, block_table, seq_len, kv_cache_dtype, k_scale, v_scale,
              work_dtype):
    """Returns K, V of one sequence as [seq_len, Hkv, D] tensors of ``work_dtype``
    (fp8 caches dequantised with the reference's rounding to the query dtype)."""
    B = value_cache.shape[3]
    nblk = (seq_len + B - 1) // B
    blocks = block_table[:nblk].to(torch.int64)
    kc = key_cache[blocks]    # [nblk, H, D/x, B, x]
    vc = value_cache[blocks]  # [nblk, H, D, B]
    nb, H, Dx, _, x = kc.shape
    k = kc.permute(0, 3, 1, 2, 4).reshape(nb * B, H, Dx * x)[:seq_len]
    v = vc.permute(0, 3, 1, 2).reshape(nb * B, H, -1)[:seq_len]
    if is_fp8(kv_cache_dtype):
        k = dequantize_fp8(k.contiguous().view(torch.uint8), _scalar(k_scale), work_dtype, kv_cache_dtype)
        v = dequantize_fp8(v.contiguous().view(torch.uint8), _scalar(v_scale), work_dtype, kv_cache_dtype)
    return k, v


def _attend_ref(q, k, v, scale, slopes, seq_len, tok0, T):
    """One (sequence, token range) with the reference's rounding points.
    q [Hq, D] (T), k/v [n, Hq, D] (T).  Returns (out fp32 [Hq, D] normalised, m [Hq], l [Hq])."""
    n = k.shape[0]
    logits = torch.einsum("hd,nhd->hn", q.float(), k.float()) * scale
    if slopes is not None:
        pos = torch.arange(tok0, tok0 + n, dtype=torch.float32) - seq_len + 1
        logits = logits + slopes.view(-1, 1).float() * pos.view(1, -1)
    m = logits.max(dim=1).values
    e = torch.exp(logits - m.view(-1, 1))
    l = e.sum(dim=1)
    p = e * (1.0 / (l + 1e-6)).view(-1, 1)
    p_t = p.to(T)
    prod = (p_t.float().transpose(0, 1).unsqueeze(-1) * v.float()).to(T)  # product formed in T
    out = prod.float().sum(dim=0)
    return out, m, l


def blocksparse_mask(seq_len, block_size, num_heads, num_kv_heads, tp_rank, local_blocks,
                     vert_stride, bs_block_size, head_sliding_step):
    """[Hq, seq_len] bool: which tokens a head attends to under the reference's block-sparse
    pattern (csrc/attention/attention_kernels.cuh:204-251): a KV block is kept when it is one
    of the last `local_blocks` sparse blocks or every `vert_stride`-th one, shifted per head."""
    tok = torch.arange(seq_len)
    kb = (tok // block_size) * block_size // bs_block_size
    q_blk = (seq_len - 1) // bs_block_size
    g = num_heads // num_kv_heads
    rows = []
    for h in range(num_heads):
        if head_sliding_step >= 0:
            off = (tp_rank * num_heads + h) * head_sliding_step + 1
        else:
            off = (tp_rank * num_kv_heads + h // g) * (-head_sliding_step) + 1
        rows.append(((kb + off) % vert_stride == 0) | (kb > q_blk - local_blocks))
    return torch.stack(rows, 0)


def paged_attention(query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
                    alibi_slopes=None, kv_cache_dtype="auto", k_scale=1.0, v_scale=1.0,
                    mode="ref", partition_size=None, seqs=None, blocksparse=None, return_lse=False):
    """Decode attention over a paged KV cache; returns ``out`` [S, Hq, D].

    mode="ref": reference rounding points, result in the query dtype.
    mode="f64": float64 mathematics, result in float64.
    partition_size: None = one pass per sequence (v1); an int = v2 split + reduce.
    seqs: optional iterable of sequence indices to compute (others are left zero).
    blocksparse: None or (tp_rank, local_blocks, vert_stride, block_size, head_sliding_step);
        only with mode="f64" (masked tokens get zero weight).
    return_lse: with mode="f64" also return lse [Hq, S] float64, the natural log of the sum of
        exp(scaled logit + bias) over each sequence's tokens (-inf for an empty sequence): the
        quantity merge_attn_states combines partial attention results with.
    """
    S, Hq, D = query.shape
    G = Hq // num_kv_heads
    T = query.dtype
    out = torch.zeros((S, Hq, D), dtype=torch.float64 if mode == "f64" else T)
    lse = torch.full((Hq, S), -math.inf, dtype=torch.float64)
    assert not return_lse or mode == "f64"
    lens = seq_lens.tolist()
    for s in (range(S) if seqs is None else seqs):
        L = int(lens[s])
        if L == 0:
            continue
        # mode "f64" dequantises fp8 exactly (no rounding to T)
        work = torch.float32 if mode == "f64" else T
        k, v = gather_kv(key_cache, value_cache, block_tables[s], L, kv_cache_dtype, k_scale,
                         v_scale, work)
        if G > 1:
            k = k.repeat_interleave(G, dim=1)
            v = v.repeat_interleave(G, dim=1)
        q = query[s]
        if mode == "f64":
            logits = torch.einsum("hd,nhd->hn", q.double(), k.double()) * scale
            if alibi_slopes is not None:
                pos = torch.arange(L, dtype=torch.float64) - L + 1
                logits = logits + alibi_slopes.view(-1, 1).double() * pos.view(1, -1)
            if blocksparse is not None:
                keep = blocksparse_mask(L, value_cache.shape[3], Hq, num_kv_heads, *blocksparse)
                logits = logits.masked_fill(~keep, -math.inf)
            p = torch.softmax(logits, dim=1)
            out[s] = torch.einsum("hn,nhd->hd", p, v.double())
            lse[:, s] = torch.logsumexp(logits, dim=1)
            continue
        if partition_size is None:
            o, _, _ = _attend_ref(q, k, v, scale, alibi_slopes, L, 0, T)
            out[s] = o.to(T)
            continue
        nparts = (L + partition_size - 1) // partition_size
        if nparts == 1:
            # the reduce kernel copies the single partial through (:577-589)
            o, _, _ = _attend_ref(q, k, v, scale, alibi_slopes, L, 0, T)
            out[s] = o.to(T)
            continue
        tmp, ms, ls = [], [], []
        for j in range(nparts):
            a, b = j * partition_size, min(L, (j + 1) * partition_size)
            o, m, l = _attend_ref(q, k[a:b], v[a:b], scale, alibi_slopes, L, a, T)
            tmp.append(o.to(T))
            ms.append(m)
            ls.append(l)
        tmp = torch.stack(tmp, 0).float()       # [P, Hq, D]
        ms = torch.stack(ms, 0)                 # [P, Hq]
        ls = torch.stack(ls, 0)
        M = ms.max(dim=0).values
        r = ls * torch.exp(ms - M.view(1, -1))
        inv = 1.0 / (r.sum(dim=0) + 1e-6)
        out[s] = (tmp * r.unsqueeze(-1) * inv.view(1, -1, 1)).sum(dim=0).to(T)
    return (out, lse) if return_lse else out


def attn_bytes(seq_lens, num_heads, num_kv_heads, head_size, block_size, q_bytes, cache_bytes):
    """Algorithmic bytes of one decode call: KV read once (GQA-shared) + Q read +
    O write + block-table entries + seq_lens."""
    lens = [int(v) for v in seq_lens]
    kv = sum(lens) * num_kv_heads * head_size * 2 * cache_bytes
    qo = 2 * len(lens) * num_heads * head_size * q_bytes
    bt = 4 * sum((n + block_size - 1) // block_size for n in lens) + 4 * len(lens)
    return kv + qo + bt


def merge_attn_states(prefix_output, prefix_lse, suffix_output, suffix_lse):
    """LSE-weighted merge of two partial attention results
    (csrc/attention/merge_attn_states.cu:14-114): outputs [T, H, D], lse [H, T].
    Infinite LSEs count as -inf; when both are, the prefix passes through.
    Returns (output in the input dtype, output_lse float32)."""
    p_lse = torch.where(torch.isinf(prefix_lse), torch.full_like(prefix_lse, -math.inf), prefix_lse)
    s_lse = torch.where(torch.isinf(suffix_lse), torch.full_like(suffix_lse, -math.inf), suffix_lse)
    mx = torch.maximum(p_lse, s_lse)
    dead = torch.isinf(mx)
    safe = torch.where(dead, torch.zeros_like(mx), mx)
    p_se = torch.exp(p_lse - safe)
    s_se = torch.exp(s_lse - safe)
    tot = p_se + s_se
    ps = (p_se / tot).transpose(0, 1).unsqueeze(-1)  # [T, H, 1]
    ss = (s_se / tot).transpose(0, 1).unsqueeze(-1)
    out = prefix_output.float() * ps + suffix_output.float() * ss
    dead_th = dead.transpose(0, 1).unsqueeze(-1)
    out = torch.where(dead_th, prefix_output.float(), out).to(prefix_output.dtype)
    lse = torch.where(dead, mx, torch.log(tot) + safe)
    return out, lse


def copy_blocks(key_caches, value_caches, block_mapping) -> None:
    """csrc/cache_kernels.cu:73-171: block src -> block dst in every layer's K and V cache."""
    for src, dst in block_mapping.tolist():
        for kc, vc in zip(key_caches, value_caches):
            kc[dst].copy_(kc[src])
            vc[dst].copy_(vc[src])


def swap_blocks(src, dst, block_mapping) -> None:
    """csrc/cache_kernels.cu:26-69: whole-block copies between two caches."""
    for s, d in block_mapping.tolist():
        dst[d].copy_(src[s])
