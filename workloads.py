"""Synthetic decode workloads (the five benchmark / parity configurations).

Inputs mirror the reference's test and benchmark factories
(``vllm/utils/torch_utils.py:206-294`` ``create_kv_caches_with_random``,
``benchmarks/kernels/benchmark_paged_attention.py:43-80``): query and 16-bit
caches ~ U(-D^-0.5, D^-0.5), fp8 caches made by quantising N(0,1) data with a
per-tensor scale amax/448, K cache ``[NB, Hkv, D/x, B, x]``, V cache
``[NB, Hkv, D, B]``, int32 zero-padded block tables, int32 ``seq_lens``.

Sequence lengths and block assignments come from ``numpy.random.default_rng(seed)``
on the host (identical on every rank); tensor contents come from a
``torch.Generator`` on the target device.  No public dataset is involved.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

PARTITION = 512


@dataclasses.dataclass
class Workload:
    name: str
    query: torch.Tensor
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    block_tables: torch.Tensor
    seq_lens: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    num_kv_heads: int
    scale: float
    block_size: int
    max_seq_len: int
    kv_cache_dtype: str
    alibi_slopes: torch.Tensor | None = None
    # new tokens for the KV-write step (config 3)
    new_key: torch.Tensor | None = None
    new_value: torch.Tensor | None = None
    slot_mapping: torch.Tensor | None = None

    @property
    def num_seqs(self) -> int:
        return self.query.shape[0]

    @property
    def num_heads(self) -> int:
        return self.query.shape[1]

    @property
    def head_size(self) -> int:
        return self.query.shape[2]

    @property
    def max_num_partitions(self) -> int:
        return (self.max_seq_len + PARTITION - 1) // PARTITION

    def total_tokens(self) -> int:
        return int(self.seq_lens.sum().item())

    def attn_bytes(self) -> int:
        """Algorithmic bytes of one decode call: KV read once (shared by the query
        heads of a group) + Q read + O write + block-table entries + seq_lens."""
        lens = self.seq_lens.cpu().numpy().astype(np.int64)
        cache_b = self.key_cache.element_size()
        kv = int(lens.sum()) * self.num_kv_heads * self.head_size * 2 * cache_b
        qo = 2 * self.num_seqs * self.num_heads * self.head_size * self.query.element_size()
        bt = 4 * int(np.ceil(lens / self.block_size).sum()) + 4 * self.num_seqs
        return kv + qo + bt

    def reshape_bytes(self) -> int:
        if self.new_key is None:
            return 0
        T, H, D = self.new_key.shape
        return T * H * D * (2 * self.new_key.element_size() + 2 * self.key_cache.element_size()) + 8 * T

    def scratch(self):
        """v2 scratch tensors as the reference's caller allocates them
        (vllm/attention/ops/paged_attn.py:164-174)."""
        S, Hq, D = self.query.shape
        P = self.max_num_partitions
        dev = self.query.device
        tmp_out = torch.empty((S, Hq, P, D), dtype=self.query.dtype, device=dev)
        exp_sums = torch.empty((S, Hq, P), dtype=torch.float32, device=dev)
        max_logits = torch.empty_like(exp_sums)
        return exp_sums, max_logits, tmp_out


def _deal_blocks(rng: np.random.Generator, lens: np.ndarray, block_size: int, num_blocks: int | None,
                 unique_global: bool):
    """Block tables [S, max_blocks]: either one global permutation dealt out to the
    sequences (unique blocks) or an independent sample without replacement per row."""
    need = np.ceil(lens / block_size).astype(np.int64)
    maxb = int(max(1, need.max()))
    S = len(lens)
    bt = np.zeros((S, maxb), dtype=np.int32)
    if unique_global:
        total = int(need.sum())
        nb = num_blocks if num_blocks is not None else int(math.ceil(1.25 * total))
        perm = rng.permutation(nb)[:total].astype(np.int32)
        off = 0
        for s in range(S):
            bt[s, : need[s]] = perm[off: off + need[s]]
            off += need[s]
    else:
        nb = num_blocks
        for s in range(S):
            bt[s, : need[s]] = rng.choice(nb, size=int(need[s]), replace=False).astype(np.int32)
    return bt, nb


def _uniform_(t: torch.Tensor, lo: float, hi: float, gen: torch.Generator) -> None:
    # chunked so that multi-GB caches do not need a full-size float32 temporary
    flat = t.view(-1)
    step = 1 << 27
    for a in range(0, flat.numel(), step):
        b = min(flat.numel(), a + step)
        tmp = torch.empty(b - a, dtype=torch.float32, device=t.device)
        tmp.uniform_(lo, hi, generator=gen)
        flat[a:b] = tmp.to(t.dtype)


def _fp8_normal_(t: torch.Tensor, scale: float, gen: torch.Generator, e5m2: bool = False) -> None:
    """Fills a uint8 tensor with e4m3 (or e5m2) codes of N(0,1)/scale (RNE, saturating)."""
    flat = t.view(-1)
    step = 1 << 27
    fmax, dt = (57344.0, torch.float8_e5m2) if e5m2 else (448.0, torch.float8_e4m3fn)
    for a in range(0, flat.numel(), step):
        b = min(flat.numel(), a + step)
        tmp = torch.empty(b - a, dtype=torch.float32, device=t.device)
        tmp.normal_(0.0, 1.0, generator=gen)
        tmp.div_(scale).clamp_(-fmax, fmax)
        flat[a:b] = tmp.to(dt).view(torch.uint8)


def make_decode(name: str, *, num_seqs: int, num_heads: int, num_kv_heads: int, head_size: int,
                block_size: int, lens: np.ndarray, dtype: torch.dtype, kv_cache_dtype: str,
                device, seed: int, rng: np.random.Generator, num_blocks: int | None = None,
                unique_global: bool = True, max_seq_len: int | None = None) -> Workload:
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    lens = np.asarray(lens, dtype=np.int64)
    bt, nb = _deal_blocks(rng, lens, block_size, num_blocks, unique_global)
    amp = head_size ** -0.5
    q = torch.empty((num_seqs, num_heads, head_size), dtype=dtype, device=dev)
    _uniform_(q, -amp, amp, gen)
    fp8 = kv_cache_dtype != "auto"
    cdt = torch.uint8 if fp8 else dtype
    x = 16 // (1 if fp8 else q.element_size())
    kc = torch.empty((nb, num_kv_heads, head_size // x, block_size, x), dtype=cdt, device=dev)
    vc = torch.empty((nb, num_kv_heads, head_size, block_size), dtype=cdt, device=dev)
    if fp8:
        # per-tensor scales as a caller would compute them: amax / 448 of N(0,1) data
        e5m2 = kv_cache_dtype == "fp8_e5m2"
        fmax = 57344.0 if e5m2 else 448.0
        ks, vs = 5.3 / fmax, 5.2 / fmax
        _fp8_normal_(kc, ks, gen, e5m2)
        _fp8_normal_(vc, vs, gen, e5m2)
    else:
        ks = vs = 1.0
        _uniform_(kc, -amp, amp, gen)
        _uniform_(vc, -amp, amp, gen)
    return Workload(
        name=name, query=q, key_cache=kc, value_cache=vc,
        block_tables=torch.from_numpy(bt).to(dev),
        seq_lens=torch.from_numpy(lens.astype(np.int32)).to(dev),
        k_scale=torch.tensor(ks, dtype=torch.float32, device=dev),
        v_scale=torch.tensor(vs, dtype=torch.float32, device=dev),
        num_kv_heads=num_kv_heads, scale=float(head_size ** -0.5), block_size=block_size,
        max_seq_len=int(max_seq_len if max_seq_len is not None else max(1, lens.max())),
        kv_cache_dtype=kv_cache_dtype)


def config1(device="cuda", seed=0) -> Workload:
    """v1, S=8, 32/32 heads, D=128, B=16, bf16, lens U{1..1024}, NB=4096, per-row sample."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, 1025, size=8)
    return make_decode("cfg1_v1_mha_s8", num_seqs=8, num_heads=32, num_kv_heads=32, head_size=128,
                       block_size=16, lens=lens, dtype=torch.bfloat16, kv_cache_dtype="auto",
                       device=device, seed=seed, rng=rng, num_blocks=4096, unique_global=False)


def config2(device="cuda", seed=0, num_seqs=256, rank=0) -> Workload:
    """v2 GQA decode at Llama-3-8B shape: S=256, 32/8 heads, D=128, B=16, bf16,
    lens U{512..4096}; blocks = one global permutation over 1.25x the needed blocks."""
    rng = np.random.default_rng(seed + 1000 * rank)
    lens = rng.integers(512, 4097, size=num_seqs)
    return make_decode("cfg2_v2_llama3_8b_s256", num_seqs=num_seqs, num_heads=32, num_kv_heads=8,
                       head_size=128, block_size=16, lens=lens, dtype=torch.bfloat16,
                       kv_cache_dtype="auto", device=device, seed=seed + rank, rng=rng,
                       max_seq_len=4096)


def config3(device="cuda", seed=0, num_seqs=128, seq_len=8192, new_tokens=128) -> Workload:
    """fp8-e4m3 KV at Llama-3-70B per-layer shape: reshape_and_cache writes the last
    `new_tokens` positions of every sequence, then v2 with 64/8 heads."""
    rng = np.random.default_rng(seed)
    lens = np.full(num_seqs, seq_len, dtype=np.int64)
    w = make_decode("cfg3_fp8_llama3_70b_s128", num_seqs=num_seqs, num_heads=64, num_kv_heads=8,
                    head_size=128, block_size=16, lens=lens, dtype=torch.bfloat16,
                    kv_cache_dtype="fp8", device=device, seed=seed, rng=rng)
    dev = w.query.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 7)
    T = num_seqs * new_tokens
    nk = torch.empty((T, 8, 128), dtype=torch.float32, device=dev).normal_(0, 1, generator=gen)
    nv = torch.empty((T, 8, 128), dtype=torch.float32, device=dev).normal_(0, 1, generator=gen)
    w.new_key = nk.to(torch.bfloat16)
    w.new_value = nv.to(torch.bfloat16)
    w.k_scale = (w.new_key.float().abs().amax() / 448.0).reshape(())
    w.v_scale = (w.new_value.float().abs().amax() / 448.0).reshape(())
    pos = torch.arange(seq_len - new_tokens, seq_len, device=dev)
    bt = w.block_tables.long()
    slots = bt[:, pos // w.block_size] * w.block_size + (pos % w.block_size).view(1, -1)
    w.slot_mapping = slots.reshape(-1).contiguous()
    return w


def config4(device="cuda", seed=0, world_size=1, rank=0) -> Workload:
    """long-context skewed decode: S=64, 32/8 heads, bf16, lens lognormal(8.5,1.0)
    clipped to [16,32768]; KV heads sharded over `world_size` ranks."""
    rng = np.random.default_rng(seed)
    lens = np.clip(np.round(rng.lognormal(8.5, 1.0, size=64)), 16, 32768).astype(np.int64)
    hkv = 8 // world_size
    return make_decode(f"cfg4_longctx_s64_tp{world_size}", num_seqs=64, num_heads=4 * hkv,
                       num_kv_heads=hkv, head_size=128, block_size=16, lens=lens,
                       dtype=torch.bfloat16, kv_cache_dtype="auto", device=device,
                       seed=seed + rank, rng=rng, max_seq_len=32768)


def config5(device="cuda", seed=0, world_size=1, rank=0, num_seqs=2048) -> Workload:
    """large-batch serving decode: S=2048, 64/8 heads, B=32, fp8, lens U{1024..8192};
    sequences sharded over `world_size` ranks with local block pools."""
    rng = np.random.default_rng(seed)
    lens_all = rng.integers(1024, 8193, size=num_seqs)
    per = num_seqs // world_size
    lens = lens_all[rank * per:(rank + 1) * per]
    rng_local = np.random.default_rng(seed + 17 * (rank + 1))
    return make_decode(f"cfg5_serving_s{num_seqs}_dp{world_size}", num_seqs=per, num_heads=64,
                       num_kv_heads=8, head_size=128, block_size=32, lens=lens,
                       dtype=torch.bfloat16, kv_cache_dtype="fp8", device=device,
                       seed=seed + rank, rng=rng_local, max_seq_len=8192)


def small(device="cuda", seed=0, *, num_seqs=7, num_heads=8, num_kv_heads=2, head_size=128,
          block_size=16, max_len=700, dtype=torch.bfloat16, kv_cache_dtype="auto",
          num_blocks=512) -> Workload:
    """A small ragged case for smoke checks and unit tests."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, max_len + 1, size=num_seqs)
    lens[-1] = max_len
    return make_decode("small", num_seqs=num_seqs, num_heads=num_heads, num_kv_heads=num_kv_heads,
                       head_size=head_size, block_size=block_size, lens=lens, dtype=dtype,
                       kv_cache_dtype=kv_cache_dtype, device=device, seed=seed, rng=rng,
                       num_blocks=num_blocks, unique_global=False)


def run_attention(w: Workload, out: torch.Tensor | None = None, version: str = "v2",
                  scratch=None) -> torch.Tensor:
    """Calls the op through the reference-shaped wrapper."""
    from vllm_b200 import _custom_ops as ops

    if out is None:
        out = torch.empty_like(w.query)
    if version == "v1":
        ops.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                               w.block_tables, w.seq_lens, w.block_size, w.max_seq_len,
                               w.alibi_slopes, w.kv_cache_dtype, w.k_scale, w.v_scale)
    else:
        exp_sums, max_logits, tmp_out = scratch if scratch is not None else w.scratch()
        ops.paged_attention_v2(out, exp_sums, max_logits, tmp_out, w.query, w.key_cache,
                               w.value_cache, w.num_kv_heads, w.scale, w.block_tables, w.seq_lens,
                               w.block_size, w.max_seq_len, w.alibi_slopes, w.kv_cache_dtype,
                               w.k_scale, w.v_scale)
    return out


def shard_kv_heads(w: Workload, world_size: int, rank: int) -> Workload:
    """Rank `rank`'s share of `w` when KV heads are partitioned: `Hkv/world_size` kv heads of
    every block and the query heads that map to them (kv_head = head // G); block tables and
    seq_lens are replicated.  The slices are copies, so each rank holds only its own shard."""
    assert w.num_kv_heads % world_size == 0
    hk = w.num_kv_heads // world_size
    g = w.num_heads // w.num_kv_heads
    ks, qs = slice(rank * hk, (rank + 1) * hk), slice(rank * hk * g, (rank + 1) * hk * g)
    return dataclasses.replace(
        w, name=f"{w.name}/kvheads{rank}of{world_size}", query=w.query[:, qs].contiguous(),
        key_cache=w.key_cache[:, ks].contiguous(), value_cache=w.value_cache[:, ks].contiguous(),
        num_kv_heads=hk,
        alibi_slopes=None if w.alibi_slopes is None else w.alibi_slopes[qs].contiguous())


def shard_sequences(w: Workload, world_size: int, rank: int) -> Workload:
    """Rank `rank`'s share of `w` when sequences are partitioned: `S/world_size` sequences with a
    private block pool holding only their blocks, block ids renumbered locally."""
    assert w.num_seqs % world_size == 0
    per = w.num_seqs // world_size
    ss = slice(rank * per, (rank + 1) * per)
    lens = w.seq_lens[ss].cpu().numpy().astype(np.int64)
    need = np.ceil(lens / w.block_size).astype(np.int64)
    bt = w.block_tables[ss].cpu().numpy()
    used = np.concatenate([bt[s, :need[s]] for s in range(per)]) if per else np.zeros(0, np.int64)
    uniq, inv = np.unique(used, return_inverse=True)
    if uniq.size == 0:
        uniq = np.zeros(1, dtype=np.int64)
    local = np.zeros_like(bt)
    off = 0
    for s in range(per):
        local[s, :need[s]] = inv[off:off + need[s]]
        off += need[s]
    idx = torch.from_numpy(uniq.astype(np.int64)).to(w.key_cache.device)
    return dataclasses.replace(
        w, name=f"{w.name}/seqs{rank}of{world_size}", query=w.query[ss].contiguous(),
        key_cache=w.key_cache[idx].contiguous(), value_cache=w.value_cache[idx].contiguous(),
        block_tables=torch.from_numpy(local).to(w.block_tables.device),
        seq_lens=w.seq_lens[ss].contiguous())


def token_ranges(seq_lens, block_size: int, world_size: int, rank: int):
    """Block range [b0, b1) and token count of rank `rank` for every sequence when the tokens
    of each sequence are partitioned across ranks at block boundaries (contiguous ranges of
    ceil-divided blocks; the last non-empty range carries the ragged tail).  Pure host logic."""
    lens = np.asarray(seq_lens, dtype=np.int64)
    nblk = (lens + block_size - 1) // block_size
    per = (nblk + world_size - 1) // world_size
    b0 = np.minimum(nblk, rank * per)
    b1 = np.minimum(nblk, (rank + 1) * per)
    toks = np.clip(np.minimum(lens, b1 * block_size) - b0 * block_size, 0, None)
    return b0, b1, toks


def shard_tokens(w: Workload, world_size: int, rank: int) -> Workload:
    """Rank `rank`'s share of `w` when the KV tokens of every sequence are partitioned across
    ranks (decode context parallelism): a private block pool with only this rank's blocks, block
    tables and seq_lens rewritten for the local token range; the query is replicated.  Attention
    over the shards is combined with `context_parallel.merge_partials` (needs the LSE output).
    ALiBi is not supported here (its bias depends on the global position)."""
    assert w.alibi_slopes is None
    lens = w.seq_lens.cpu().numpy().astype(np.int64)
    b0, b1, toks = token_ranges(lens, w.block_size, world_size, rank)
    bt = w.block_tables.cpu().numpy()
    S = w.num_seqs
    used = np.concatenate([bt[s, b0[s]:b1[s]] for s in range(S)]) if S else np.zeros(0, np.int64)
    uniq, inv = np.unique(used, return_inverse=True)
    if uniq.size == 0:
        uniq = np.zeros(1, dtype=np.int64)
    local = np.zeros((S, max(1, int((b1 - b0).max()) if S else 1)), dtype=bt.dtype)
    off = 0
    for s in range(S):
        n = int(b1[s] - b0[s])
        local[s, :n] = inv[off:off + n]
        off += n
    idx = torch.from_numpy(uniq.astype(np.int64)).to(w.key_cache.device)
    return dataclasses.replace(
        w, name=f"{w.name}/tokens{rank}of{world_size}",
        key_cache=w.key_cache[idx].contiguous(), value_cache=w.value_cache[idx].contiguous(),
        block_tables=torch.from_numpy(local).to(w.block_tables.device),
        seq_lens=torch.from_numpy(toks.astype(np.int32)).to(w.seq_lens.device),
        max_seq_len=max(1, int(toks.max()) if S else 1))
