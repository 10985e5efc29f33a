"""GPU parity of reshape_and_cache / reshape_and_cache_flash / convert_fp8:
bit-exact against the CPU oracle and the reference's CUDA kernels.  Case matrix
modelled on tests/kernels/attention/test_cache.py:129-410 of the reference."""
import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200 import _custom_ops as ops
from vllm_b200 import capi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _slots(rng, T, total, runs=True):
    s = rng.permutation(total)[:T].astype(np.int64)
    if runs and T >= 40:
        # a few runs of consecutive slots (whole blocks and ragged pieces)
        base = (total // 2 // 32) * 32
        run = np.arange(base, base + 37, dtype=np.int64)
        rest = np.setdiff1d(rng.permutation(total), run)[:T - 37]
        s = np.concatenate([rest[:3], run, rest[3:]])
    s[1] = -1
    return s


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("kv", ["auto", "fp8", "fp8_e5m2"])
@pytest.mark.parametrize("head_size", [64, 80, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_reshape_and_cache_bit_exact(dtype, kv, head_size, block_size, ref_cuda_ops):
    if kv != "auto" and head_size % 16:
        pytest.skip("fp8 caches need head_size % 16 == 0")
    T, H, NB = 123, 8, 96
    rng = np.random.default_rng(0)
    g = torch.Generator(device=DEV).manual_seed(0)
    key = torch.randn(T, H, head_size, device=DEV, generator=g).mul(3).to(dtype)
    val = torch.randn(T, H, head_size, device=DEV, generator=g).mul(3).to(dtype)
    key[0, 0, 0] = float("nan")
    val[2, 1, 3] = float("inf")
    slots = torch.from_numpy(_slots(rng, T, NB * block_size)).to(DEV)
    fp8 = kv != "auto"
    cdt = torch.uint8 if fp8 else dtype
    x = 16 // (1 if fp8 else key.element_size())
    ks = (key.float().nan_to_num(0, 0, 0).abs().amax() / 64.0).reshape(())
    vs = (val.float().nan_to_num(0, 0, 0).abs().amax() / 64.0).reshape(())
    kc = torch.zeros(NB, H, head_size // x, block_size, x, dtype=cdt, device=DEV)
    vc = torch.zeros(NB, H, head_size, block_size, dtype=cdt, device=DEV)
    ops.reshape_and_cache(key, val, kc, vc, slots, kv, ks, vs)
    kco, vco = torch.zeros_like(kc, device="cpu"), torch.zeros_like(vc, device="cpu")
    O.reshape_and_cache(key.cpu(), val.cpu(), kco, vco, slots.cpu(), kv, float(ks), float(vs))
    same = lambda a, b: torch.equal(a.cpu().view(torch.uint8), b.cpu().view(torch.uint8))
    assert same(kc, kco) and same(vc, vco)
    if ref_cuda_ops is not None:
        kcr, vcr = torch.zeros_like(kc), torch.zeros_like(vc)
        ref_cuda_ops[1].reshape_and_cache(key, val, kcr, vcr, slots, kv, ks, vs)
        assert same(kc, kcr) and same(vc, vcr)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("head_size", [64, 80, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_reshape_and_cache_flash_bit_exact(dtype, kv, layout, head_size, block_size, ref_cuda_ops):
    T, H, NB = 77, 8, 64
    rng = np.random.default_rng(1)
    g = torch.Generator(device=DEV).manual_seed(1)
    # key has more rows than slot_mapping (padding for CUDA graphs) and a padded row stride
    pad = torch.randn(T + 5, H * head_size + 16, device=DEV, generator=g).to(dtype)
    key = pad[:, :H * head_size].view(T + 5, H, head_size)
    val = torch.randn(T + 5, H, head_size, device=DEV, generator=g).to(dtype)
    slots = torch.from_numpy(_slots(rng, T, NB * block_size, runs=False)).to(DEV)
    fp8 = kv != "auto"
    cdt = torch.uint8 if fp8 else dtype
    ks = torch.tensor(0.037, device=DEV)
    vs = torch.tensor(0.051, device=DEV)

    def mk():
        if layout == "NHD":
            a = torch.zeros(NB, block_size, H, head_size, dtype=cdt, device=DEV)
            b = torch.zeros_like(a)
            return a, b
        a = torch.zeros(NB, H, block_size, head_size, dtype=cdt, device=DEV)
        b = torch.zeros_like(a)
        return a.permute(0, 2, 1, 3), b.permute(0, 2, 1, 3)

    kc, vc = mk()
    ops.reshape_and_cache_flash(key, val, kc, vc, slots, kv, ks, vs)
    kco, vco = torch.zeros(kc.shape, dtype=cdt), torch.zeros(vc.shape, dtype=cdt)
    O.reshape_and_cache_flash(key.cpu(), val.cpu(), kco, vco, slots.cpu(), kv, float(ks), float(vs))
    same = lambda a, b: torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
    assert same(kc, kco) and same(vc, vco)
    if ref_cuda_ops is not None:
        kcr, vcr = mk()
        ref_cuda_ops[1].reshape_and_cache_flash(key, val, kcr, vcr, slots, kv, ks, vs)
        assert same(kc, kcr) and same(vc, vcr)


def test_fp8_quantiser_exhaustive_on_device(ref_cuda_ops):
    """Every bf16 bit pattern through the device quantiser == oracle == reference."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.bfloat16).to(DEV)
    for kv in ("fp8", "fp8_e5m2"):
        for scale in (1.0, 0.011826, 3.7):
            dst = torch.empty(65536, dtype=torch.uint8, device=DEV)
            ops.convert_fp8(dst, x, scale, kv)
            want = O.quantize_fp8(x.cpu(), scale, kv)
            assert torch.equal(dst.cpu(), want), (kv, scale)
            if ref_cuda_ops is not None and kv == "fp8":
                r = torch.empty_like(dst)
                ref_cuda_ops[1].convert_fp8(r.view(1, -1), x.view(1, -1), scale, kv)
                assert torch.equal(r, dst)


def test_convert_fp8_round_trip():
    """reference tests/kernels/attention/test_cache.py:514-545"""
    g = torch.Generator(device=DEV).manual_seed(2)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        x = torch.empty(4, 1024, device=DEV).uniform_(-224, 224, generator=g).to(dtype)
        q = torch.empty_like(x, dtype=torch.uint8)
        ops.convert_fp8(q, x)
        y = torch.empty_like(x)
        ops.convert_fp8(y, q)
        torch.testing.assert_close(x, y, atol=1e-3, rtol=0.25)
        want = O.dequantize_fp8(q.cpu(), 1.0, dtype)
        assert torch.equal(y.cpu(), want)


def test_write_then_attend_uses_the_written_tokens():
    """reshape_and_cache -> paged_attention_v2 on the same cache (the decode step)."""
    import workloads as W
    w = W.config3(DEV, num_seqs=4, seq_len=1024, new_tokens=128)
    ops.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping, "fp8",
                          w.k_scale, w.v_scale)
    kc, vc = w.key_cache.cpu().clone(), w.value_cache.cpu().clone()
    out = W.run_attention(w, version="v2").cpu()
    want = O.paged_attention(w.query.cpu(), kc, vc, w.num_kv_heads, w.scale, w.block_tables.cpu(),
                             w.seq_lens.cpu(), None, "fp8", float(w.k_scale), float(w.v_scale), mode="f64")
    torch.testing.assert_close(out.double(), want, atol=2e-2, rtol=2e-2)
    # the last 128 positions of sequence 0 hold exactly the quantised new tokens
    k0, _ = O.gather_kv(kc, vc, w.block_tables.cpu()[0], 1024, "fp8", 1.0, 1.0, torch.float32)
    qk = O.quantize_fp8(w.new_key[:128].cpu(), float(w.k_scale), "fp8").view(torch.float8_e4m3fn).float()
    assert torch.equal(k0[-128:], qk)


def test_fp8_quantiser_fp32_inputs_ties_and_odd_scales():
    """The quantiser must give the bits of cvt(x / scale) with an IEEE division for arbitrary
    fp32 inputs: random bit patterns (specials included), inputs built to sit on and next to
    fp8 rounding ties, and awkward scales (a reciprocal multiply would fail here)."""
    g = torch.Generator().manual_seed(3)
    n = 1 << 21
    rand_bits = torch.randint(-(1 << 31), (1 << 31) - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32)
    x_rand = rand_bits.view(torch.float32)
    x_norm = torch.randn(n, generator=g) * 3
    scales = [1.0, 0.011826, 3.7, 1 / 3, 5.3 / 448, 2.0 ** -20, 1.0000001, 0.9999999, 123456.7,
              float(torch.rand(1, generator=g)) + 1e-3,
              # significand of all ones, and both sides of the range in which the kernel replaces
              # the division by reciprocal + residual corrections; a denormal scale
              1.9999999, 1.9999999 * 2.0 ** -30, 2.0 ** -60, 2.0 ** -61, 2.0 ** 60, 2.0 ** 61,
              1e-38, 1e-40, 3e38]
    for kv in ("fp8", "fp8_e5m2"):
        dt, fmax = O.FP8_FORMATS[kv]
        # every finite fp8 value and the midpoints between neighbours, times the scale, +- a few ulps
        codes = torch.arange(256, dtype=torch.int16).to(torch.uint8).view(dt).float()
        vals = torch.sort(codes[torch.isfinite(codes)]).values
        mids = (vals[1:] + vals[:-1]) / 2
        for scale in scales:
            s32 = torch.tensor(scale, dtype=torch.float32)
            base = torch.cat([mids, vals]) * s32
            near = torch.cat([torch.nextafter(base, torch.tensor(float("inf"))),
                              torch.nextafter(base, torch.tensor(-float("inf"))), base])
            for _ in range(2):
                near = torch.cat([near, torch.nextafter(near, torch.tensor(float("inf"))),
                                  torch.nextafter(near, torch.tensor(-float("inf")))])
            x = torch.cat([near, x_norm * s32 * 100, x_rand])
            dst = torch.empty(x.numel(), dtype=torch.uint8, device=DEV)
            ops.convert_fp8(dst, x.to(DEV), float(s32), kv)
            want = O.quantize_fp8(x, float(s32), kv)
            bad = torch.nonzero(dst.cpu() != want).flatten()
            assert bad.numel() == 0, (kv, scale, bad.numel(), x[bad[:4]].tolist(),
                                      dst.cpu()[bad[:4]].tolist(), want[bad[:4]].tolist())


@pytest.mark.parametrize("seed", range(40))
def test_reshape_and_cache_random_shapes_and_slot_patterns(seed):
    """Seeded random draws: token counts around the 16-token tile, head counts and sizes that make
    the per-token item count smaller or larger than a CTA, prefill-like consecutive slots (the
    transposing fast path), decode-like scattered slots, padding tokens, both layouts."""
    rng = np.random.default_rng(500 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][int(rng.integers(3))]
    kv = ["auto", "fp8", "fp8_e5m2"][int(rng.integers(3))]
    fp8 = kv != "auto"
    block_size = int(rng.choice([8, 16, 32]))
    H = int(rng.choice([1, 2, 3, 8, 16]))
    head_size = int(rng.choice([32, 64, 128, 256]))
    T = int(rng.choice([1, 15, 16, 17, 31, 48, 100, 257]))
    NB = (T + block_size - 1) // block_size + 40
    pattern = int(rng.integers(3))
    if pattern == 0:    # prefill: consecutive slots from a block boundary
        start = int(rng.integers(0, 20)) * block_size
        slots = np.arange(start, start + T, dtype=np.int64)
    elif pattern == 1:  # decode: scattered
        slots = rng.permutation(NB * block_size)[:T].astype(np.int64)
    else:               # chunks of consecutive slots at odd offsets, with padding tokens
        slots = np.full(T, -1, dtype=np.int64)
        pos, t = int(rng.integers(0, 7)), 0
        while t < T:
            n = int(min(T - t, rng.integers(1, 40)))
            slots[t:t + n] = np.arange(pos, pos + n)
            pos += n + int(rng.integers(0, 50))
            t += n + int(rng.integers(0, 3))
        slots = np.where(slots >= NB * block_size, -1, slots)
    g = torch.Generator(device=DEV).manual_seed(seed)
    key = torch.randn(T, H, head_size, device=DEV, generator=g).mul(2).to(dtype)
    val = torch.randn(T, H, head_size, device=DEV, generator=g).mul(2).to(dtype)
    slots_t = torch.from_numpy(slots).to(DEV)
    ks = torch.tensor(float(rng.choice([1.0, 0.0173, 0.37, 2.0 ** -61])), device=DEV)
    vs = torch.tensor(float(rng.choice([1.0, 0.0291, 0.11])), device=DEV)
    cdt = torch.uint8 if fp8 else dtype
    same = lambda a, b: torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
    # x layout
    x = 16 // (1 if fp8 else key.element_size())
    kc = torch.zeros(NB, H, head_size // x, block_size, x, dtype=cdt, device=DEV)
    vc = torch.zeros(NB, H, head_size, block_size, dtype=cdt, device=DEV)
    ops.reshape_and_cache(key, val, kc, vc, slots_t, kv, ks, vs)
    kco, vco = torch.zeros_like(kc, device="cpu"), torch.zeros_like(vc, device="cpu")
    O.reshape_and_cache(key.cpu(), val.cpu(), kco, vco, slots_t.cpu(), kv, float(ks), float(vs))
    assert same(kc, kco) and same(vc, vco), ("x layout", dtype, kv, block_size, H, head_size, T, pattern)
    # flash layout
    kf = torch.zeros(NB, block_size, H, head_size, dtype=cdt, device=DEV)
    vf = torch.zeros_like(kf)
    ops.reshape_and_cache_flash(key, val, kf, vf, slots_t, kv, ks, vs)
    kfo, vfo = torch.zeros(kf.shape, dtype=cdt), torch.zeros(vf.shape, dtype=cdt)
    O.reshape_and_cache_flash(key.cpu(), val.cpu(), kfo, vfo, slots_t.cpu(), kv, float(ks), float(vs))
    assert same(kf, kfo) and same(vf, vfo), ("flash layout", dtype, kv, block_size, H, head_size, T, pattern)


@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("block_size", [16, 32])
def test_prefill_chunks_that_start_inside_a_block(kv, block_size):
    """A large write whose sequences start at arbitrary offsets inside their first block (the
    continuation of earlier context): 16-token tiles that straddle cache blocks, runs of every
    length that follow each other, some tokens padding."""
    rng = np.random.default_rng(77 + block_size)
    H, D = 8, 128
    lens = [300, 17, 16, 15, 1, 700, 33, 64, 5, 2, 1000, 31, 48, 260, 129, 500, 1029]
    starts, slots, pos = [], [], 0
    for n in lens:
        pos = (pos + block_size - 1) // block_size * block_size + int(rng.integers(0, block_size))
        slots.append(np.arange(pos, pos + n, dtype=np.int64))
        pos += n + int(rng.integers(0, 3)) * block_size
        if rng.integers(0, 3) == 0:
            slots.append(np.full(int(rng.integers(1, 20)), -1, dtype=np.int64))
    slots = np.concatenate(slots)
    T = len(slots)
    NB = int(slots.max()) // block_size + 2
    fp8 = kv != "auto"
    g = torch.Generator(device=DEV).manual_seed(9)
    key = torch.randn(T, H, D, device=DEV, generator=g).mul(2).to(torch.bfloat16)
    val = torch.randn(T, H, D, device=DEV, generator=g).mul(2).to(torch.bfloat16)
    slots_t = torch.from_numpy(slots).to(DEV)
    ks, vs = torch.tensor(0.0173, device=DEV), torch.tensor(0.0291, device=DEV)
    cdt = torch.uint8 if fp8 else torch.bfloat16
    x = 16 // (1 if fp8 else 2)
    kc = torch.zeros(NB, H, D // x, block_size, x, dtype=cdt, device=DEV)
    vc = torch.zeros(NB, H, D, block_size, dtype=cdt, device=DEV)
    for _ in range(2):  # (twice: the second call overwrites with the same bytes)
        ops.reshape_and_cache(key, val, kc, vc, slots_t, kv, ks, vs)
    kco, vco = torch.zeros_like(kc, device="cpu"), torch.zeros_like(vc, device="cpu")
    O.reshape_and_cache(key.cpu(), val.cpu(), kco, vco, slots_t.cpu(), kv, float(ks), float(vs))
    same = lambda a, b: torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
    assert same(kc, kco), "key cache"
    assert same(vc, vco), "value cache"
    assert capi.device_status() == 0


@pytest.mark.parametrize("seed", range(16))
def test_large_mixed_batches_of_chunks_and_single_tokens(seed):
    """Large writes (the size range in which tiles are moved onto 16-slot boundaries) made of
    prefill chunks of random length at random offsets, single decode tokens and padding, in
    random order, with random head counts and sizes: every token lands in its own slot."""
    rng = np.random.default_rng(9000 + seed)
    block_size = int(rng.choice([16, 32]))
    H = int(rng.choice([1, 3, 8]))
    D = int(rng.choice([64, 128, 256]))
    kv = ["auto", "fp8", "fp8_e5m2"][int(rng.integers(3))]
    dtype = [torch.bfloat16, torch.float16][int(rng.integers(2))]
    target = int(rng.choice([4096, 4500, 7000, 10000]))
    pieces, free = [], 0  # slots are handed out in increasing order, with gaps: no duplicates
    total = 0
    while total < target:
        kind = int(rng.integers(4))
        if kind == 0:      # a decode token somewhere
            free += int(rng.integers(1, 5 * block_size))
            pieces.append(np.array([free], dtype=np.int64))
            free += 1
        elif kind == 1:    # padding
            pieces.append(np.full(int(rng.integers(1, 9)), -1, dtype=np.int64))
        else:              # a chunk of consecutive positions starting anywhere in a block
            n = int(rng.integers(1, 400))
            free += int(rng.integers(0, 3 * block_size))
            pieces.append(np.arange(free, free + n, dtype=np.int64))
            free += n
        total += len(pieces[-1])
    order = rng.permutation(len(pieces))
    slots = np.concatenate([pieces[i] for i in order])
    T = len(slots)
    NB = free // block_size + 2
    fp8 = kv != "auto"
    g = torch.Generator(device=DEV).manual_seed(seed)
    key = torch.randn(T, H, D, device=DEV, generator=g).mul(2).to(dtype)
    val = torch.randn(T, H, D, device=DEV, generator=g).mul(2).to(dtype)
    slots_t = torch.from_numpy(slots).to(DEV)
    ks, vs = torch.tensor(0.0173, device=DEV), torch.tensor(0.11, device=DEV)
    cdt = torch.uint8 if fp8 else dtype
    x = 16 // (1 if fp8 else 2)
    kc = torch.zeros(NB, H, D // x, block_size, x, dtype=cdt, device=DEV)
    vc = torch.zeros(NB, H, D, block_size, dtype=cdt, device=DEV)
    ops.reshape_and_cache(key, val, kc, vc, slots_t, kv, ks, vs)
    kco, vco = torch.zeros_like(kc, device="cpu"), torch.zeros_like(vc, device="cpu")
    O.reshape_and_cache(key.cpu(), val.cpu(), kco, vco, slots_t.cpu(), kv, float(ks), float(vs))
    same = lambda a, b: torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))
    assert same(kc, kco), ("key cache", block_size, H, D, kv, dtype, T)
    assert same(vc, vco), ("value cache", block_size, H, D, kv, dtype, T)
    assert capi.device_status() == 0


@pytest.mark.parametrize("knobs", [
    {"B200PA_TUNE_KVW_STAGED": "0"},
    {"B200PA_TUNE_KVW_STAGED": "1", "B200PA_TUNE_KVW_HSPLIT": "1", "B200PA_TUNE_KVW_SHIFT": "0"},
    {"B200PA_TUNE_KVW_STAGED": "1", "B200PA_TUNE_KVW_HSPLIT": "2", "B200PA_TUNE_KVW_SHIFT": "0"},
    {"B200PA_TUNE_KVW_STAGED": "1", "B200PA_TUNE_KVW_HSPLIT": "1", "B200PA_TUNE_KVW_SHIFT": "1"},
    {"B200PA_TUNE_KVW_STAGED": "1", "B200PA_TUNE_KVW_HSPLIT": "2", "B200PA_TUNE_KVW_SHIFT": "1"},
], ids=["plain", "staged-whole-heads", "staged-half-heads", "staged-whole-heads-moved-tiles",
        "staged-half-heads-moved-tiles"])
def test_both_kv_write_implementations(knobs):
    """The library has two implementations of the KV write (plain loads; rows staged through
    shared memory by bulk async copies, with a whole head or half a head of 128 per work item)
    and picks per call by layout, cache type and size; large x-layout writes use a variant that
    moves 16-token tiles onto 16-slot boundaries of the cache.  B200PA_TUNE_KVW_STAGED / _HSPLIT
    / _SHIFT force one setting for every call that it can take; they are read once per process, so the parity tests of
    this file run again in a child process for each setting."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, **knobs)
    r = subprocess.run(
        [sys.executable, "-m", "pytest", str(Path(__file__)), "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
         "-k", "not both_kv_write", str(root / "tests" / "test_full_size_gpu.py") + "::test_full_size_kv_write_round_trip"],
        env=env, cwd=str(root), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
