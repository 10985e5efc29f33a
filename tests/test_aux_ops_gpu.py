"""GPU parity of the operators next to the decode path: merge_attn_states,
copy_blocks, swap_blocks.  Modelled on the reference's
tests/kernels/attention/test_merge_attn_states.py and test_cache.py
(test_copy_blocks :53-126, test_swap_blocks :413-470)."""
import numpy as np
import pytest
import torch

from oracle import paged_oracle as O
from vllm_b200 import _custom_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("num_tokens", [1, 39, 512])
@pytest.mark.parametrize("heads_size", [(4, 32), (16, 128), (9, 96), (8, 256)])
@pytest.mark.parametrize("with_lse", [True, False])
def test_merge_attn_states(dtype, num_tokens, heads_size, with_lse):
    H, D = heads_size
    g = torch.Generator(device=DEV).manual_seed(0)
    p = torch.randn(num_tokens, H, D, device=DEV, generator=g).to(dtype)
    s = torch.randn(num_tokens, H, D, device=DEV, generator=g).to(dtype)
    pl = torch.randn(H, num_tokens, device=DEV, generator=g) * 3
    sl = torch.randn(H, num_tokens, device=DEV, generator=g) * 3
    # the special cases of the reference: +inf and -inf entries, and both dead
    mask = torch.rand(H, num_tokens, device=DEV, generator=g)
    pl[mask < 0.05] = float("inf")
    sl[(mask > 0.05) & (mask < 0.10)] = float("-inf")
    both = mask > 0.97
    pl[both] = float("-inf")
    sl[both] = float("inf")
    out = torch.full_like(p, float("nan"))
    lse = torch.full((H, num_tokens), float("nan"), device=DEV) if with_lse else None
    ops.merge_attn_states(out, p, pl, s, sl, lse)
    want, want_lse = O.merge_attn_states(p.cpu(), pl.cpu(), s.cpu(), sl.cpu())
    # same formula in fp32; expf/logf may differ from the host's by an ulp
    # 16-bit outputs: two ulps of the output type (the rounding input differs by fp32 noise)
    tol = dict(atol=1e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-4, rtol=1.6e-2)
    torch.testing.assert_close(out.cpu().float(), want.float(), **tol)
    if with_lse:
        torch.testing.assert_close(lse.cpu(), want_lse, atol=1e-5, rtol=1e-5, equal_nan=True)


def test_merge_attn_states_rejects_bad_head_size():
    p = torch.zeros(2, 2, 12, device=DEV, dtype=torch.bfloat16)  # 12 is not a multiple of 8
    l = torch.zeros(2, 2, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of pack_size"):
        ops.merge_attn_states(torch.empty_like(p), p, l, p, l)


@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("num_layers", [1, 3, 70])
@pytest.mark.parametrize("block_size", [8, 16])
def test_copy_blocks(kv, num_layers, block_size):
    NB, H, D = 200, 4, 64
    cdt = torch.uint8 if kv == "fp8" else torch.bfloat16
    x = 16 // (1 if kv == "fp8" else 2)
    g = torch.Generator(device=DEV).manual_seed(1)
    mk = lambda shape: torch.randint(0, 200, shape, device=DEV, generator=g).to(cdt)
    kcs = [mk((NB, H, D // x, block_size, x)) for _ in range(num_layers)]
    vcs = [mk((NB, H, D, block_size)) for _ in range(num_layers)]
    rng = np.random.default_rng(1)
    srcs = rng.choice(NB // 2, size=20, replace=False)
    dsts = NB // 2 + rng.choice(NB // 2, size=40, replace=False)
    pairs = [(int(srcs[i // 2]), int(dsts[i])) for i in range(40)]  # each source copied twice
    bm = torch.tensor(pairs, dtype=torch.int64, device=DEV)
    wk = [k.cpu().clone() for k in kcs]
    wv = [v.cpu().clone() for v in vcs]
    O.copy_blocks(wk, wv, bm.cpu())
    ops.copy_blocks(kcs, vcs, bm)
    for a, b in zip(kcs + vcs, wk + wv):
        assert torch.equal(a.cpu(), b)


@pytest.mark.parametrize("direction", [("cuda", "cpu"), ("cpu", "cuda"), ("cuda", "cuda")])
@pytest.mark.parametrize("kv", ["auto", "fp8"])
def test_swap_blocks(direction, kv):
    NB, H, D, B = 64, 4, 64, 16
    cdt = torch.uint8 if kv == "fp8" else torch.bfloat16
    src_dev, dst_dev = direction
    g = torch.Generator().manual_seed(2)
    mk = lambda dev: torch.randint(0, 200, (NB, H, D, B), generator=g).to(cdt).to(dev)
    src, dst = mk(src_dev), mk(dst_dev)
    if src_dev == "cpu":
        src = src.pin_memory()
    if dst_dev == "cpu":
        dst = dst.pin_memory()
    rng = np.random.default_rng(2)
    pairs = list(zip(rng.choice(NB, 20, replace=False).tolist(), rng.choice(NB, 20, replace=False).tolist()))
    bm = torch.tensor(pairs, dtype=torch.int64, device="cpu")
    want = dst.cpu().clone()
    O.swap_blocks(src.cpu(), want, bm)
    ops.swap_blocks(src, dst, bm)
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), want)
    with pytest.raises(RuntimeError, match="block_mapping must be on CPU"):
        ops.swap_blocks(src, dst, bm.to(DEV))
