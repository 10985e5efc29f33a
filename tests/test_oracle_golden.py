"""Pins the CPU oracle against fixtures produced by the reference's own code
(tests/golden/*.npz; generating scripts beside them)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import paged_oracle as O

GOLD = Path(__file__).parent / "golden"


def _all_bf16():
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    return bits.view(torch.bfloat16)


@pytest.mark.parametrize("fmt,key", [("fp8_e4m3", "e4m3"), ("fp8_e5m2", "e5m2")])
def test_quantiser_matches_nvidia_host_conversion(fmt, key):
    g = np.load(GOLD / "fp8_golden.npz")
    x = _all_bf16()
    for i, scale in enumerate(g["scales"].tolist()):
        got = O.quantize_fp8(x, scale, fmt).numpy()
        want = g[key][i]
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, f"{fmt} scale={scale}: {bad.size} mismatches, first bf16 bits {bad[:5]}"


def test_quantiser_rounding_and_saturation_known_answers():
    # e4m3: RNE at the 3-bit mantissa, saturate to +-448, NaN -> 0x7F
    x = torch.tensor([17.0, 19.0, 21.0, 460.0, 1e9, -1e9, float("inf"), float("-inf"), 0.0],
                     dtype=torch.float32)
    got = O.quantize_fp8(x, 1.0, "fp8").view(torch.float8_e4m3fn).float().tolist()
    assert got == [16.0, 20.0, 20.0, 448.0, 448.0, -448.0, 448.0, -448.0, 0.0]
    nan = O.quantize_fp8(torch.tensor([float("nan"), -float("nan")]), 1.0, "fp8").tolist()
    assert nan == [0x7F, 0x7F]


def test_dequantise_is_exact_inverse_on_codes():
    codes = torch.arange(256, dtype=torch.int16).to(torch.uint8)
    finite = codes[(codes & 0x7F) != 0x7F]
    back = O.quantize_fp8(O.dequantize_fp8(finite, 1.0, torch.float32, "fp8"), 1.0, "fp8")
    # -0 and +0 keep their sign bit
    assert torch.equal(back, finite)


def _paged_from_flash(kf, vf):
    """flash logical [NB,B,H,D] -> x-layout caches used by paged_attention."""
    nb, b, h, d = kf.shape
    x = 16 // kf.element_size()
    kc = kf.permute(0, 2, 3, 1).reshape(nb, h, d // x, x, b).permute(0, 1, 2, 4, 3).contiguous()
    vc = vf.permute(0, 2, 3, 1).contiguous()
    return kc, vc


@pytest.mark.parametrize("case", ["gqa_b16", "mha_b32_alibi", "gqa9_3_d96_b16"])
@pytest.mark.parametrize("mode,part", [("ref", None), ("ref", 64), ("f64", None)])
def test_attention_oracle_matches_reference_cpu_kernel(case, mode, part):
    g = np.load(GOLD / "cpu_attn_golden.npz")
    t = lambda n: torch.from_numpy(g[f"{case}/{n}"])
    q = t("query").view(torch.bfloat16)
    kf = t("key_flash").view(torch.bfloat16)
    vf = t("value_flash").view(torch.bfloat16)
    want = t("out").view(torch.bfloat16).float()
    alibi = t("alibi") if f"{case}/alibi" in g.files else None
    kc, vc = _paged_from_flash(kf, vf)
    hkv = kf.shape[2]
    d = q.shape[2]
    got = O.paged_attention(q, kc, vc, hkv, d ** -0.5, t("block_tables"), t("seq_lens"), alibi,
                            mode=mode, partition_size=part).float()
    # the reference's own CPU test tolerates atol 1.5e-2 / rtol 1e-2
    # (tests/kernels/attention/test_cpu_attn.py:320); the restatement is far inside it
    torch.testing.assert_close(got, want, atol=2e-4, rtol=1e-2)


def test_reshape_and_cache_layout_roundtrip():
    g = torch.Generator().manual_seed(0)
    T, H, D, B, NB = 37, 3, 64, 8, 9
    key = torch.randn(T, H, D, generator=g).to(torch.bfloat16)
    val = torch.randn(T, H, D, generator=g).to(torch.bfloat16)
    slots = torch.randperm(NB * B, generator=g)[:T]
    slots[3] = -1
    kc = torch.zeros(NB, H, D // 8, B, 8, dtype=torch.bfloat16)
    vc = torch.zeros(NB, H, D, B, dtype=torch.bfloat16)
    O.reshape_and_cache(key, val, kc, vc, slots, "auto", 1.0, 1.0)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        b, o = divmod(s, B)
        assert torch.equal(kc[b, :, :, o, :].reshape(H, D), key[t])
        assert torch.equal(vc[b, :, :, o], val[t])
    # the padded token wrote nothing
    assert int((kc != 0).any(dim=(1, 2, 4)).sum()) == T - 1


def test_cuda_reference_fixture_if_present():
    """Outputs of the reference's CUDA kernels captured on a B200 (see
    tests/golden/make_cuda_ref_golden.py) must agree with the oracle."""
    f = GOLD / "cuda_ref_golden.npz"
    if not f.exists():
        pytest.skip("cuda_ref_golden.npz not generated yet")
    g = np.load(f)
    cases = sorted({k.split("/")[0] for k in g.files})
    assert cases
    for case in cases:
        t = lambda n: torch.from_numpy(g[f"{case}/{n}"])
        meta = g[f"{case}/meta"]  # hkv, block_size, is_fp8, version
        hkv, is_fp8, ver = int(meta[0]), bool(meta[2]), int(meta[3])
        q = t("query").view(torch.bfloat16)
        kc, vc = t("key_cache"), t("value_cache")
        if not is_fp8:
            kc, vc = kc.view(torch.bfloat16), vc.view(torch.bfloat16)
        scales = g[f"{case}/scales"]
        want = t("out").view(torch.bfloat16).float()
        alibi = t("alibi") if f"{case}/alibi" in g.files else None
        got = O.paged_attention(q, kc, vc, hkv, float(scales[2]), t("block_tables"), t("seq_lens"),
                                alibi, "fp8" if is_fp8 else "auto", float(scales[0]), float(scales[1]),
                                mode="ref", partition_size=512 if ver == 2 else None).float()
        # same arithmetic, different summation order: a few bf16 ulps of the output
        torch.testing.assert_close(got, want, atol=1e-3, rtol=2e-2, msg=lambda m: f"{case}: {m}")
        if f"{case}/kc_written" in g.files:
            nk, nv = t("new_key").view(torch.bfloat16), t("new_value").view(torch.bfloat16)
            kcw = torch.zeros_like(t("kc_written"))
            vcw = torch.zeros_like(t("vc_written"))
            O.reshape_and_cache(nk, nv, kcw, vcw, t("slots"), "fp8", float(scales[0]), float(scales[1]))
            assert torch.equal(kcw, t("kc_written")) and torch.equal(vcw, t("vc_written")), case
