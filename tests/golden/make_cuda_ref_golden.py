"""Generates cuda_ref_golden.npz from the reference's own CUDA kernels on a GPU.

Runs ``paged_attention_v1/v2`` and ``reshape_and_cache`` of the reference
(csrc/attention/paged_attention_v1.cu, paged_attention_v2.cu, csrc/cache_kernels.cu
compiled unmodified for sm_100a into oracle/_ref/_C_ref.so by oracle/build_ref.py)
on small seeded inputs and stores inputs and outputs.  Needs a CUDA device and the
prebuilt _C_ref.so (not the reference checkout).  Writes to the directory given as
argv[1] (default: this directory).

    python tests/golden/make_cuda_ref_golden.py [out_dir]
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

CASES = [
    # name, version, S, Hq, Hkv, D, B, max_len, fp8, alibi
    ("v1_bf16_gqa", 1, 4, 8, 2, 128, 16, 200, False, False),
    ("v2_bf16_parts", 2, 3, 4, 1, 64, 16, 1100, False, False),
    ("v2_fp8_gqa8", 2, 3, 8, 1, 128, 16, 600, True, False),
    ("v1_bf16_alibi_b32", 1, 3, 4, 2, 64, 32, 300, False, True),
]


def main() -> None:
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).parent
    torch.ops.load_library(str(ROOT / "oracle" / "_ref" / "_C_ref.so"))
    ref, ref_cache = torch.ops._C_ref, torch.ops._C_ref_cache_ops
    dev = "cuda"
    out = {}
    for name, ver, S, Hq, Hkv, D, B, max_len, fp8, alibi in CASES:
        g = torch.Generator().manual_seed(4321)
        rng = np.random.default_rng(4321)
        lens = rng.integers(1, max_len + 1, size=S)
        lens[-1] = max_len
        maxb = (max_len + B - 1) // B
        nb = maxb + 2
        amp = D ** -0.5
        q = (torch.rand(S, Hq, D, generator=g) * 2 - 1).mul(amp * 6).to(torch.bfloat16)
        x = 16 if fp8 else 8
        if fp8:
            ks, vs = 0.0131, 0.0117
            kc = (torch.randn(nb, Hkv, D // x, B, x, generator=g) / ks).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
            vc = (torch.randn(nb, Hkv, D, B, generator=g) / vs).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        else:
            ks = vs = 1.0
            kc = (torch.rand(nb, Hkv, D // x, B, x, generator=g) * 2 - 1).mul(amp).to(torch.bfloat16)
            vc = (torch.rand(nb, Hkv, D, B, generator=g) * 2 - 1).mul(amp).to(torch.bfloat16)
        bt = np.stack([rng.permutation(nb)[:maxb] for _ in range(S)]).astype(np.int32)
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / Hq) for i in range(Hq)], dtype=torch.float32) if alibi else None
        scale = float(D ** -0.5)
        d = lambda t: t.to(dev) if t is not None else None
        o = torch.empty(S, Hq, D, dtype=torch.bfloat16, device=dev)
        kst = torch.tensor(ks, dtype=torch.float32, device=dev)
        vst = torch.tensor(vs, dtype=torch.float32, device=dev)
        args = (d(q), d(kc), d(vc), Hkv, scale, d(torch.from_numpy(bt)), d(torch.from_numpy(lens.astype(np.int32))),
                B, int(max_len), d(slopes), "fp8" if fp8 else "auto", kst, vst, 0, 0, 0, 64, 0)
        if ver == 1:
            ref.paged_attention_v1(o, *args)
        else:
            P = (max_len + 511) // 512
            es = torch.empty(S, Hq, P, dtype=torch.float32, device=dev)
            ml = torch.empty_like(es)
            tmp = torch.empty(S, Hq, P, D, dtype=torch.bfloat16, device=dev)
            ref.paged_attention_v2(o, es, ml, tmp, *args)
        torch.cuda.synchronize()
        pre = name + "/"
        out[pre + "meta"] = np.array([Hkv, B, int(fp8), ver], dtype=np.int32)
        out[pre + "scales"] = np.array([ks, vs, scale], dtype=np.float32)
        out[pre + "query"] = q.view(torch.int16).numpy()
        out[pre + "key_cache"] = kc.numpy() if fp8 else kc.view(torch.int16).numpy()
        out[pre + "value_cache"] = vc.numpy() if fp8 else vc.view(torch.int16).numpy()
        out[pre + "block_tables"] = bt
        out[pre + "seq_lens"] = lens.astype(np.int32)
        out[pre + "out"] = o.cpu().view(torch.int16).numpy()
        if alibi:
            out[pre + "alibi"] = slopes.numpy()
        if fp8:
            T = 40
            nk = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
            nv = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
            slots = torch.from_numpy(rng.permutation(nb * B)[:T].astype(np.int64))
            slots[7] = -1
            kcw = torch.zeros_like(kc).to(dev)
            vcw = torch.zeros_like(vc).to(dev)
            ref_cache.reshape_and_cache(nk.to(dev), nv.to(dev), kcw, vcw, slots.to(dev), "fp8", kst, vst)
            torch.cuda.synchronize()
            out[pre + "new_key"] = nk.view(torch.int16).numpy()
            out[pre + "new_value"] = nv.view(torch.int16).numpy()
            out[pre + "slots"] = slots.numpy()
            out[pre + "kc_written"] = kcw.cpu().numpy()
            out[pre + "vc_written"] = vcw.cpu().numpy()
        print(name, "ok", float(o.float().abs().max()))
    out_dir.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_dir / "cuda_ref_golden.npz", **out)


if __name__ == "__main__":
    main()
