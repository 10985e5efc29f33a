"""Generates tests/golden/cpu_attn_golden.npz from the reference's own CPU attention.

Runs ``cpu_attention_with_kv_cache`` (reference csrc/cpu/cpu_attn.cpp, built
unmodified into oracle/_ref/_C_ref_cpu.so by oracle/build_ref.py) on small seeded
decode batches and stores inputs and outputs.  Must be run where the reference
checkout is mounted; the resulting fixture pins oracle/paged_oracle.py on any box.

    python tests/golden/make_cpu_attn_golden.py
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_cpu  # noqa: E402

CASES = [
    # name, S, Hq, Hkv, D, B, max_len, alibi, kv_split
    ("gqa_b16", 5, 8, 2, 128, 16, 150, False, True),
    ("mha_b32_alibi", 4, 2, 2, 128, 32, 120, True, False),
    ("gqa9_3_d96_b16", 3, 9, 3, 96, 16, 100, False, True),
]


def main() -> None:
    out = {}
    for name, S, Hq, Hkv, D, B, max_len, alibi, split in CASES:
        g = torch.Generator().manual_seed(1234)
        rng = np.random.default_rng(1234)
        lens = rng.integers(1, max_len + 1, size=S)
        lens[-1] = max_len
        nb = (max_len + B - 1) // B
        amp = D ** -0.5
        q = (torch.rand(S, Hq, D, generator=g) * 2 - 1).mul(amp * 8).to(torch.bfloat16)
        kf = (torch.rand(nb, B, Hkv, D, generator=g) * 2 - 1).mul(amp).to(torch.bfloat16)
        vf = (torch.rand(nb, B, Hkv, D, generator=g) * 2 - 1).mul(amp).to(torch.bfloat16)
        maxb = (max_len + B - 1) // B
        bt = np.stack([rng.permutation(nb)[:maxb] for _ in range(S)]).astype(np.int32)
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / Hq) for i in range(Hq)], dtype=torch.float32) if alibi else None
        r = ref_cpu.RefCpuDecode(q, kf, vf, torch.from_numpy(bt), torch.from_numpy(lens.astype(np.int32)),
                                 D ** -0.5, slopes, kv_split=split)
        o = r.run().clone()
        pre = name + "/"
        out[pre + "query"] = q.view(torch.int16).numpy()
        out[pre + "key_flash"] = kf.view(torch.int16).numpy()
        out[pre + "value_flash"] = vf.view(torch.int16).numpy()
        out[pre + "block_tables"] = bt
        out[pre + "seq_lens"] = lens.astype(np.int32)
        out[pre + "out"] = o.view(torch.int16).numpy()
        if alibi:
            out[pre + "alibi"] = slopes.numpy()
        print(name, "ok", float(o.float().abs().max()))
    np.savez_compressed(Path(__file__).with_name("cpu_attn_golden.npz"), **out)


if __name__ == "__main__":
    main()
