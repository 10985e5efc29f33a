"""Generates tests/golden/fp8_golden.npz with NVIDIA's host fp8 conversion.

The reference quantises with ``__nv_cvt_float_to_fp8(float(x) / scale,
__NV_SATFINITE, fmt)`` (csrc/quantization/w8a8/fp8/nvidia/quant_utils.cuh:469-502).
That function has a host implementation in the CUDA toolkit's ``cuda_fp8.hpp``;
this script compiles a few lines of host C++ against it (nvcc, no GPU needed),
feeds it every bf16 bit pattern at several scales and stores the resulting bytes
for e4m3 and e5m2.  The fixture pins oracle.paged_oracle.quantize_fp8.

    python tests/golden/make_fp8_golden.py
"""
import subprocess
import tempfile
from pathlib import Path

import numpy as np

SRC = r"""
#include <cuda_fp8.h>
#include <cstdio>
#include <cstdint>
#include <cstring>
int main(int argc, char** argv) {
  const float scales[] = {1.0f, 0.011826f, 3.7f};
  FILE* f = fopen(argv[1], "wb");
  for (int fmt = 0; fmt < 2; ++fmt)
    for (float scale : scales)
      for (uint32_t b = 0; b < 65536; ++b) {
        uint32_t bits = b << 16;  // bf16 -> f32 is exact
        float x; memcpy(&x, &bits, 4);
        float q = x / scale;
        uint8_t r = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, fmt == 0 ? __NV_E4M3 : __NV_E5M2);
        fputc(r, f);
      }
  fclose(f);
  return 0;
}
"""


def main() -> None:
    with tempfile.TemporaryDirectory() as td:
        src = Path(td) / "cvt.cu"
        src.write_text(SRC)
        exe = Path(td) / "cvt"
        subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-O1", "-o", str(exe), str(src)])
        raw = Path(td) / "out.bin"
        subprocess.check_call([str(exe), str(raw)])
        data = np.fromfile(raw, dtype=np.uint8).reshape(2, 3, 65536)
    np.savez_compressed(Path(__file__).with_name("fp8_golden.npz"),
                        scales=np.array([1.0, 0.011826, 3.7], dtype=np.float32),
                        e4m3=data[0], e5m2=data[1])
    print("wrote fp8_golden.npz", data.shape)


if __name__ == "__main__":
    main()
