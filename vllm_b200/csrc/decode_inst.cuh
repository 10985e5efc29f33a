// Explicit-instantiation helper: each decode_d*.cu file builds the tensor-core
// decode kernel for one or two head sizes so the files compile in parallel.
#pragma once

#include "decode_kernel.cuh"

namespace b200pa {

using DecodeLaunchFn = cudaError_t (*)(const DecodeParams&, int grid, int threads, size_t smem,
                                       cudaStream_t stream);

template <typename QT, int KV, int D, int GP>
cudaError_t decode_launch(const DecodeParams& p, int grid, int threads, size_t smem,
                          cudaStream_t stream) {
  auto kern = pa_decode_kernel<QT, KV, D, GP>;
  // opt in to large dynamic shared memory once per device
  static bool done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !done[dev]) {
    // the opt-in limit covers static + dynamic shared memory
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, kern);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               227 * 1024 - int(fa.sharedSizeBytes));
    if (e != cudaSuccess) {
      (void)cudaGetLastError();  // do not leave the error for the next caller
      return e;
    }
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  kern<<<grid, threads, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int D>
DecodeLaunchFn find_decode_for(int q_dtype, int kv_dtype, int gp) {
#define B200PA_PICK(QT)                                                                  \
  switch (kv_dtype) {                                                                    \
    case B200PA_KV_AUTO:                                                                 \
      return gp == 1 ? decode_launch<QT, kCache16, D, 1> : decode_launch<QT, kCache16, D, 2>; \
    case B200PA_KV_FP8_E4M3:                                                             \
      return gp == 1 ? decode_launch<QT, kCacheE4M3, D, 1> : decode_launch<QT, kCacheE4M3, D, 2>; \
    case B200PA_KV_FP8_E5M2:                                                             \
      return gp == 1 ? decode_launch<QT, kCacheE5M2, D, 1> : decode_launch<QT, kCacheE5M2, D, 2>; \
  }                                                                                      \
  return nullptr;
  if (gp != 1 && gp != 2) return nullptr;
  if (q_dtype == B200PA_BF16) { B200PA_PICK(__nv_bfloat16) }
  if (q_dtype == B200PA_F16) { B200PA_PICK(__half) }
#undef B200PA_PICK
  return nullptr;
}

// One finder per translation unit (defined in decode_d*.cu).
DecodeLaunchFn find_decode_d32(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d64(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d80(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d96(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d112(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d128(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d192(int q_dtype, int kv_dtype, int gp);
DecodeLaunchFn find_decode_d256(int q_dtype, int kv_dtype, int gp);

}  // namespace b200pa
