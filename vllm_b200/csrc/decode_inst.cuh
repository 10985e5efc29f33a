// Explicit-instantiation helper: each decode_d*.cu file builds the tensor-core
// decode kernel for one or two head sizes so the files compile in parallel.
#pragma once

#include "decode_kernel.cuh"

namespace b200pa {

using DecodeLaunchFn = cudaError_t (*)(const DecodeParams&, int grid, int threads, size_t smem,
                                       cudaStream_t stream);

// A built kernel variant: its launcher and the most warps per CTA it may be launched with.
struct DecodeKernelInfo {
  DecodeLaunchFn fn;
  int max_warps;
  int pages_per_step;  // cache blocks per pipeline step (sizes the ring slots)
};

// Warps per CTA the kernel is compiled for, by its register footprint (accumulators and
// query fragments grow with D * GP): 16 warps (<= 128 registers per thread), 12 (<= 168) or 8.
template <int KV, int D, int GP>
constexpr int decode_max_warps() {
  return (D * GP <= 128) ? 16 : (D * GP <= 256 ? 12 : 8);
}

template <typename QT, int KV, int D, int GP, int NT>
cudaError_t decode_launch(const DecodeParams& p, int grid, int threads, size_t smem,
                          cudaStream_t stream) {
  auto kern = pa_decode_kernel<QT, KV, D, GP, NT, decode_max_warps<KV, D, GP>()>;
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

template <typename QT, int KV, int D, int GP>
DecodeKernelInfo pick_nt(int nt) {
  constexpr int es = KV == kCache16 ? 2 : 1;
  if (nt == 1)
    return {decode_launch<QT, KV, D, GP, 1>, decode_max_warps<KV, D, GP>(),
            decode_pages_per_step(es, D, 1)};
  return {decode_launch<QT, KV, D, GP, 2>, decode_max_warps<KV, D, GP>(),
          decode_pages_per_step(es, D, 2)};
}

template <typename QT, int KV, int D>
DecodeKernelInfo pick_gp(int gp, int nt) {
  if (gp == 1) return pick_nt<QT, KV, D, 1>(nt);
  return pick_nt<QT, KV, D, 2>(nt);
}

template <typename QT, int D>
DecodeKernelInfo pick_kv(int kv_dtype, int gp, int nt) {
  switch (kv_dtype) {
    case B200PA_KV_AUTO: return pick_gp<QT, kCache16, D>(gp, nt);
    case B200PA_KV_FP8_E4M3: return pick_gp<QT, kCacheE4M3, D>(gp, nt);
    case B200PA_KV_FP8_E5M2: return pick_gp<QT, kCacheE5M2, D>(gp, nt);
  }
  return {nullptr, 0, 1};
}

// gp: 8-head n-tiles per work item (1 or 2); nt: 16-token tiles per cache block (1 or 2).
template <int D>
DecodeKernelInfo find_decode_for(int q_dtype, int kv_dtype, int gp, int nt) {
  if ((gp != 1 && gp != 2) || (nt != 1 && nt != 2)) return {nullptr, 0, 1};
  if (q_dtype == B200PA_BF16) return pick_kv<__nv_bfloat16, D>(kv_dtype, gp, nt);
  if (q_dtype == B200PA_F16) return pick_kv<__half, D>(kv_dtype, gp, nt);
  return {nullptr, 0, 1};
}

// One finder per translation unit (defined in decode_d*.cu).
DecodeKernelInfo find_decode_d32(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d64(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d80(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d96(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d112(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d128(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d192(int q_dtype, int kv_dtype, int gp, int nt);
DecodeKernelInfo find_decode_d256(int q_dtype, int kv_dtype, int gp, int nt);

}  // namespace b200pa
