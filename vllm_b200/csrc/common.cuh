// Shared host/device helpers of libb200pa: error reporting, dtype traits and the
// fp8 conversions used by both the KV-write kernels and the decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/b200pa.h"

namespace b200pa {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);  // defined in capi.cu (thread-local buffer)
void count_launch(int n = 1);          // defined in capi.cu

#define B200PA_CHECK_ARG(cond, ...)     \
  do {                                  \
    if (!(cond)) {                      \
      ::b200pa::set_error(__VA_ARGS__); \
      return B200PA_EINVAL;             \
    }                                   \
  } while (0)

#define B200PA_CHECK_CUDA(expr)                                                   \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess) {                                                      \
      ::b200pa::set_error("%s failed: %s", #expr, cudaGetErrorString(e_));        \
      return B200PA_ECUDA;                                                        \
    }                                                                             \
  } while (0)

inline int dtype_size(int dt) { return dt == B200PA_F32 ? 4 : 2; }

// Device address of the status word of the current device (one word per device
// that loads the library).  Bounded waits in the decode kernel record a non-zero
// code there instead of spinning forever.  Returns nullptr (and sets the error
// text) if the address cannot be resolved.  Defined in capi.cu.
int* device_status_ptr();

// ---------------------------------------------------------------- device side
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Two floats -> two fp8 bytes, round-to-nearest-even, saturate-to-finite, NaN -> 0x7F.
// Low byte = first argument.  kE5M2 selects the e5m2 interpretation.
template <bool kE5M2>
__device__ __forceinline__ uint16_t f32x2_to_fp8x2(float lo, float hi) {
  uint16_t r;
  if constexpr (kE5M2) {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

template <bool kE5M2>
__device__ __forceinline__ uint8_t f32_to_fp8(float v) {
  return static_cast<uint8_t>(f32x2_to_fp8x2<kE5M2>(v, 0.f) & 0xFF);
}

// Two fp8 bytes (low 16 bits of `v`) -> packed f16x2 (exact: every e4m3/e5m2
// value is representable in f16).
template <bool kE5M2>
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint16_t v) {
  uint32_t r;
  if constexpr (kE5M2) {
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(v));
  } else {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  }
  return r;
}

template <bool kE5M2>
__device__ __forceinline__ float fp8_to_f32(uint8_t v) {
  uint32_t h2 = fp8x2_to_f16x2<kE5M2>(static_cast<uint16_t>(v));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half2float(__low2half(h));
}

}  // namespace b200pa
