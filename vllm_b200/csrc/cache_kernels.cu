// KV-write kernels: scatter new K/V tokens into the paged cache, optionally
// quantising to fp8.  Replaces the reference's reshape_and_cache_kernel,
// reshape_and_cache_flash_kernel and convert_fp8_kernel
// (csrc/cache_kernels.cu:225-283, :285-358, :826-899).
//
// The work is pure data movement, so the design goal is full-sector traffic:
//   * x-layout K: one 16-byte store per (token, head, d/x) chunk.
//   * x-layout V is a transpose ([token][d] -> [d][token-in-block]).  A CTA owns
//     a tile of 16 consecutive tokens.  When the tile fills 16 consecutive slots
//     of one block (prefill, chunked writes) a thread reads 16 bytes of 8 d per
//     token and writes 8 rows of 16 tokens with 16-byte stores; otherwise each
//     thread owns one (head, d) row and writes every run of tokens that landed
//     in consecutive slots with the widest aligned store, instead of one
//     1-2 byte store per element.
//   * flash layout: 16-byte vector row copies, NHD or HND by strides.
// Quantisation is cvt.rn.satfinite of the correctly rounded fp32 quotient x / scale,
// bit-identical to the reference's scaled_convert (quant_utils.cuh:469-502).
#include "common.cuh"

namespace b200pa {

enum : int { kKvAuto = 0, kKvE4M3 = 1, kKvE5M2 = 2 };

// x / scale, correctly rounded, for one scale and many x.  The compiler's division spends a
// MUFU.RCP, a range check and a slow-path branch on every element, which made the KV write
// XU-bound; here the reciprocal is taken once and each quotient is the product x * r followed
// by two residual corrections q += fma(-q, s, x) * r.  The first leaves q within one ulp, the
// second then yields the correctly rounded quotient (Markstein's theorem; r is the correctly
// rounded reciprocal).  Only used while nothing can overflow or lose residual bits to
// underflow: scales within 2^+-60 and 2^-20 <= |q| < 2^17.  Outside that window the plain
// product x * r is returned: larger quotients saturate in both fp8 formats and smaller ones
// round to zero whatever their last bits are (the product also keeps the sign of a zero and
// passes inf / NaN through, which the corrections would not).  Other scales use the division.
struct ScaledDiv {
  float s, r;
  bool fast;
  __device__ __forceinline__ explicit ScaledDiv(float scale) : s(scale) {
    r = __fdiv_rn(1.f, scale);
    const float a = fabsf(scale);
    fast = a >= 0x1p-60f && a <= 0x1p60f;
  }
  // Two quotients at once on the packed fp32 pipe (fma.rn.f32x2, sm_100).
  __device__ __forceinline__ void pair(float x0, float x1, float& o0, float& o1) const {
    if (!fast) {
      o0 = __fdiv_rn(x0, s);
      o1 = __fdiv_rn(x1, s);
      return;
    }
    float p0, p1, c0, c1;
    asm("{\n"
        " .reg .b64 x, r, ns, q, e;\n"
        " mov.b64 x, {%4, %5};\n"
        " mov.b64 r, {%6, %6};\n"
        " mov.b64 ns, {%7, %7};\n"
        " mul.rn.f32x2 q, x, r;\n"
        " mov.b64 {%0, %1}, q;\n"
        " fma.rn.f32x2 e, q, ns, x;\n"
        " fma.rn.f32x2 q, e, r, q;\n"
        " fma.rn.f32x2 e, q, ns, x;\n"
        " fma.rn.f32x2 q, e, r, q;\n"
        " mov.b64 {%2, %3}, q;\n"
        "}"
        : "=f"(p0), "=f"(p1), "=f"(c0), "=f"(c1)
        : "f"(x0), "f"(x1), "f"(r), "f"(-s));
    const float a0 = fabsf(p0), a1 = fabsf(p1);
    o0 = (a0 >= 0x1p-20f && a0 < 0x1p17f) ? c0 : p0;
    o1 = (a1 >= 0x1p-20f && a1 < 0x1p17f) ? c1 : p1;
  }
  __device__ __forceinline__ float operator()(float x) const {
    if (!fast) return __fdiv_rn(x, s);
    const float q0 = x * r;
    float q = fmaf(fmaf(-q0, s, x), r, q0);
    q = fmaf(fmaf(-q, s, x), r, q);
    const float a = fabsf(q0);
    return (a >= 0x1p-20f && a < 0x1p17f) ? q : q0;
  }
};

template <typename in_t, typename cache_t, int KV>
__device__ __forceinline__ cache_t store_convert(in_t v, const ScaledDiv& div) {
  if constexpr (KV == kKvAuto) {
    return v;
  } else {
    return f32_to_fp8<KV == kKvE5M2>(div(to_f32(v)));
  }
}

// N consecutive elements; fp8 conversions go two at a time (one cvt for a byte pair).
template <typename in_t, typename cache_t, int KV, int N>
__device__ __forceinline__ void convert_n(const in_t (&in)[N], cache_t* out, const ScaledDiv& div) {
  if constexpr (KV == kKvAuto) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = in[i];
  } else {
    static_assert(N % 2 == 0, "pairs");
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      float q0, q1;
      div.pair(to_f32(in[i]), to_f32(in[i + 1]), q0, q1);
      const uint16_t two = f32x2_to_fp8x2<KV == kKvE5M2>(q0, q1);
      out[i] = static_cast<cache_t>(two & 0xFF);
      out[i + 1] = static_cast<cache_t>(two >> 8);
    }
  }
}

constexpr int kTokTile = 16;

// Widest store that the address and byte count allow.
template <typename cache_t, int N>
__device__ __forceinline__ void store_run(cache_t* dst, const cache_t (&vals)[N], int len) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(dst);
  const int bytes = len * int(sizeof(cache_t));
  if (((a | bytes) & 15) == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(vals);
#pragma unroll
    for (int i = 0; i < int(N * sizeof(cache_t) / 16); ++i)
      if (i * 16 < bytes) reinterpret_cast<uint4*>(dst)[i] = src[i];
  } else if (((a | bytes) & 7) == 0) {
    const uint2* src = reinterpret_cast<const uint2*>(vals);
#pragma unroll
    for (int i = 0; i < int(N * sizeof(cache_t) / 8); ++i)
      if (i * 8 < bytes) reinterpret_cast<uint2*>(dst)[i] = src[i];
  } else if (((a | bytes) & 3) == 0) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(vals);
#pragma unroll
    for (int i = 0; i < int(N * sizeof(cache_t) / 4); ++i)
      if (i * 4 < bytes) reinterpret_cast<uint32_t*>(dst)[i] = src[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < len) dst[i] = vals[i];
  }
}

// grid.x = ceil(num_tokens / kTokTile); block = 256 threads.
template <typename in_t, typename cache_t, int KV>
__global__ void __launch_bounds__(256)
reshape_and_cache_kernel(const in_t* __restrict__ key, const in_t* __restrict__ value,
                         cache_t* __restrict__ key_cache, cache_t* __restrict__ value_cache,
                         const int64_t* __restrict__ slot_mapping, int64_t key_stride,
                         int64_t value_stride, int num_tokens, int num_heads, int head_size,
                         int block_size, int x, const float* __restrict__ k_scale_ptr,
                         const float* __restrict__ v_scale_ptr) {
  __shared__ int64_t s_slot[kTokTile];
  const int tok0 = blockIdx.x * kTokTile;
  const int ntok = min(kTokTile, num_tokens - tok0);
  if (threadIdx.x < kTokTile)
    s_slot[threadIdx.x] = threadIdx.x < ntok ? slot_mapping[tok0 + threadIdx.x] : int64_t(-1);
  __syncthreads();

  const ScaledDiv k_scale((KV == kKvAuto) ? 1.f : *k_scale_ptr);
  const ScaledDiv v_scale((KV == kKvAuto) ? 1.f : *v_scale_ptr);
  const int chunks = head_size / x;  // per head
  const int hd = num_heads * head_size;
  // 16-byte loads from key/value rows are legal when bases and row strides are 16-byte multiples
  const bool in_vec_ok =
      ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
        (size_t(key_stride) * sizeof(in_t)) | (size_t(value_stride) * sizeof(in_t)) |
        (size_t(head_size) * sizeof(in_t)) | (size_t(x) * sizeof(in_t))) & 15) == 0;

  // ---- K: work item = (token, head, chunk); chunk fastest for coalesced reads.
  const int k_items = ntok * num_heads * chunks;
  for (int it = threadIdx.x; it < k_items; it += blockDim.x) {
    const int c = it % chunks;
    const int h = (it / chunks) % num_heads;
    const int t = it / (chunks * num_heads);
    const int64_t slot = s_slot[t];
    if (slot < 0) continue;
    const int64_t b = slot / block_size;
    const int off = int(slot % block_size);
    const in_t* src = key + int64_t(tok0 + t) * key_stride + h * head_size + c * x;
    cache_t* dst = key_cache + ((b * num_heads + h) * chunks + c) * int64_t(block_size) * x +
                   int64_t(off) * x;
    // x elements = 16 bytes of cache in the standard layout; handle any x generically.
    if (x * int(sizeof(cache_t)) == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      constexpr int N = 16 / sizeof(cache_t);        // elements per 16-byte store
      constexpr int L = N * sizeof(in_t) / 16;       // 16-byte loads that feed it
      __align__(16) in_t in[N];
      if (in_vec_ok) {
#pragma unroll
        for (int i = 0; i < L; ++i)
          reinterpret_cast<uint4*>(in)[i] = reinterpret_cast<const uint4*>(src)[i];
      } else {
#pragma unroll
        for (int i = 0; i < N; ++i) in[i] = src[i];
      }
      __align__(16) cache_t vals[N];
      convert_n<in_t, cache_t, KV, N>(in, vals, k_scale);
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
    } else {
      for (int i = 0; i < x; ++i) dst[i] = store_convert<in_t, cache_t, KV>(src[i], k_scale);
    }
  }

  // ---- V fast path: the whole tile is one run that fills slots [off, off+16) of one block
  // (prefill / chunked writes).  A thread takes VD consecutive d of one head, reads them
  // for the 16 tokens with 16-byte loads and writes VD rows of 16 tokens each.
  constexpr int VD = 16 / sizeof(in_t);
  bool full_run = ntok == kTokTile && in_vec_ok && head_size % VD == 0 && block_size % kTokTile == 0;
  if (full_run) {
    const int64_t s0 = s_slot[0];
    full_run = s0 >= 0 && (s0 % kTokTile) == 0;
#pragma unroll
    for (int i = 1; i < kTokTile; ++i) full_run = full_run && s_slot[i] == s0 + i;
    full_run = full_run &&
               ((reinterpret_cast<uintptr_t>(value_cache) | (size_t(block_size) * sizeof(cache_t))) &
                (kTokTile * sizeof(cache_t) >= 16 ? 15 : (kTokTile * sizeof(cache_t) - 1))) == 0;
  }
  if (full_run) {
    const int64_t s0 = s_slot[0];
    const int64_t b = s0 / block_size;
    const int off = int(s0 % block_size);
    const int groups = hd / VD;
    for (int gidx = threadIdx.x; gidx < groups; gidx += blockDim.x) {
      const int row0 = gidx * VD;  // (head, d) flattened; a group never straddles a head
      const in_t* src = value + int64_t(tok0) * value_stride + row0;
      __align__(16) cache_t vals[VD][kTokTile];
#pragma unroll
      for (int t = 0; t < kTokTile; t += 2) {
        __align__(16) in_t in0[VD], in1[VD];
        *reinterpret_cast<uint4*>(in0) = *reinterpret_cast<const uint4*>(src + int64_t(t) * value_stride);
        *reinterpret_cast<uint4*>(in1) =
            *reinterpret_cast<const uint4*>(src + int64_t(t + 1) * value_stride);
#pragma unroll
        for (int d = 0; d < VD; ++d) {
          const in_t two[2] = {in0[d], in1[d]};
          convert_n<in_t, cache_t, KV, 2>(two, &vals[d][t], v_scale);
        }
      }
      cache_t* dst = value_cache + (b * hd + row0) * int64_t(block_size) + off;
#pragma unroll
      for (int d = 0; d < VD; ++d) {
        constexpr int W = kTokTile * sizeof(cache_t) / 16;  // 16-byte stores per row (0 for 1-byte x 8...)
        if constexpr (W >= 1) {
#pragma unroll
          for (int w = 0; w < W; ++w)
            reinterpret_cast<uint4*>(dst + int64_t(d) * block_size)[w] =
                reinterpret_cast<const uint4*>(vals[d])[w];
        }
      }
    }
    return;
  }

  // ---- V: thread owns one (head, d) row of the tile; writes runs of consecutive slots.
  for (int row = threadIdx.x; row < hd; row += blockDim.x) {
    const int h = row / head_size;
    const int d = row % head_size;
    const in_t* src = value + int64_t(tok0) * value_stride + row;
    int i = 0;
    while (i < ntok) {
      const int64_t slot = s_slot[i];
      if (slot < 0) { ++i; continue; }
      const int64_t b = slot / block_size;
      const int off = int(slot % block_size);
      int len = 1;
      while (i + len < ntok && off + len < block_size && s_slot[i + len] == slot + len) ++len;
      cache_t vals[kTokTile];
#pragma unroll
      for (int k = 0; k < kTokTile; ++k)
        if (k < len)
          vals[k] = store_convert<in_t, cache_t, KV>(src[int64_t(i + k) * value_stride], v_scale);
      cache_t* dst = value_cache + ((b * num_heads + h) * head_size + d) * int64_t(block_size) + off;
      store_run<cache_t, kTokTile>(dst, vals, len);
      i += len;
    }
  }
}

// One CTA per token; 16-byte vector copies when everything is aligned.
template <typename in_t, typename cache_t, int KV>
__global__ void __launch_bounds__(256)
reshape_and_cache_flash_kernel(const in_t* __restrict__ key, const in_t* __restrict__ value,
                               cache_t* __restrict__ key_cache, cache_t* __restrict__ value_cache,
                               const int64_t* __restrict__ slot_mapping, int64_t block_stride,
                               int64_t page_stride, int64_t head_stride, int64_t key_stride,
                               int64_t value_stride, int num_heads, int head_size, int block_size,
                               int vec_ok, const float* __restrict__ k_scale_ptr,
                               const float* __restrict__ v_scale_ptr) {
  const int64_t token = blockIdx.x;
  const int64_t slot = slot_mapping[token];
  if (slot < 0) return;
  const int64_t b = slot / block_size;
  const int64_t off = slot % block_size;
  const float k_scale = (KV == kKvAuto) ? 1.f : *k_scale_ptr;
  const float v_scale = (KV == kKvAuto) ? 1.f : *v_scale_ptr;
  const in_t* ksrc = key + token * key_stride;
  const in_t* vsrc = value + token * value_stride;
  cache_t* kdst = key_cache + b * block_stride + off * page_stride;
  cache_t* vdst = value_cache + b * block_stride + off * page_stride;

  constexpr int VEC = 16 / sizeof(in_t);  // elements per 16-byte read
  if (vec_ok) {
    const int vec_per_head = head_size / VEC;
    const int items = num_heads * vec_per_head;
    // a thread's items are K first, then V: the divider is set up once per tensor it touches
    ScaledDiv scale(k_scale);
    bool scale_is_v = false;
    for (int it = threadIdx.x; it < 2 * items; it += blockDim.x) {
      const bool is_v = it >= items;
      if (is_v && !scale_is_v) {
        scale = ScaledDiv(v_scale);
        scale_is_v = true;
      }
      const int j = is_v ? it - items : it;
      const int h = j / vec_per_head;
      const int e = (j % vec_per_head) * VEC;
      const in_t* s = (is_v ? vsrc : ksrc) + h * head_size + e;
      cache_t* d = (is_v ? vdst : kdst) + h * head_stride + e;
      __align__(16) in_t in[VEC];
      *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(s);
      __align__(16) cache_t outv[VEC];
      convert_n<in_t, cache_t, KV, VEC>(in, outv, scale);
      if constexpr (sizeof(cache_t) * VEC == 16) {
        *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(outv);
      } else if constexpr (sizeof(cache_t) * VEC == 8) {
        *reinterpret_cast<uint2*>(d) = *reinterpret_cast<const uint2*>(outv);
      } else {
        *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(outv);
      }
    }
  } else {
    const int items = num_heads * head_size;
    const ScaledDiv kdiv(k_scale), vdiv(v_scale);
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int h = it / head_size;
      const int e = it % head_size;
      kdst[h * head_stride + e] = store_convert<in_t, cache_t, KV>(ksrc[it], kdiv);
      vdst[h * head_stride + e] = store_convert<in_t, cache_t, KV>(vsrc[it], vdiv);
    }
  }
}

// Elementwise quantise / dequantise, grid-stride.
template <typename wide_t, bool kE5M2, bool kToFp8>
__global__ void convert_fp8_kernel(void* __restrict__ dst_, const void* __restrict__ src_,
                                   int64_t numel, float scale) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const ScaledDiv div(scale);
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += stride) {
    if constexpr (kToFp8) {
      const wide_t v = static_cast<const wide_t*>(src_)[i];
      static_cast<uint8_t*>(dst_)[i] = f32_to_fp8<kE5M2>(div(to_f32(v)));
    } else {
      // reference order (quant_utils.cuh:360-372): fp8 -> half -> float * scale -> wide
      const uint8_t v = static_cast<const uint8_t*>(src_)[i];
      static_cast<wide_t*>(dst_)[i] = from_f32<wide_t>(fp8_to_f32<kE5M2>(v) * scale);
    }
  }
}

// ------------------------------------------------------------------ launchers
template <typename in_t, typename cache_t, int KV>
static int launch_reshape(const b200pa_cache_args& a, cudaStream_t stream, bool flash) {
  if (a.num_tokens == 0) return B200PA_OK;
  if (!flash) {
    dim3 grid((a.num_tokens + kTokTile - 1) / kTokTile);
    reshape_and_cache_kernel<in_t, cache_t, KV><<<grid, 256, 0, stream>>>(
        static_cast<const in_t*>(a.key), static_cast<const in_t*>(a.value),
        static_cast<cache_t*>(a.key_cache), static_cast<cache_t*>(a.value_cache), a.slot_mapping,
        a.key_stride, a.value_stride, a.num_tokens, a.num_heads, a.head_size, a.block_size, a.x,
        a.k_scale, a.v_scale);
  } else {
    constexpr int VEC = 16 / sizeof(in_t);
    auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; };
    const int out_bytes = VEC * int(sizeof(cache_t));
    const bool vec_ok =
        a.head_size % VEC == 0 && al(a.key, 16) && al(a.value, 16) && a.key_stride % VEC == 0 &&
        a.value_stride % VEC == 0 && al(a.key_cache, out_bytes) && al(a.value_cache, out_bytes) &&
        a.block_stride % VEC == 0 && a.page_stride % VEC == 0 && a.head_stride % VEC == 0;
    const int threads = 256;
    reshape_and_cache_flash_kernel<in_t, cache_t, KV><<<a.num_tokens, threads, 0, stream>>>(
        static_cast<const in_t*>(a.key), static_cast<const in_t*>(a.value),
        static_cast<cache_t*>(a.key_cache), static_cast<cache_t*>(a.value_cache), a.slot_mapping,
        a.block_stride, a.page_stride, a.head_stride, a.key_stride, a.value_stride, a.num_heads,
        a.head_size, a.block_size, vec_ok ? 1 : 0, a.k_scale, a.v_scale);
  }
  count_launch();
  B200PA_CHECK_CUDA(cudaGetLastError());
  return B200PA_OK;
}

template <typename in_t>
static int dispatch_kv(const b200pa_cache_args& a, cudaStream_t s, bool flash) {
  switch (a.kv_dtype) {
    case B200PA_KV_AUTO: return launch_reshape<in_t, in_t, kKvAuto>(a, s, flash);
    case B200PA_KV_FP8_E4M3: return launch_reshape<in_t, uint8_t, kKvE4M3>(a, s, flash);
    case B200PA_KV_FP8_E5M2: return launch_reshape<in_t, uint8_t, kKvE5M2>(a, s, flash);
  }
  set_error("Unsupported data type of kv cache: %d", a.kv_dtype);
  return B200PA_EUNSUPPORTED;
}

static int reshape_entry(const b200pa_cache_args* a, void* stream, bool flash) {
  B200PA_CHECK_ARG(a != nullptr, "args is NULL");
  B200PA_CHECK_ARG(a->num_tokens >= 0 && a->num_heads > 0 && a->head_size > 0 && a->block_size > 0,
                   "bad sizes: num_tokens=%d num_heads=%d head_size=%d block_size=%d",
                   a->num_tokens, a->num_heads, a->head_size, a->block_size);
  if (a->num_tokens > 0) {
    B200PA_CHECK_ARG(a->key && a->value && a->key_cache && a->value_cache && a->slot_mapping,
                     "null tensor pointer");
    B200PA_CHECK_ARG(a->kv_dtype == B200PA_KV_AUTO || (a->k_scale && a->v_scale),
                     "fp8 kv cache needs k_scale and v_scale");
  }
  if (!flash)
    B200PA_CHECK_ARG(a->x > 0 && a->head_size % a->x == 0, "head_size %d is not a multiple of x=%d",
                     a->head_size, a->x);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->in_dtype) {
    case B200PA_F32: return dispatch_kv<float>(*a, s, flash);
    case B200PA_F16: return dispatch_kv<__half>(*a, s, flash);
    case B200PA_BF16: return dispatch_kv<__nv_bfloat16>(*a, s, flash);
  }
  set_error("Unsupported input type of kv cache: %d", a->in_dtype);
  return B200PA_EUNSUPPORTED;
}

template <typename wide_t>
static int convert_dispatch(void* dst, const void* src, int64_t numel, float scale, int kv,
                            int to_fp8, cudaStream_t s) {
  const int threads = 256;
  const int64_t want = (numel + threads - 1) / threads;
  const int blocks = int(want < 148 * 16 ? want : 148 * 16);
  const bool e5 = kv == B200PA_KV_FP8_E5M2;
  if (to_fp8) {
    if (e5) convert_fp8_kernel<wide_t, true, true><<<blocks, threads, 0, s>>>(dst, src, numel, scale);
    else convert_fp8_kernel<wide_t, false, true><<<blocks, threads, 0, s>>>(dst, src, numel, scale);
  } else {
    if (e5) convert_fp8_kernel<wide_t, true, false><<<blocks, threads, 0, s>>>(dst, src, numel, scale);
    else convert_fp8_kernel<wide_t, false, false><<<blocks, threads, 0, s>>>(dst, src, numel, scale);
  }
  count_launch();
  B200PA_CHECK_CUDA(cudaGetLastError());
  return B200PA_OK;
}

}  // namespace b200pa

extern "C" int b200pa_reshape_and_cache(const b200pa_cache_args* args, void* stream) {
  return b200pa::reshape_entry(args, stream, false);
}

extern "C" int b200pa_reshape_and_cache_flash(const b200pa_cache_args* args, void* stream) {
  return b200pa::reshape_entry(args, stream, true);
}

extern "C" int b200pa_convert_fp8(void* dst, const void* src, int64_t numel, float scale,
                                  int32_t wide_dtype, int32_t kv_dtype, int32_t to_fp8,
                                  void* stream) {
  using namespace b200pa;
  B200PA_CHECK_ARG(numel >= 0, "numel < 0");
  if (numel == 0) return B200PA_OK;
  B200PA_CHECK_ARG(dst && src, "null pointer");
  if (kv_dtype != B200PA_KV_FP8_E4M3 && kv_dtype != B200PA_KV_FP8_E5M2) {
    set_error("Unsupported data type: %d", kv_dtype);
    return B200PA_EUNSUPPORTED;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (wide_dtype) {
    case B200PA_F32: return convert_dispatch<float>(dst, src, numel, scale, kv_dtype, to_fp8, s);
    case B200PA_F16: return convert_dispatch<__half>(dst, src, numel, scale, kv_dtype, to_fp8, s);
    case B200PA_BF16:
      return convert_dispatch<__nv_bfloat16>(dst, src, numel, scale, kv_dtype, to_fp8, s);
  }
  set_error("Unsupported wide dtype: %d", wide_dtype);
  return B200PA_EUNSUPPORTED;
}
