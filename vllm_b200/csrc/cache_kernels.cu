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
  // Callers check `fast` once per kernel, not per pair.
  __device__ __forceinline__ void pair(float x0, float x1, float& o0, float& o1) const {
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

// n / d for small operands (n * d < 2^32) by one multiply-high with a precomputed factor:
// the index arithmetic below would otherwise spend more instructions on runtime divisions
// than on the data.
struct SmallDiv {
  uint32_t m, d;
  __device__ __forceinline__ explicit SmallDiv(uint32_t d_) : d(d_) {
    m = d_ > 1 ? 0xFFFFFFFFu / d_ + 1 : 0;  // ceil(2^32 / d)
  }
  __device__ __forceinline__ uint32_t operator()(uint32_t n) const {
    return d == 1 ? n : __umulhi(n, m);
  }
};

// Per-tile set-up shared by both layouts: cache block and offset of each of the tile's
// tokens (block -1 = padding token, skipped), and whether the tile fills 16 consecutive
// slots that start at a multiple of 16 (true for prefill and chunked writes).
struct TileSlots {
  int64_t blk[kTokTile];
  int off[kTokTile];
  int full_run;
};

__device__ __forceinline__ void load_tile_slots(TileSlots& ts, const int64_t* __restrict__ slot_mapping,
                                                int tok0, int ntok, int block_size) {
  if (threadIdx.x < 32) {
    const int t = threadIdx.x;
    const int64_t slot = t < ntok ? slot_mapping[tok0 + t] : int64_t(-1);
    if (t < kTokTile) {
      const int64_t b = slot >= 0 ? slot / block_size : int64_t(-1);
      ts.blk[t] = b;
      ts.off[t] = slot >= 0 ? int(slot - b * block_size) : 0;
    }
    const int64_t s0 = __shfl_sync(0xffffffffu, slot, 0);
    const bool in_run = t >= kTokTile || slot == s0 + t;
    const bool all = __all_sync(0xffffffffu, in_run);
    if (t == 0)
      ts.full_run = all && ntok == kTokTile && s0 >= 0 && s0 % kTokTile == 0 &&
                    block_size % kTokTile == 0;
  }
  __syncthreads();
}

// Plain element-by-element path: scales outside the range ScaledDiv corrects in, x that does
// not give 16-byte chunks, unaligned tensors.
template <typename in_t, typename cache_t, int KV>
__device__ __noinline__ void reshape_tile_generic(const TileSlots& ts, const in_t* key, const in_t* value,
                                                  cache_t* key_cache, cache_t* value_cache,
                                                  int64_t key_stride, int64_t value_stride, int tok0,
                                                  int ntok, int num_heads, int head_size,
                                                  int block_size, int x, float k_scale, float v_scale) {
  const int hd = num_heads * head_size;
  for (int i = threadIdx.x; i < ntok * hd; i += blockDim.x) {
    const int t = i / hd, r = i % hd;
    if (ts.blk[t] < 0) continue;
    const int h = r / head_size, d = r % head_size;
    const int64_t bh = ts.blk[t] * num_heads + h;
    const in_t kv = key[int64_t(tok0 + t) * key_stride + r];
    const in_t vv = value[int64_t(tok0 + t) * value_stride + r];
    cache_t kq, vq;
    if constexpr (KV == kKvAuto) {
      kq = kv;
      vq = vv;
    } else {
      kq = f32_to_fp8<KV == kKvE5M2>(__fdiv_rn(to_f32(kv), k_scale));
      vq = f32_to_fp8<KV == kKvE5M2>(__fdiv_rn(to_f32(vv), v_scale));
    }
    key_cache[((bh * (head_size / x) + d / x) * block_size + ts.off[t]) * x + d % x] = kq;
    value_cache[(bh * head_size + d) * int64_t(block_size) + ts.off[t]] = vq;
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
  __shared__ TileSlots ts;
  const int tok0 = blockIdx.x * kTokTile;
  const int ntok = min(kTokTile, num_tokens - tok0);
  load_tile_slots(ts, slot_mapping, tok0, ntok, block_size);

  const float k_scale_f = (KV == kKvAuto) ? 1.f : *k_scale_ptr;
  const float v_scale_f = (KV == kKvAuto) ? 1.f : *v_scale_ptr;
  const ScaledDiv k_scale(k_scale_f), v_scale(v_scale_f);
  const int chunks = head_size / x;  // per head
  const int hd = num_heads * head_size;
  // 16-byte loads from key/value rows are legal when bases and row strides are 16-byte
  // multiples; x elements = 16 bytes of cache in the standard layout
  const bool vec_ok =
      ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
        reinterpret_cast<uintptr_t>(key_cache) | (size_t(key_stride) * sizeof(in_t)) |
        (size_t(value_stride) * sizeof(in_t)) | (size_t(head_size) * sizeof(in_t)) |
        (size_t(x) * sizeof(in_t))) & 15) == 0 &&
      x * int(sizeof(cache_t)) == 16 && (KV == kKvAuto || (k_scale.fast && v_scale.fast));
  if (!vec_ok) {
    reshape_tile_generic<in_t, cache_t, KV>(ts, key, value, key_cache, value_cache, key_stride,
                                            value_stride, tok0, ntok, num_heads, head_size,
                                            block_size, x, k_scale_f, v_scale_f);
    return;
  }

  // ---- K: work item = (token, head, chunk), chunk fastest for coalesced reads; one 16-byte
  // store per item, KB items in flight per thread.
  {
    constexpr int N = 16 / sizeof(cache_t);   // elements per 16-byte store
    constexpr int L = N * sizeof(in_t) / 16;  // 16-byte loads that feed it
    constexpr int KB = 4;
    const int per_tok = num_heads * chunks;
    const int k_items = ntok * per_tok;
    const SmallDiv by_tok(per_tok), by_chunks(chunks);
    for (int it0 = threadIdx.x; it0 < k_items; it0 += KB * blockDim.x) {
      __align__(16) in_t in[KB][N];
      cache_t* dst[KB];
#pragma unroll
      for (int k = 0; k < KB; ++k) {
        const int it = it0 + k * blockDim.x;
        dst[k] = nullptr;
        if (it < k_items) {
          const int t = int(by_tok(it));
          const int j = it - t * per_tok;
          const int h = int(by_chunks(j));
          const int c = j - h * chunks;
          const int64_t b = ts.blk[t];
          if (b >= 0) {
            const in_t* src = key + int64_t(tok0 + t) * key_stride + j * x;  // j * x = h * head_size + c * x
            dst[k] = key_cache + (((b * num_heads + h) * chunks + c) * int64_t(block_size) + ts.off[t]) * x;
#pragma unroll
            for (int i = 0; i < L; ++i)
              reinterpret_cast<uint4*>(in[k])[i] = reinterpret_cast<const uint4*>(src)[i];
          }
        }
      }
#pragma unroll
      for (int k = 0; k < KB; ++k) {
        if (dst[k] != nullptr) {
          __align__(16) cache_t vals[N];
          convert_n<in_t, cache_t, KV, N>(in[k], vals, k_scale);
          *reinterpret_cast<uint4*>(dst[k]) = *reinterpret_cast<const uint4*>(vals);
        }
      }
    }
  }

  // ---- V is a transpose ([token][d] -> [d][token in block]).
  constexpr int VD = 8 / sizeof(in_t);  // d per thread: one 8-byte load per token
  const bool v_rows_ok =
      ((reinterpret_cast<uintptr_t>(value_cache) | (size_t(block_size) * sizeof(cache_t))) &
       (kTokTile * sizeof(cache_t) >= 16 ? 15 : (kTokTile * sizeof(cache_t) - 1))) == 0;
  if (ts.full_run && v_rows_ok && head_size % VD == 0) {
    // Fast path: the tile fills slots [off, off+16) of one block.  A thread takes VD
    // consecutive d of one head for the 16 tokens and writes VD rows of 16 tokens each.
    const int64_t b = ts.blk[0];
    const int off = ts.off[0];
    const int groups = hd / VD;
    for (int gidx = threadIdx.x; gidx < groups; gidx += blockDim.x) {
      const int row0 = gidx * VD;  // (head, d) flattened; a group never straddles a head
      const in_t* src = value + int64_t(tok0) * value_stride + row0;
      __align__(8) in_t in[kTokTile][VD];
#pragma unroll
      for (int t = 0; t < kTokTile; ++t)
        *reinterpret_cast<uint2*>(in[t]) = *reinterpret_cast<const uint2*>(src + int64_t(t) * value_stride);
      __align__(16) cache_t vals[VD][kTokTile];
#pragma unroll
      for (int t = 0; t < kTokTile; t += 2) {
#pragma unroll
        for (int d = 0; d < VD; ++d) {
          const in_t two[2] = {in[t][d], in[t + 1][d]};
          convert_n<in_t, cache_t, KV, 2>(two, &vals[d][t], v_scale);
        }
      }
      cache_t* dst = value_cache + (b * hd + row0) * int64_t(block_size) + off;
#pragma unroll
      for (int d = 0; d < VD; ++d) {
        constexpr int W = kTokTile * sizeof(cache_t) / 16;  // 16-byte stores per row
#pragma unroll
        for (int w = 0; w < W; ++w)
          reinterpret_cast<uint4*>(dst + int64_t(d) * block_size)[w] =
              reinterpret_cast<const uint4*>(vals[d])[w];
      }
    }
    return;
  }

  // Ragged tile (decode steps): a thread owns one (head, d) row and writes every run of
  // tokens that landed in consecutive slots of one block with the widest aligned store.
  for (int row = threadIdx.x; row < hd; row += blockDim.x) {
    const in_t* src = value + int64_t(tok0) * value_stride + row;
    int i = 0;
    while (i < ntok) {
      const int64_t b = ts.blk[i];
      if (b < 0) { ++i; continue; }
      const int off = ts.off[i];
      int len = 1;
      while (i + len < ntok && ts.blk[i + len] == b && ts.off[i + len] == off + len) ++len;
      __align__(16) cache_t vals[kTokTile];
#pragma unroll
      for (int k = 0; k < kTokTile; ++k)
        if (k < len)
          vals[k] = store_convert<in_t, cache_t, KV>(src[int64_t(i + k) * value_stride], v_scale);
      cache_t* dst = value_cache + (b * hd + row) * int64_t(block_size) + off;
      store_run<cache_t, kTokTile>(dst, vals, len);
      i += len;
    }
  }
}

// Flash layout ([block][slot][head][d], NHD or HND by strides): row copies.  Same tiling as
// above (16 tokens per CTA, KB 16-byte loads in flight per thread), K pass then V pass so
// that each pass sets its divider up once.
template <typename in_t, typename cache_t, int KV>
__global__ void __launch_bounds__(256)
reshape_and_cache_flash_kernel(const in_t* __restrict__ key, const in_t* __restrict__ value,
                               cache_t* __restrict__ key_cache, cache_t* __restrict__ value_cache,
                               const int64_t* __restrict__ slot_mapping, int64_t block_stride,
                               int64_t page_stride, int64_t head_stride, int64_t key_stride,
                               int64_t value_stride, int num_tokens, int num_heads, int head_size,
                               int block_size, int vec_ok, const float* __restrict__ k_scale_ptr,
                               const float* __restrict__ v_scale_ptr) {
  __shared__ TileSlots ts;
  const int tok0 = blockIdx.x * kTokTile;
  const int ntok = min(kTokTile, num_tokens - tok0);
  load_tile_slots(ts, slot_mapping, tok0, ntok, block_size);
  const float k_scale_f = (KV == kKvAuto) ? 1.f : *k_scale_ptr;
  const float v_scale_f = (KV == kKvAuto) ? 1.f : *v_scale_ptr;
  constexpr int VEC = 16 / sizeof(in_t);  // elements per 16-byte read
  constexpr int KB = 4;

#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const in_t* src_base = pass ? value : key;
    cache_t* dst_base = pass ? value_cache : key_cache;
    const int64_t src_stride = pass ? value_stride : key_stride;
    const float scale_f = pass ? v_scale_f : k_scale_f;
    const ScaledDiv scale(scale_f);
    if (vec_ok && (KV == kKvAuto || scale.fast)) {
      const int vec_per_head = head_size / VEC;
      const int per_tok = num_heads * vec_per_head;
      const int items = ntok * per_tok;
      const SmallDiv by_tok(per_tok), by_head(vec_per_head);
      for (int it0 = threadIdx.x; it0 < items; it0 += KB * blockDim.x) {
        __align__(16) in_t in[KB][VEC];
        cache_t* dst[KB];
#pragma unroll
        for (int k = 0; k < KB; ++k) {
          const int it = it0 + k * blockDim.x;
          dst[k] = nullptr;
          if (it < items) {
            const int t = int(by_tok(it));
            const int j = it - t * per_tok;
            const int h = int(by_head(j));
            const int e = (j - h * vec_per_head) * VEC;
            const int64_t b = ts.blk[t];
            if (b >= 0) {
              dst[k] = dst_base + b * block_stride + ts.off[t] * page_stride + h * head_stride + e;
              *reinterpret_cast<uint4*>(in[k]) = *reinterpret_cast<const uint4*>(
                  src_base + int64_t(tok0 + t) * src_stride + h * head_size + e);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < KB; ++k) {
          if (dst[k] != nullptr) {
            __align__(16) cache_t outv[VEC];
            convert_n<in_t, cache_t, KV, VEC>(in[k], outv, scale);
            if constexpr (sizeof(cache_t) * VEC == 16) {
              *reinterpret_cast<uint4*>(dst[k]) = *reinterpret_cast<const uint4*>(outv);
            } else if constexpr (sizeof(cache_t) * VEC == 8) {
              *reinterpret_cast<uint2*>(dst[k]) = *reinterpret_cast<const uint2*>(outv);
            } else {
              *reinterpret_cast<uint32_t*>(dst[k]) = *reinterpret_cast<const uint32_t*>(outv);
            }
          }
        }
      }
    } else {
      const int hd = num_heads * head_size;
      for (int i = threadIdx.x; i < ntok * hd; i += blockDim.x) {
        const int t = i / hd, r = i % hd;
        if (ts.blk[t] < 0) continue;
        const int h = r / head_size, e = r % head_size;
        const in_t v = src_base[int64_t(tok0 + t) * src_stride + r];
        cache_t q;
        if constexpr (KV == kKvAuto) q = v;
        else q = f32_to_fp8<KV == kKvE5M2>(__fdiv_rn(to_f32(v), scale_f));
        dst_base[ts.blk[t] * block_stride + ts.off[t] * page_stride + h * head_stride + e] = q;
      }
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
    dim3 grid((a.num_tokens + kTokTile - 1) / kTokTile);
    reshape_and_cache_flash_kernel<in_t, cache_t, KV><<<grid, threads, 0, stream>>>(
        static_cast<const in_t*>(a.key), static_cast<const in_t*>(a.value),
        static_cast<cache_t*>(a.key_cache), static_cast<cache_t*>(a.value_cache), a.slot_mapping,
        a.block_stride, a.page_stride, a.head_stride, a.key_stride, a.value_stride, a.num_tokens,
        a.num_heads, a.head_size, a.block_size, vec_ok ? 1 : 0, a.k_scale, a.v_scale);
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
