// KV-write kernels: scatter new K/V tokens into the paged cache, optionally
// quantising to fp8.  Replaces the reference's reshape_and_cache_kernel,
// reshape_and_cache_flash_kernel and convert_fp8_kernel
// (csrc/cache_kernels.cu:225-283, :285-358, :826-899).
//
// The work is pure data movement, so the design goal is full-sector traffic:
//   * x-layout K: one 16-byte store per (token, head, d/x) chunk.
//   * x-layout V is a transpose ([token][d] -> [d][token-in-block]).  A CTA owns
//     a tile of 16 consecutive tokens.  When the tile fills 16 consecutive slots
//     of one block (prefill, chunked writes) a thread reads 8 bytes of 4 d per
//     token and writes 4 rows of 16 tokens with 16-byte stores; otherwise each
//     thread owns one (head, d) row, reads its element of all 16 tokens at once
//     and writes four bytes at a time wherever tokens landed in consecutive,
//     aligned slots, instead of one 1-2 byte store per element.
//   * flash layout: 16-byte vector row copies, NHD or HND by strides.
// Quantisation is cvt.rn.satfinite of the correctly rounded fp32 quotient x / scale,
// bit-identical to the reference's scaled_convert (quant_utils.cuh:469-502).
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace b200pa {

enum : int { kKvAuto = 0, kKvE4M3 = 1, kKvE5M2 = 2 };

// x / scale, correctly rounded, for one scale and many x.  The compiler's division spends a
// MUFU.RCP, a range check and a slow-path branch on every element, which made the KV write
// XU-bound; here the reciprocal is taken once and each quotient is the product x * r followed
// by two residual corrections q += fma(-q, s, x) * r.  The first leaves q within one ulp, the
// second then yields the correctly rounded quotient (Markstein's theorem; r is the correctly
// rounded reciprocal).  Used for positive scales within 2^+-60: there a residual can only
// lose bits to underflow for |x / s| < 2^-42, which is zero in both fp8 formats whatever its
// last bits are.  Other scales use the division.
struct ScaledDiv {
  float s, r;
  bool fast;
  uint64_t s2, nr2;  // {s, s} and {-r, -r} for the packed fp32 pipe
  __device__ __forceinline__ explicit ScaledDiv(float scale) : s(scale) {
    r = __fdiv_rn(1.f, scale);
    fast = scale >= 0x1p-60f && scale <= 0x1p60f;
    const float nr = -r;
    asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(s));
    asm("mov.b64 %0, {%1, %1};" : "=l"(nr2) : "f"(nr));
  }
  // MINUS the two quotients, on the packed fp32 pipe (fma.rn.f32x2, sm_100).  The sequence
  // runs on the negated quotient q' = -x/s because that keeps the sign of a zero:
  //   q' = x * (-r);  e = fma(q', s, x) = x - q*s;  q' = fma(e, -r, q')
  // gives q' = -0 for x = +0 and +0 for x = -0, where the same steps on q itself turn -0
  // into +0.  The caller flips the sign bit of the fp8 codes instead (one XOR per four
  // codes).  An infinite or overflowing quotient comes out as NaN (inf - inf); the caller
  // sees its NaN code and redoes those elements with the division.
  // Callers check `fast` once per kernel, not per pair.
  __device__ __forceinline__ void neg_pair(float x0, float x1, float& o0, float& o1) const {
    asm("{\n"
        " .reg .b64 x, q, e;\n"
        " mov.b64 x, {%2, %3};\n"
        " mul.rn.f32x2 q, x, %4;\n"
        " fma.rn.f32x2 e, q, %5, x;\n"
        " fma.rn.f32x2 q, e, %4, q;\n"
        " fma.rn.f32x2 e, q, %5, x;\n"
        " fma.rn.f32x2 q, e, %4, q;\n"
        " mov.b64 {%0, %1}, q;\n"
        "}"
        : "=f"(o0), "=f"(o1)
        : "f"(x0), "f"(x1), "l"(nr2), "l"(s2));
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

// Four 16-bit inputs (two 32-bit words of two elements each) -> four fp8 codes of MINUS the
// quotients x / s (ScaledDiv::neg_pair explains the sign), in one asm block so that the
// packed-fp32 register pairs are formed where the values are produced and no moves are
// needed around the packed instructions.
template <typename in_t, bool kE5M2>
__device__ __forceinline__ uint32_t neg_quant4(uint32_t w0, uint32_t w1, const ScaledDiv& div) {
  uint32_t out;
  if constexpr (std::is_same_v<in_t, __nv_bfloat16>) {
    if constexpr (kE5M2) {
      asm("{\n"
          " .reg .b32 a0, a1, b0, b1;\n"
          " .reg .b64 x, y, q, r, e;\n"
          " .reg .b16 lo, hi;\n"
          " shl.b32 a0, %1, 16;\n and.b32 a1, %1, 0xffff0000;\n"
          " shl.b32 b0, %2, 16;\n and.b32 b1, %2, 0xffff0000;\n"
          " mov.b64 x, {a0, a1};\n mov.b64 y, {b0, b1};\n"
          " mul.rn.f32x2 q, x, %3;\n mul.rn.f32x2 r, y, %3;\n"
          " fma.rn.f32x2 e, q, %4, x;\n fma.rn.f32x2 q, e, %3, q;\n"
          " fma.rn.f32x2 e, r, %4, y;\n fma.rn.f32x2 r, e, %3, r;\n"
          " fma.rn.f32x2 e, q, %4, x;\n fma.rn.f32x2 q, e, %3, q;\n"
          " fma.rn.f32x2 e, r, %4, y;\n fma.rn.f32x2 r, e, %3, r;\n"
          " mov.b64 {a0, a1}, q;\n mov.b64 {b0, b1}, r;\n"
          " cvt.rn.satfinite.e5m2x2.f32 lo, a1, a0;\n"
          " cvt.rn.satfinite.e5m2x2.f32 hi, b1, b0;\n"
          " mov.b32 %0, {lo, hi};\n"
          "}"
          : "=r"(out)
          : "r"(w0), "r"(w1), "l"(div.nr2), "l"(div.s2));
    } else {
      asm("{\n"
          " .reg .b32 a0, a1, b0, b1;\n"
          " .reg .b64 x, y, q, r, e;\n"
          " .reg .b16 lo, hi;\n"
          " shl.b32 a0, %1, 16;\n and.b32 a1, %1, 0xffff0000;\n"
          " shl.b32 b0, %2, 16;\n and.b32 b1, %2, 0xffff0000;\n"
          " mov.b64 x, {a0, a1};\n mov.b64 y, {b0, b1};\n"
          " mul.rn.f32x2 q, x, %3;\n mul.rn.f32x2 r, y, %3;\n"
          " fma.rn.f32x2 e, q, %4, x;\n fma.rn.f32x2 q, e, %3, q;\n"
          " fma.rn.f32x2 e, r, %4, y;\n fma.rn.f32x2 r, e, %3, r;\n"
          " fma.rn.f32x2 e, q, %4, x;\n fma.rn.f32x2 q, e, %3, q;\n"
          " fma.rn.f32x2 e, r, %4, y;\n fma.rn.f32x2 r, e, %3, r;\n"
          " mov.b64 {a0, a1}, q;\n mov.b64 {b0, b1}, r;\n"
          " cvt.rn.satfinite.e4m3x2.f32 lo, a1, a0;\n"
          " cvt.rn.satfinite.e4m3x2.f32 hi, b1, b0;\n"
          " mov.b32 %0, {lo, hi};\n"
          "}"
          : "=r"(out)
          : "r"(w0), "r"(w1), "l"(div.nr2), "l"(div.s2));
    }
  } else {
    const __half2 h0 = *reinterpret_cast<const __half2*>(&w0);
    const __half2 h1 = *reinterpret_cast<const __half2*>(&w1);
    float q0, q1, q2, q3;
    div.neg_pair(__low2float(h0), __high2float(h0), q0, q1);
    div.neg_pair(__low2float(h1), __high2float(h1), q2, q3);
    out = uint32_t(f32x2_to_fp8x2<kE5M2>(q0, q1)) | (uint32_t(f32x2_to_fp8x2<kE5M2>(q2, q3)) << 16);
  }
  return out;
}

// N consecutive elements.  fp8: four at a time - two pair conversions of the negated
// quotients, sign bits flipped back in the assembled word; a group of up to 16 codes that holds
// a NaN code (a NaN, or a quotient that overflowed inside neg_pair) is redone with the division,
// which is rare.
template <typename in_t, typename cache_t, int KV, int N>
__device__ __forceinline__ void convert_n(const in_t (&in)[N], cache_t* out, const ScaledDiv& div) {
  if constexpr (KV == kKvAuto) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = in[i];
  } else if constexpr (N % 4 == 0) {
    constexpr bool kE5 = KV == kKvE5M2;
    if (!div.fast) {  // the same for every thread of the launch
#pragma unroll
      for (int i = 0; i < N; ++i) out[i] = f32_to_fp8<kE5>(__fdiv_rn(to_f32(in[i]), div.s));
      return;
    }
    uint32_t w[N / 4];
    uint32_t nan_bits = 0;
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      uint32_t v;
      if constexpr (sizeof(in_t) == 2) {
        uint32_t w0, w1;
        const uint16_t b0 = *reinterpret_cast<const uint16_t*>(&in[i]);
        const uint16_t b1 = *reinterpret_cast<const uint16_t*>(&in[i + 1]);
        const uint16_t b2 = *reinterpret_cast<const uint16_t*>(&in[i + 2]);
        const uint16_t b3 = *reinterpret_cast<const uint16_t*>(&in[i + 3]);
        w0 = uint32_t(b0) | (uint32_t(b1) << 16);
        w1 = uint32_t(b2) | (uint32_t(b3) << 16);
        v = neg_quant4<in_t, kE5>(w0, w1, div);
      } else {
        float q0, q1, q2, q3;
        div.neg_pair(to_f32(in[i]), to_f32(in[i + 1]), q0, q1);
        div.neg_pair(to_f32(in[i + 2]), to_f32(in[i + 3]), q2, q3);
        v = uint32_t(f32x2_to_fp8x2<kE5>(q0, q1)) | (uint32_t(f32x2_to_fp8x2<kE5>(q2, q3)) << 16);
      }
      // a byte whose low seven bits are all ones is a NaN code in both formats
      nan_bits |= ((v & 0x7F7F7F7Fu) + 0x01010101u) & 0x80808080u;
      w[i / 4] = v ^ 0x80808080u;
    }
    if (nan_bits != 0) {
#pragma unroll
      for (int i = 0; i < N; i += 4) {
        uint32_t v = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          v |= uint32_t(f32_to_fp8<kE5>(__fdiv_rn(to_f32(in[i + k]), div.s))) << (8 * k);
        w[i / 4] = v;
      }
    }
#pragma unroll
    for (int i = 0; i < N / 4; ++i) reinterpret_cast<uint32_t*>(out)[i] = w[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = f32_to_fp8<KV == kKvE5M2>(div(to_f32(in[i])));
  }
}

// The same conversion for 16-bit inputs that are already in registers as 32-bit words of two
// elements each (what 16-byte loads deliver): NW input words -> NW / 2 words of fp8 codes.  Works
// on the words directly, so nothing is unpacked into elements and packed again.
template <typename in_t, int KV, int NW>
__device__ __forceinline__ void convert_words(const uint32_t (&w)[NW], uint32_t (&out)[NW / 2],
                                              const ScaledDiv& div) {
  static_assert(sizeof(in_t) == 2 && KV != kKvAuto && NW % 2 == 0, "16-bit inputs, fp8 cache");
  constexpr bool kE5 = KV == kKvE5M2;
  auto slow4 = [&](uint32_t w0, uint32_t w1) -> uint32_t {
    const in_t* e0 = reinterpret_cast<const in_t*>(&w0);
    const in_t* e1 = reinterpret_cast<const in_t*>(&w1);
    return uint32_t(f32_to_fp8<kE5>(__fdiv_rn(to_f32(e0[0]), div.s))) |
           (uint32_t(f32_to_fp8<kE5>(__fdiv_rn(to_f32(e0[1]), div.s))) << 8) |
           (uint32_t(f32_to_fp8<kE5>(__fdiv_rn(to_f32(e1[0]), div.s))) << 16) |
           (uint32_t(f32_to_fp8<kE5>(__fdiv_rn(to_f32(e1[1]), div.s))) << 24);
  };
  if (!div.fast) {  // the same for every thread of the launch
#pragma unroll
    for (int i = 0; i < NW; i += 2) out[i / 2] = slow4(w[i], w[i + 1]);
    return;
  }
  uint32_t nan_bits = 0;
#pragma unroll
  for (int i = 0; i < NW; i += 2) {
    const uint32_t v = neg_quant4<in_t, kE5>(w[i], w[i + 1], div);
    nan_bits |= (v & 0x7F7F7F7Fu) + 0x01010101u;  // bit 7 of a byte: its low seven bits were all ones
    out[i / 2] = v ^ 0x80808080u;
  }
  if ((nan_bits & 0x80808080u) != 0) {
#pragma unroll
    for (int i = 0; i < NW; i += 2) out[i / 2] = slow4(w[i], w[i + 1]);
  }
}

}  // namespace b200pa

#include "kv_write_staged.cuh"

namespace b200pa {

constexpr int kTokTile = 16;

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
// tokens (block -1 = padding token, skipped), whether the tile fills 16 consecutive slots
// that start at a multiple of 16 (true for prefill and chunked writes whose sequences start
// on a tile boundary), and for every other tile how its tokens go into a V row of the
// x-layout: `cnt[t]` = 0 when token t is written together with an earlier one, else the
// number of tokens from t on that sit in consecutive slots at a 4-byte aligned address and
// fill one 4-byte store (4 / element size), else 1.
struct TileSlots {
  int64_t blk[kTokTile];
  int off[kTokTile];
  int cnt[kTokTile];
  int full_run;
};

__device__ __forceinline__ void load_tile_slots(TileSlots& ts, const int64_t* __restrict__ slot_mapping,
                                                int tok0, int ntok, int block_size, int elem_size) {
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
    // 4-byte groups: token t can start one when its slot is 4-byte aligned inside a block whose
    // rows are (block_size * elem_size is a multiple of 4 for every supported block size) and
    // the next w - 1 tokens follow in the same block
    const int w = elem_size >= 4 ? 1 : 4 / elem_size;
    bool start = false;
    if (w > 1) {
      const int64_t b = slot >= 0 ? slot / block_size : int64_t(-1);
      const int off = slot >= 0 ? int(slot - b * block_size) : 0;
      bool follows = true;  // tokens t+1 .. t+w-1 continue t's run inside its block
      for (int k = 1; k < w; ++k) {
        const int64_t sk = __shfl_down_sync(0xffffffffu, slot, k);
        follows &= (t + k < kTokTile) && sk == slot + k;
      }
      start = slot >= 0 && follows && (off * elem_size) % 4 == 0 && off + w <= block_size &&
              (block_size * elem_size) % 4 == 0;
    }
    // groups cannot overlap (two starts inside one run are at least w tokens apart, because
    // both are aligned): a token is covered when one of the w - 1 tokens before it starts one
    const unsigned starts = __ballot_sync(0xffffffffu, start);
    unsigned covered = 0;
    for (int k = 1; k < w; ++k) covered |= starts << k;
    if (t < kTokTile) ts.cnt[t] = ((starts >> t) & 1u) ? w : (((covered >> t) & 1u) ? 0 : 1);
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

// V of every tile that is not 16 aligned consecutive slots (decode steps: each token in a
// block of its own; prefill whose sequences do not start on a tile boundary: runs of
// consecutive slots).  A thread owns one (head, d) row: it reads the row's element of every
// token of the tile (independent loads, adjacent threads adjacent addresses), converts them,
// and stores them as the tile's plan says - four bytes at a time where consecutive tokens
// allow it, else one element.  Out of line: it must not cost the common path registers.
template <typename in_t, typename cache_t, int KV>
__device__ __noinline__ void reshape_tile_v_general(const TileSlots& ts, const in_t* __restrict__ value,
                                                    cache_t* __restrict__ value_cache,
                                                    int64_t value_stride, int tok0, int ntok, int h0,
                                                    int nh, int head_size, int hd, int block_size,
                                                    const ScaledDiv& v_scale) {
  constexpr int W4 = sizeof(cache_t) >= 4 ? 1 : 4 / int(sizeof(cache_t));  // tokens per 4-byte store
  for (int row = h0 * head_size + threadIdx.x; row < (h0 + nh) * head_size; row += blockDim.x) {
    const in_t* src = value + int64_t(tok0) * value_stride + row;
    in_t raw[kTokTile];
#pragma unroll
    for (int t = 0; t < kTokTile; ++t)
      raw[t] = (t < ntok && ts.blk[t] >= 0) ? src[int64_t(t) * value_stride] : in_t(0.f);
    __align__(16) cache_t conv[kTokTile];
    convert_n<in_t, cache_t, KV, kTokTile>(raw, conv, v_scale);
#pragma unroll
    for (int t = 0; t < kTokTile; ++t) {
      const int n = ts.cnt[t];  // the same for every thread of the CTA
      if (n == 0 || t >= ntok || ts.blk[t] < 0) continue;
      cache_t* dst = value_cache + (ts.blk[t] * hd + row) * int64_t(block_size) + ts.off[t];
      if (W4 > 1 && n == W4 && t + W4 <= kTokTile) {
        __align__(4) cache_t four[W4];
#pragma unroll
        for (int k = 0; k < W4; ++k) four[k] = conv[(t + k) % kTokTile];
        *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(four);
      } else {
        *dst = conv[t];
      }
    }
  }
}

// grid.x = ceil(num_tokens / kTokTile), grid.y = parts the heads are split into (small
// writes - decode steps - would otherwise occupy a handful of SMs); block = 256 threads.
template <typename in_t, typename cache_t, int KV>
__global__ void __launch_bounds__(256, 3)
reshape_and_cache_kernel(const in_t* __restrict__ key, const in_t* __restrict__ value,
                         cache_t* __restrict__ key_cache, cache_t* __restrict__ value_cache,
                         const int64_t* __restrict__ slot_mapping, int64_t key_stride,
                         int64_t value_stride, int num_tokens, int num_heads, int head_size,
                         int block_size, int x, const float* __restrict__ k_scale_ptr,
                         const float* __restrict__ v_scale_ptr) {
  __shared__ TileSlots ts;
  const int tok0 = blockIdx.x * kTokTile;
  const int ntok = min(kTokTile, num_tokens - tok0);
  load_tile_slots(ts, slot_mapping, tok0, ntok, block_size, int(sizeof(cache_t)));

  const float k_scale_f = (KV == kKvAuto) ? 1.f : *k_scale_ptr;
  const float v_scale_f = (KV == kKvAuto) ? 1.f : *v_scale_ptr;
  const ScaledDiv k_scale(k_scale_f), v_scale(v_scale_f);
  const int chunks = head_size / x;  // per head
  const int hd = num_heads * head_size;
  // this CTA's heads
  const int heads_per = (num_heads + gridDim.y - 1) / gridDim.y;
  const int h0 = blockIdx.y * heads_per;
  const int nh = min(heads_per, num_heads - h0);
  if (nh <= 0) return;
  // 16-byte loads from key/value rows are legal when bases and row strides are 16-byte
  // multiples; x elements = 16 bytes of cache in the standard layout
  const bool vec_ok =
      ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
        reinterpret_cast<uintptr_t>(key_cache) | (size_t(key_stride) * sizeof(in_t)) |
        (size_t(value_stride) * sizeof(in_t)) | (size_t(head_size) * sizeof(in_t)) |
        (size_t(x) * sizeof(in_t))) & 15) == 0 &&
      x * int(sizeof(cache_t)) == 16 && (KV == kKvAuto || (k_scale.fast && v_scale.fast));
  if (!vec_ok) {
    if (blockIdx.y == 0)
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
    const int per_tok = nh * chunks;
    const int k_items = ntok * per_tok;
    const SmallDiv by_tok(per_tok), by_chunks(chunks);
    const int e0 = h0 * head_size;  // first element of this CTA's heads in a token row
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
          const int hl = int(by_chunks(j));
          const int c = j - hl * chunks;
          const int64_t b = ts.blk[t];
          if (b >= 0) {
            // j * x = hl * head_size + c * x
            const in_t* src = key + int64_t(tok0 + t) * key_stride + e0 + j * x;
            dst[k] = key_cache +
                     (((b * num_heads + h0 + hl) * chunks + c) * int64_t(block_size) + ts.off[t]) * x;
#pragma unroll
            for (int i = 0; i < L; ++i)
              reinterpret_cast<uint4*>(in[k])[i] = reinterpret_cast<const uint4*>(src)[i];
          }
        }
      }
#pragma unroll
      for (int k = 0; k < KB; ++k) {
        if (dst[k] != nullptr) {
          if constexpr (KV != kKvAuto && sizeof(in_t) == 2) {
            uint32_t wi[8], wo[4];
#pragma unroll
            for (int i = 0; i < 8; ++i) wi[i] = reinterpret_cast<const uint32_t*>(in[k])[i];
            convert_words<in_t, KV, 8>(wi, wo, k_scale);
            *reinterpret_cast<uint4*>(dst[k]) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
          } else {
            __align__(16) cache_t vals[N];
            convert_n<in_t, cache_t, KV, N>(in[k], vals, k_scale);
            *reinterpret_cast<uint4*>(dst[k]) = *reinterpret_cast<const uint4*>(vals);
          }
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
    const int groups = nh * head_size / VD;
    for (int gidx = threadIdx.x; gidx < groups; gidx += blockDim.x) {
      const int row0 = h0 * head_size + gidx * VD;  // (head, d) flattened; a group never straddles a head
      const in_t* src = value + int64_t(tok0) * value_stride + row0;
      __align__(8) in_t in[kTokTile][VD];
#pragma unroll
      for (int t = 0; t < kTokTile; ++t)
        *reinterpret_cast<uint2*>(in[t]) = *reinterpret_cast<const uint2*>(src + int64_t(t) * value_stride);
      __align__(16) cache_t vals[VD][kTokTile];
      if constexpr (KV != kKvAuto && sizeof(in_t) == 2) {
        // token t's 8 bytes are two words: (d0, d1) and (d2, d3).  The cache row of d0 needs the
        // low halves of the first words of consecutive tokens, d1 the high halves, and so on: one
        // byte permute per pair of tokens.
#pragma unroll
        for (int d = 0; d < VD; ++d) {
          const uint32_t sel = (d & 1) ? 0x7632u : 0x5410u;
          uint32_t wi[kTokTile / 2], wo[kTokTile / 4];
#pragma unroll
          for (int t = 0; t < kTokTile; t += 2)
            wi[t / 2] = __byte_perm(reinterpret_cast<const uint32_t*>(in[t])[d >> 1],
                                    reinterpret_cast<const uint32_t*>(in[t + 1])[d >> 1], sel);
          convert_words<in_t, KV, kTokTile / 2>(wi, wo, v_scale);
#pragma unroll
          for (int i = 0; i < kTokTile / 4; ++i) reinterpret_cast<uint32_t*>(vals[d])[i] = wo[i];
        }
      } else {
#pragma unroll
        for (int t = 0; t < kTokTile; t += 4) {
#pragma unroll
          for (int d = 0; d < VD; ++d) {
            const in_t four[4] = {in[t][d], in[t + 1][d], in[t + 2][d], in[t + 3][d]};
            convert_n<in_t, cache_t, KV, 4>(four, &vals[d][t], v_scale);
          }
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

  reshape_tile_v_general<in_t, cache_t, KV>(ts, value, value_cache, value_stride, tok0, ntok, h0, nh,
                                            head_size, hd, block_size, v_scale);
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
  load_tile_slots(ts, slot_mapping, tok0, ntok, block_size, int(sizeof(cache_t)));
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
            if constexpr (KV != kKvAuto && sizeof(in_t) == 2) {
              uint32_t wi[4], wo[2];
#pragma unroll
              for (int i = 0; i < 4; ++i) wi[i] = reinterpret_cast<const uint32_t*>(in[k])[i];
              convert_words<in_t, KV, 4>(wi, wo, scale);
              reinterpret_cast<uint32_t*>(outv)[0] = wo[0];
              reinterpret_cast<uint32_t*>(outv)[1] = wo[1];
            } else {
              convert_n<in_t, cache_t, KV, VEC>(in[k], outv, scale);
            }
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
static int cache_sm_count() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

// The staged kernel takes 16-bit key/value tensors whose rows, and the cache's 16-byte chunks,
// are 16-byte aligned.  Returns false when the call does not qualify (the caller then uses the
// plain kernels); otherwise launches and stores the return code in *rc.
template <typename in_t, typename cache_t, int KV, bool kFlash, bool kShift>
static bool launch_staged_as(const b200pa_cache_args& a, cudaStream_t stream, int* rc, int hsplit) {
  if constexpr (sizeof(in_t) != 2 || sizeof(cache_t) > 2) {
    return false;
  } else {
    constexpr int E = sizeof(cache_t);
    auto al16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    const int D = a.head_size;
    if (D % 16 != 0 || D > 512) return false;
    if (!al16(a.key) || !al16(a.value) || !al16(a.key_cache) || !al16(a.value_cache)) return false;
    if ((a.key_stride * 2) % 16 != 0 || (a.value_stride * 2) % 16 != 0) return false;
    if (kFlash) {
      if ((a.block_stride * E) % 16 != 0 || (a.page_stride * E) % 16 != 0 || (a.head_stride * E) % 16 != 0)
        return false;
    } else {
      if (a.x != 16 / E || (a.block_size * E) % 4 != 0) return false;
    }
    StagedWriteParams p{};
    p.key = a.key;
    p.value = a.value;
    p.key_cache = a.key_cache;
    p.value_cache = a.value_cache;
    p.slot_mapping = a.slot_mapping;
    p.k_scale = a.k_scale;
    p.v_scale = a.v_scale;
    p.status = device_status_ptr();
    if (p.status == nullptr) return false;
    p.key_stride = a.key_stride;
    p.value_stride = a.value_stride;
    p.block_stride = a.block_stride;
    p.page_stride = a.page_stride;
    p.head_stride = a.head_stride;
    p.num_tokens = a.num_tokens;
    p.num_heads = a.num_heads;
    p.head_size = D;
    p.block_size = a.block_size;
    p.hsplit = hsplit;
    p.nstages = 2;
    int max_warps = kStagedMaxWarps;
    {  // developer knobs, read once
      static const int kn_stages = [] { const char* e = getenv("B200PA_TUNE_KVW_STAGES"); return e ? atoi(e) : 0; }();
      static const int kn_warps = [] { const char* e = getenv("B200PA_TUNE_KVW_WARPS"); return e ? atoi(e) : 0; }();
      if (kn_stages >= 1 && kn_stages <= 8) p.nstages = kn_stages;
      if (kn_warps >= 4 && kn_warps <= kStagedMaxWarps) max_warps = kn_warps;
    }
    p.pitch = D / p.hsplit * 2 + 16;
    p.stage_bytes = kStagedTile * p.pitch + 128 + (kShift ? 16 : 0);
    const size_t budget = 220 * 1024;
    int warps = int(std::min<size_t>(max_warps, (budget - 1024) / (size_t(p.nstages) * p.stage_bytes)));
    warps &= ~3;
    if (warps < 4) return false;
    const int64_t items = int64_t((a.num_tokens + kStagedTile - 1) / kStagedTile) * a.num_heads * p.hsplit * 2;
    // few items (decode steps): one per warp, spread over the SMs
    const int sms = cache_sm_count();
    const int per_cta = int(std::min<int64_t>(warps, std::max<int64_t>(4, ((items + sms - 1) / sms + 3) & ~3)));
    const int grid = int(std::min<int64_t>(sms, (items + per_cta - 1) / per_cta));
    const size_t smem = ((size_t(per_cta) * p.nstages * 8 + 127) & ~size_t(127)) +
                        size_t(per_cta) * p.nstages * p.stage_bytes;
    auto kern = kv_write_staged_kernel<in_t, cache_t, KV, kFlash, kShift>;
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && (dev < 0 || dev >= 64 || !done[dev])) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
      if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    }
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    kern<<<grid, per_cta * 32, smem, stream>>>(p);
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_error("KV write kernel launch failed: %s", cudaGetErrorString(e));
      *rc = B200PA_ECUDA;
    } else {
      *rc = B200PA_OK;
    }
    return true;
  }
}

// Picks the variant of the staged kernel for a call.
template <typename in_t, typename cache_t, int KV, bool kFlash>
static bool launch_staged(const b200pa_cache_args& a, cudaStream_t stream, int* rc) {
  static const int kn_hsplit = [] { const char* e = getenv("B200PA_TUNE_KVW_HSPLIT"); return e ? atoi(e) : 0; }();
  static const int kn_shift = [] { const char* e = getenv("B200PA_TUNE_KVW_SHIFT"); return e ? atoi(e) : -1; }();
  // Small writes (decode steps) are bound by the latency of one work item: half a head per
  // item while that still leaves every item a warp of its own (measured: 256 scattered
  // tokens 14.0 -> 11.2 us); large ones pay for the doubled per-item bookkeeping (27 -> 35 us).
  const int64_t items1 = int64_t((a.num_tokens + kStagedTile - 1) / kStagedTile) * a.num_heads * 2;
  const bool small = 2 * items1 <= int64_t(cache_sm_count()) * kStagedMaxWarps;
  const int hsplit = (a.head_size % 128 == 0 && (kn_hsplit == 2 || (kn_hsplit == 0 && small))) ? 2 : 1;
  // Large x-layout writes use the variant that moves tiles onto 16-slot boundaries of the cache
  // (prefill chunks that start inside a block: 16 384 tokens x 8 heads, fp8 51 -> 38 us, 16-bit
  // cache 67 -> 36 us; chunks that start on a boundary are not affected).  Its extra code costs
  // writes of scattered tokens 3-5 us below 4096 tokens (fp8; nothing from 8192 on), and those
  // are decode steps, which have no runs to move.
  bool shift = !kFlash && a.num_tokens >= 4096 && a.block_size % kStagedTile == 0;
  if (kn_shift >= 0) shift = !kFlash && kn_shift != 0 && a.block_size % kStagedTile == 0;
  if constexpr (!kFlash) {
    if (shift) return launch_staged_as<in_t, cache_t, KV, false, true>(a, stream, rc, hsplit);
  }
  return launch_staged_as<in_t, cache_t, KV, kFlash, false>(a, stream, rc, hsplit);
}

template <typename in_t, typename cache_t, int KV>
static int launch_reshape(const b200pa_cache_args& a, cudaStream_t stream, bool flash) {
  if (a.num_tokens == 0) return B200PA_OK;
  // Two implementations; which one is faster was measured per case on B200 (16 384 tokens x 8
  // heads x 128, us, staged / plain): x-layout fp8 29 / 31, flash fp8 27 / 29, x-layout 16-bit
  // cache 27 / 40, 256 scattered tokens (a decode step) 11 / 17, x-layout fp8 with sequences
  // that start inside a block 38 / 92 - and flash with a 16-bit cache 30 / 25, the
  // one case that stays with the plain kernel.  B200PA_TUNE_KVW_STAGED=0/1 forces one of them
  // (for the tests that compare the two).
  static const int kn_staged = [] { const char* e = getenv("B200PA_TUNE_KVW_STAGED"); return e ? atoi(e) : -1; }();
  const bool prefer_staged = !(flash && KV == kKvAuto) || a.num_tokens <= 4096;
  if (kn_staged == 1 || (kn_staged != 0 && prefer_staged)) {
    int rc = B200PA_OK;
    const bool took = flash ? launch_staged<in_t, cache_t, KV, true>(a, stream, &rc)
                            : launch_staged<in_t, cache_t, KV, false>(a, stream, &rc);
    if (took) return rc;
  }
  if (!flash) {
    // small writes (decode steps): split the heads over grid.y so that the write still spreads
    // over the GPU (about two CTAs per SM)
    const int tiles = (a.num_tokens + kTokTile - 1) / kTokTile;
    const int parts = std::max(1, std::min(a.num_heads, (2 * 148 + tiles - 1) / tiles));
    dim3 grid(tiles, parts);
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
