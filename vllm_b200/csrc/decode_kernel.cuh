// Persistent split-KV decode kernel (the hot loop of paged_attention_v1/v2).
// Replaces the reference's paged_attention_kernel
// (csrc/attention/attention_kernels.cuh:81-491).
//
// Design (bandwidth first; the KV cache is read exactly once):
//   * One persistent CTA per SM.  Every WARP is an independent worker that streams
//     KV pages through its own ring of shared-memory slots and writes its results
//     itself.  There is no CTA-wide barrier after set-up, and a warp keeps
//     prefetching pages of its NEXT work item while it finishes the current one, so
//     the pipeline never drains.
//   * Split-KV work is cut by PAGE COUNT, not by sequence: the cache blocks of all
//     (kv head, sequence) pairs form one flat list, every warp takes one contiguous
//     range of equal length, and the pieces of a sequence that a range covers are its
//     work items.  The cut is computed inside the kernel from the real sequence
//     lengths, so every warp reads the same number of bytes whatever the length
//     distribution.  Without scratch memory a work item is a whole (sequence, kv
//     head), dealt out by a fixed stride when there are few and pulled from a global
//     ticket counter when there are many.
//   * The warp that delivers the last partial of a sequence merges all of them
//     (no second launch, nobody waits).
//   * A KV page (one block of one kv head) is contiguous in both cache layouts:
//     K [D/x][B][x] and V [D][B].  Each is fetched with ONE 1-D bulk async copy
//     (cp.async.bulk, completion on an mbarrier; no cluster multicast).
//   * All query heads that share the kv head are processed together on the
//     tensor cores with tokens on the M axis and heads on the 8-wide N axis
//     (mma.sync m16n8k16, fp32 accumulate):
//         S^T[16 tok x 8 heads] = K[16 tok x D] . Q^T          (A = K via ldmatrix)
//         O^T[D x 8 heads]     += V^T[D x 16 tok] . P^T         (A = V via ldmatrix)
//     The x-layout of K and the [D][B] layout of V are exactly the row-major A
//     operands these products need, so pages are used as they land, untransposed.
//     P^T is produced from the S^T accumulators with one movmatrix per 8 tokens.
//   * fp8 caches are dequantised after ldmatrix (4 bytes per lane) with
//     cvt.rn.f16x2.e4m3x2; the dot-product index order inside a 16-wide k-step is
//     permuted consistently in Q / P, which is free.  k_scale is folded into the
//     logit scale and v_scale into the output scale.
//   * Online softmax in the log2 domain, fp32 state, warp-shuffle reductions.
//   * Every mbarrier wait is bounded; on expiry the warp records a status code
//     and leaves.
#pragma once

#include <type_traits>

#include "decode_common.cuh"

namespace b200pa {

enum : int { kCache16 = 0, kCacheE4M3 = 1, kCacheE5M2 = 2 };

// Cache blocks per pipeline step of the decode kernel: 2 for 16-token blocks whose K page is
// at most 1 KiB, else 1 (measured: pairing 1 KiB pages gains 6-9 %, pairing 2 KiB pages loses
// 1-5 %).  esize = bytes per cache element, bt = 16-token tiles per block.
constexpr int decode_pages_per_step(int esize, int d, int bt) {
  return (bt == 1 && d * 16 * esize <= 1024) ? 2 : 1;
}

struct WorkItem {
  int seq;
  int kvh;
  int hg;          // head group inside the kv head
  int part;        // partition index inside the sequence
  int nparts;      // partitions of this sequence (>= 1)
  int tok_begin;
  int tok_end;
  int first_page;
  int npages;
  int win;         // which 32-page window `bt` holds
  int bt;          // per-lane block id of page first_page + 32*win + lane
  bool valid;
};

template <typename QT, int KV, int D, int GP>
struct DecodeTraits {
  static constexpr bool kFp8 = KV != kCache16;
  static constexpr bool kMmaBf16 = !kFp8 && std::is_same_v<QT, __nv_bfloat16>;
  static constexpr int kEsize = kFp8 ? 1 : 2;
  static constexpr int kKSteps = D / 16;   // k-steps of QK / m-tiles of PV
  static constexpr int kHeadsPerItem = 8 * GP;
};

// Reads this lane's block id for the 32-page window `win` of an item.
__device__ __forceinline__ int load_bt(const DecodeParams& p, const WorkItem& it, int win, int lane) {
  const int pg = win * 32 + lane;
  if (pg >= it.npages) return 0;
  return __ldg(p.block_tables + int64_t(it.seq) * p.max_blocks_per_seq + it.first_page + pg);
}

// Sequences cut into more than kMergeDirectMax pieces are merged in two levels: the pieces form
// groups of kMergeFan consecutive ones, the warp that completes a group merges it into one
// partial (kept in the group's first slot), and the warp that completes the last group merges
// the groups.  One warp merging 60 partials of four heads takes ~14 us, which would be the
// tail of the launch; groups are merged by different warps as they finish.
constexpr int kMergeFan = 8;
constexpr int kMergeDirectMax = 32;  // (16 measured 2 % slower on a 4-way kv-head shard, equal elsewhere)

// Merges split-KV partials of `nheads` consecutive heads of one sequence (the reference's
// paged_attention_v2_reduce_kernel, attention_kernels.cuh:559-664, for one warp).
// Partial j of head h has its (max logit, exp sum) at index row0 + h*P + j*pstride of
// max_logits / exp_sums and its normalised output at that index times D in tmp.
//   group == false: writes out = sum_j w_j O_j with w_j = l_j 2^(m_j-M) / (sum + 1e-6) to
//     outp + h*out_head_stride, and the log-sum-exp if asked.
//   group == true (pstride 1, 2 <= np <= 32): the same sum with w_j = l_j 2^(m_j-M) / sum goes
//     into partial 0's slot of tmp (outp points there) and (M, sum) into its statistics, so that
//     the slot again holds a partial in the format above.
// This is the general form (any number of partials and heads): the weights go through memory
// (it overwrites exp_sums with them), three dependent round trips.
template <typename QT, int D>
__device__ __noinline__ void merge_partials_general(float* exp_sums, float* max_logits, const QT* tmp,
                                            QT* outp, int64_t out_head_stride, int64_t row0, int np,
                                            int P, int pstride, int nheads, int lane, float* lse,
                                            int lse_stride, bool group) {
  constexpr bool kOutBf = std::is_same_v<QT, __nv_bfloat16>;
  // Phase 1: per head, turn (max logit, exp sum) of its partials into normalised weights.
  // Lanes run over partials, four heads share one memory round trip.
  for (int h0 = 0; h0 < nheads; h0 += 4) {
    float ml0[4], es0[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool ok = h0 + k < nheads && lane < np;
      const int64_t at = row0 + int64_t(ok ? h0 + k : h0) * P + int64_t(ok ? lane : 0) * pstride;
      ml0[k] = ok ? __ldcg(max_logits + at) : -INFINITY;
      es0[k] = ok ? __ldcg(exp_sums + at) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (h0 + k >= nheads) break;  // warp-uniform
      float* ml = max_logits + row0 + int64_t(h0 + k) * P;
      float* es = exp_sums + row0 + int64_t(h0 + k) * P;
      float mx = ml0[k];
      for (int j = lane + 32; j < np; j += 32) mx = fmaxf(mx, __ldcg(ml + int64_t(j) * pstride));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float w0 = lane < np ? es0[k] * fast_exp2(ml0[k] - mx) : 0.f;
      float sum = w0;
      for (int j = lane + 32; j < np; j += 32) {
        const float w = __ldcg(es + int64_t(j) * pstride) * fast_exp2(__ldcg(ml + int64_t(j) * pstride) - mx);
        es[int64_t(j) * pstride] = w;
        sum += w;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float winv = __fdividef(1.f, group ? sum : sum + 1e-6f);
      if (lane < np) es[int64_t(lane) * pstride] = w0 * winv;
      for (int j = lane + 32; j < np; j += 32) es[int64_t(j) * pstride] *= winv;
      if (group) {
        // every lane has its max logits in registers (np <= 32): their slots can take the
        // merged statistics; the exp sum waits in partial 1's slot until the weights are used
        __syncwarp();
        if (lane == 0) {
          ml[0] = mx;
          ml[1] = sum;
        }
      }
      // log-sum-exp of the whole sequence (logits are kept in the log2 domain)
      if (!group && lse != nullptr && lane == 0)
        lse[int64_t(h0 + k) * lse_stride] = (mx + log2f(sum)) * kLn2;
    }
  }
  __syncwarp();  // weights written by other lanes are read below
  // Phase 2: out = sum_j weight_j * partial_j.  Work unit = 8 consecutive output elements
  // (16 bytes) of one head; every load is independent of every other.
  constexpr int UPH = D / 8;  // units per head
  const int units = nheads * UPH;
  const int64_t jstep = int64_t(pstride) * D;
  auto fma8 = [&](float* acc, float w, const uint4& v) {
    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f0, f1;
      if constexpr (kOutBf) {
        f0 = __uint_as_float(vv[i] << 16);
        f1 = __uint_as_float(vv[i] & 0xffff0000u);
      } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&vv[i]);
        f0 = __low2float(h);
        f1 = __high2float(h);
      }
      acc[2 * i] += w * f0;
      acc[2 * i + 1] += w * f1;
    }
  };
  auto store8 = [&](QT* dst, const float* acc) {
    uint4 o4;
    o4.x = pack2<kOutBf>(acc[0], acc[1]);
    o4.y = pack2<kOutBf>(acc[2], acc[3]);
    o4.z = pack2<kOutBf>(acc[4], acc[5]);
    o4.w = pack2<kOutBf>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dst) = o4;
  };
  if (units <= 32) {
    // few units: several lanes share a unit and split its partials
    int u2 = 1;
    while (u2 < units) u2 <<= 1;
    const int lpu = 32 / u2;  // lanes per unit
    const int unit = lane & (u2 - 1);
    const int sub = lane / u2;
    const bool ok = unit < units;
    const int uu = ok ? unit : 0;
    const int hl = uu / UPH;
    const int e0 = (uu % UPH) * 8;
    const float* wt = exp_sums + row0 + int64_t(hl) * P;
    const QT* src = tmp + (row0 + int64_t(hl) * P) * D + e0;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 8
    for (int j = sub; j < np; j += lpu) {
      const float w = __ldcg(wt + int64_t(j) * pstride);
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + int64_t(j) * jstep));
      fma8(acc, w, v);
    }
    for (int o = u2; o < 32; o <<= 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
    __syncwarp();  // (group) partial 0 is a source of other lanes and the destination
    if (ok && sub == 0) store8(outp + hl * out_head_stride + e0, acc);
  } else {
    // many units: a lane works on two of them at once
    for (int u0 = lane; u0 < units; u0 += 64) {
      const float* wt[2];
      const QT* src[2];
      float acc[2][8];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int u = u0 + 32 * k < units ? u0 + 32 * k : u0;
        const int hl = u / UPH;
        const int e0 = (u % UPH) * 8;
        wt[k] = exp_sums + row0 + int64_t(hl) * P;
        src[k] = tmp + (row0 + int64_t(hl) * P) * D + e0;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[k][i] = 0.f;
      }
#pragma unroll 8
      for (int j = 0; j < np; ++j) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float w = __ldcg(wt[k] + int64_t(j) * pstride);
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src[k] + int64_t(j) * jstep));
          fma8(acc[k], w, v);
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int u = u0 + 32 * k;
        if (u < units) store8(outp + (u / UPH) * out_head_stride + (u % UPH) * 8, acc[k]);
      }
    }
  }
  if (group) {
    // the merged partial's exp sum moves to its place (the weights have been used)
    __syncwarp();
    if (lane < nheads) {
      const int64_t at = row0 + int64_t(lane) * P;
      exp_sums[at] = max_logits[at + 1];
    }
  }
}

// Up to 32 partials of up to 4 heads (64 output units) in ONE memory round trip: the statistics
// and the first partials are requested together, the weights stay in registers (lane j holds
// those of partial j) and reach the lanes that accumulate by shuffle instead of through memory.
// A lane owns two 16-byte output units; JB = partials requested per round trip.
template <typename QT, int D, int JB>
__device__ __noinline__ void merge_partials_fast(float* exp_sums, float* max_logits, const QT* tmp,
                                                    QT* outp, int64_t out_head_stride, int64_t row0,
                                                    int np, int P, int pstride, int nh, int lane,
                                                    float* lse, int lse_stride, bool group) {
  constexpr bool kOutBf = std::is_same_v<QT, __nv_bfloat16>;
  constexpr int NU = 2;
  constexpr int UPH = D / 8;  // units per head
  const int units = nh * UPH;
  const int64_t jstep = int64_t(pstride) * D;
  // ---- requests: statistics of partial `lane` for the nh heads ...
  float ml0[4], es0[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const bool ok = k < nh && lane < np;
    const int64_t at = row0 + int64_t(ok ? k : 0) * P + int64_t(ok ? lane : 0) * pstride;
    ml0[k] = ok ? __ldcg(max_logits + at) : -INFINITY;
    es0[k] = ok ? __ldcg(exp_sums + at) : 0.f;
  }
  // ... and the first JB partials of this lane's units
  int hl[NU];
  bool uok[NU];
  const QT* src[NU];
  QT* dst[NU];
#pragma unroll
  for (int k2 = 0; k2 < NU; ++k2) {
    const int u = lane + 32 * k2;
    uok[k2] = u < units;
    const int uu = uok[k2] ? u : 0;
    hl[k2] = uu / UPH;
    const int e0 = (uu % UPH) * 8;
    src[k2] = tmp + (row0 + int64_t(hl[k2]) * P) * D + e0;
    dst[k2] = outp + hl[k2] * out_head_stride + e0;
  }
  uint4 v[NU][JB];
  auto request = [&](int jb) {
#pragma unroll
    for (int jj = 0; jj < JB; ++jj)
#pragma unroll
      for (int k2 = 0; k2 < NU; ++k2)
        if (jb + jj < np && uok[k2])
          v[k2][jj] = __ldcg(reinterpret_cast<const uint4*>(src[k2] + int64_t(jb + jj) * jstep));
  };
  request(0);
  // ---- weights (registers): lane j holds w_j / sum of each head
  float wn[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float mx = ml0[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float w = (k < nh && lane < np) ? es0[k] * fast_exp2(ml0[k] - mx) : 0.f;
    float sum = w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    wn[k] = w * __fdividef(1.f, group ? sum : sum + 1e-6f);
    if (k < nh && lane == 0) {
      if (group) {
        // every lane has its statistics in registers: partial 0's slots take the merged ones
        max_logits[row0 + int64_t(k) * P] = mx;
        exp_sums[row0 + int64_t(k) * P] = sum;
      } else if (lse != nullptr) {
        lse[int64_t(k) * lse_stride] = (mx + log2f(sum)) * kLn2;
      }
    }
  }
  // ---- weighted sum
  float acc[NU][8];
#pragma unroll
  for (int k2 = 0; k2 < NU; ++k2)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[k2][i] = 0.f;
  for (int jb = 0; jb < np; jb += JB) {
    if (jb > 0) request(jb);
#pragma unroll
    for (int jj = 0; jj < JB; ++jj) {
      const int j = jb + jj;
      if (j >= np) break;  // warp-uniform
      const float s0 = __shfl_sync(0xffffffffu, wn[0], j);
      const float s1 = __shfl_sync(0xffffffffu, wn[1], j);
      const float s2 = __shfl_sync(0xffffffffu, wn[2], j);
      const float s3 = __shfl_sync(0xffffffffu, wn[3], j);
#pragma unroll
      for (int k2 = 0; k2 < NU; ++k2) {
        if (!uok[k2]) continue;
        const float w = hl[k2] == 0 ? s0 : (hl[k2] == 1 ? s1 : (hl[k2] == 2 ? s2 : s3));
        const uint32_t vv[4] = {v[k2][jj].x, v[k2][jj].y, v[k2][jj].z, v[k2][jj].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f0, f1;
          if constexpr (kOutBf) {
            f0 = __uint_as_float(vv[i] << 16);
            f1 = __uint_as_float(vv[i] & 0xffff0000u);
          } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&vv[i]);
            f0 = __low2float(h);
            f1 = __high2float(h);
          }
          acc[k2][2 * i] += w * f0;
          acc[k2][2 * i + 1] += w * f1;
        }
      }
    }
  }
#pragma unroll
  for (int k2 = 0; k2 < NU; ++k2) {
    if (!uok[k2]) continue;
    uint4 o4;
    o4.x = pack2<kOutBf>(acc[k2][0], acc[k2][1]);
    o4.y = pack2<kOutBf>(acc[k2][2], acc[k2][3]);
    o4.z = pack2<kOutBf>(acc[k2][4], acc[k2][5]);
    o4.w = pack2<kOutBf>(acc[k2][6], acc[k2][7]);
    *reinterpret_cast<uint4*>(dst[k2]) = o4;
  }
}

// The same idea for at most 32 output units (one or two heads of 128): several lanes share a
// unit and split its partials between them, their sums are added by shuffles.
template <typename QT, int D, int JB>
__device__ __noinline__ void merge_partials_fast_few(float* exp_sums, float* max_logits, const QT* tmp,
                                                     QT* outp, int64_t out_head_stride, int64_t row0, int np,
                                                     int P, int pstride, int nh, int lane, float* lse,
                                                     int lse_stride, bool group) {
  constexpr bool kOutBf = std::is_same_v<QT, __nv_bfloat16>;
  constexpr int UPH = D / 8;  // units per head
  const int units = nh * UPH;
  const int64_t jstep = int64_t(pstride) * D;
  float ml0[4], es0[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const bool ok = k < nh && lane < np;
    const int64_t at = row0 + int64_t(ok ? k : 0) * P + int64_t(ok ? lane : 0) * pstride;
    ml0[k] = ok ? __ldcg(max_logits + at) : -INFINITY;
    es0[k] = ok ? __ldcg(exp_sums + at) : 0.f;
  }
  int u2 = 1;
  while (u2 < units) u2 <<= 1;
  const int lpu = 32 / u2;  // lanes per unit
  const int unit = lane & (u2 - 1);
  const int sub = lane / u2;
  const bool uok = unit < units;
  const int uu = uok ? unit : 0;
  const int hl = uu / UPH;
  const int e0 = (uu % UPH) * 8;
  const QT* src = tmp + (row0 + int64_t(hl) * P) * D + e0;
  uint4 v[JB];
  auto request = [&](int jb) {
#pragma unroll
    for (int jj = 0; jj < JB; ++jj) {
      const int j = jb + jj * lpu + sub;
      if (j < np && uok) v[jj] = __ldcg(reinterpret_cast<const uint4*>(src + int64_t(j) * jstep));
    }
  };
  request(0);
  float wn[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float mx = ml0[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float w = (k < nh && lane < np) ? es0[k] * fast_exp2(ml0[k] - mx) : 0.f;
    float sum = w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    wn[k] = w * __fdividef(1.f, group ? sum : sum + 1e-6f);
    if (k < nh && lane == 0) {
      if (group) {
        max_logits[row0 + int64_t(k) * P] = mx;
        exp_sums[row0 + int64_t(k) * P] = sum;
      } else if (lse != nullptr) {
        lse[int64_t(k) * lse_stride] = (mx + log2f(sum)) * kLn2;
      }
    }
  }
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int jb = 0; jb < np; jb += JB * lpu) {
    if (jb > 0) request(jb);
#pragma unroll
    for (int jj = 0; jj < JB; ++jj) {
      if (jb + jj * lpu >= np) break;  // warp-uniform: no lane has a partial at this step
      const int j = jb + jj * lpu + sub;
      const int jc = j < np ? j : 0;
      const float s0 = __shfl_sync(0xffffffffu, wn[0], jc);
      const float s1 = __shfl_sync(0xffffffffu, wn[1], jc);
      const float s2 = __shfl_sync(0xffffffffu, wn[2], jc);
      const float s3 = __shfl_sync(0xffffffffu, wn[3], jc);
      if (j < np && uok) {
        const float w = hl == 0 ? s0 : (hl == 1 ? s1 : (hl == 2 ? s2 : s3));
        const uint32_t vv[4] = {v[jj].x, v[jj].y, v[jj].z, v[jj].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f0, f1;
          if constexpr (kOutBf) {
            f0 = __uint_as_float(vv[i] << 16);
            f1 = __uint_as_float(vv[i] & 0xffff0000u);
          } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&vv[i]);
            f0 = __low2float(h);
            f1 = __high2float(h);
          }
          acc[2 * i] += w * f0;
          acc[2 * i + 1] += w * f1;
        }
      }
    }
  }
  for (int o = u2; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  __syncwarp();  // (group) partial 0 is a source of other lanes' loads and the destination
  if (uok && sub == 0) {
    uint4 o4;
    o4.x = pack2<kOutBf>(acc[0], acc[1]);
    o4.y = pack2<kOutBf>(acc[2], acc[3]);
    o4.z = pack2<kOutBf>(acc[4], acc[5]);
    o4.w = pack2<kOutBf>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(outp + hl * out_head_stride + e0) = o4;
  }
}

// The merge of one (sequence, kv head, head group).  Both forms are out of line, each with its
// own register frame, and called after the page loop only (a call from inside it made the
// compiler spill the loop's state around the call).
template <typename QT, int D>
__device__ __forceinline__ void merge_partials(float* exp_sums, float* max_logits, const QT* tmp,
                                            QT* outp, int64_t out_head_stride, int64_t row0, int np,
                                            int P, int pstride, int nheads, int lane, float* lse,
                                            int lse_stride, bool group) {
  constexpr int UPH = D / 8;
  constexpr int HB = UPH <= 16 ? 4 : 2;  // heads per pass: at most 64 output units
  // Up to 32 partials: the forms that request statistics and partials together (measured on
  // B200 against the general form: MHA decode of 8 sequences 27.5 -> 25.2 us, an 8-way kv-head
  // shard of a long-context batch 65 -> 60.5 us).  Four partials per request and lane: with eight
  // the functions need so many registers that the compiler spills in the kernel around the
  // calls, which costs more than the round trip saves.
  if (np > 32) {
    merge_partials_general<QT, D>(exp_sums, max_logits, tmp, outp, out_head_stride, row0, np, P, pstride,
                                  nheads, lane, lse, lse_stride, group);
    return;
  }
  if (nheads * UPH <= 32) {
    for (int h0 = 0; h0 < nheads; h0 += 4) {  // (the forms carry the weights of four heads)
      float* lse_h = lse ? lse + int64_t(h0) * lse_stride : nullptr;
      merge_partials_fast_few<QT, D, 4>(exp_sums, max_logits, tmp, outp + h0 * out_head_stride, out_head_stride,
                                        row0 + int64_t(h0) * P, np, P, pstride, min(4, nheads - h0), lane, lse_h,
                                        lse_stride, group);
    }
    return;
  }
  for (int h0 = 0; h0 < nheads; h0 += HB) {
    const int nh = min(HB, nheads - h0);
    float* lse_h = lse ? lse + int64_t(h0) * lse_stride : nullptr;
    merge_partials_fast<QT, D, 4>(exp_sums, max_logits, tmp, outp + h0 * out_head_stride, out_head_stride,
                                  row0 + int64_t(h0) * P, np, P, pstride, nh, lane, lse_h, lse_stride, group);
  }
}

template <typename QT, int KV, int D, int GP, int BT, int MAXW>
__global__ void __launch_bounds__(MAXW * 32, 1) pa_decode_kernel(const DecodeParams p) {
  using TR = DecodeTraits<QT, KV, D, GP>;
  constexpr bool kFp8 = TR::kFp8;
  constexpr bool kBf = TR::kMmaBf16;
  constexpr int ES = TR::kEsize;
  constexpr int KS = TR::kKSteps;
  constexpr bool kE5 = KV == kCacheE5M2;
  constexpr bool kOutBf = std::is_same_v<QT, __nv_bfloat16>;
  extern __shared__ __align__(128) unsigned char smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2;  // fragment row group
  const int c = lane & 3;   // fragment column pair
  constexpr int B = 16 * BT;  // tokens per cache block (16 or 32)
  // One pipeline step covers PP consecutive blocks of the sequence: two when blocks are very
  // small, so that barrier traffic, softmax bookkeeping and producer run once per 32 tokens.
  constexpr int PP = decode_pages_per_step(KV != kCache16 ? 1 : 2, D, BT);
  constexpr int NT = BT * PP;  // 16-token tiles per step
  constexpr int ST = 16 * NT;  // tokens per step
  constexpr uint32_t page_bytes = uint32_t(D) * B * (KV != kCache16 ? 1 : 2);
  constexpr uint32_t step_bytes = PP * page_bytes;  // K (or V) bytes of one step
  const int slots_per_warp = p.nstages;  // ring slots the launch provides per warp
  // Steps of 4 KiB and more get one slot and one barrier each for K and V (finer prefetch
  // granularity: the K slot is refilled while the softmax runs); smaller ones share one slot
  // and one barrier (half the barrier traffic).  The host uses the same rule.
  constexpr bool split_kv = step_bytes >= 4096;
  constexpr uint32_t slot_bytes = split_kv ? step_bytes : 2 * step_bytes;
  // ---- shared memory carve-up: [unit prefix table][mbarriers][stages]
  int* cum = reinterpret_cast<int*>(smem_raw);
  const int table_ints = p.use_table ? ((p.num_seqs + 1 + 3) & ~3) : 0;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + size_t(table_ints) * 4);
  const uint32_t bars_bytes = (uint32_t(nwarps) * slots_per_warp * 8 + 127u) & ~127u;
  unsigned char* slots = smem_raw + size_t(table_ints) * 4 + bars_bytes;
  // the dynamic buffer is 128-byte aligned and table_ints*4 is a multiple of 16

  // ---- set-up of a split launch: the flat list of work units.
  // A unit is one cache block of one (kv head, head group, sequence); a sequence counts
  // max(2, blocks rounded up to even) units, so that every sequence start - and with an even
  // range length every cut - falls on an even block and an empty sequence still has a unit
  // that gets its (zero) output written.  The list is ordered (head, sequence, block); warp r
  // of the grid takes units [r*C, (r+1)*C).
  __shared__ int s_plan[4];      // [0] C: units per range, [1] units of one head, [2] ranges
  __shared__ int4 s_iter[MAXW];  // per warp: units left, block offset, sequence, head
  __shared__ int4 s_todo[MAXW][2];  // per warp: merges owed (sequence, head item, pieces, piece | level)
  __shared__ int s_ntodo[MAXW];
  const bool flat = p.use_table != 0;
  const int hsubs = p.num_kv_heads * p.head_groups;
  if (flat) {
    __shared__ int warp_tot[MAXW];
    __shared__ int warp_mx[MAXW];
    const int S = p.num_seqs;
    const int per = (S + blockDim.x - 1) / blockDim.x;
    const int s0 = min(S, int(threadIdx.x) * per);
    const int s1 = min(S, s0 + per);
    auto units_of = [&](int s) {
      const int len = min(max(p.seq_lens[s], 0), p.len_cap);
      return max(2, ((len + B - 1) / B + 1) & ~1);
    };
    int mine = 0, mx = 0;
    for (int s = s0; s < s1; ++s) {
      const int n = units_of(s);
      mine += n;
      mx = max(mx, n);
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 31) {
      warp_tot[warp] = incl;
      warp_mx[warp] = mx;
    }
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    int run = base + incl - mine;
    for (int s = s0; s < s1; ++s) {
      cum[s] = run;
      run += units_of(s);
    }
    if (threadIdx.x == blockDim.x - 1) cum[S] = run;
    if (threadIdx.x == 0) {
      int total = 0, n_max = 2;
      for (int w = 0; w < nwarps; ++w) {
        total += warp_tot[w];
        n_max = max(n_max, warp_mx[w]);
      }
      // Range length: an equal share for every warp of the grid, at least the smallest range
      // worth a work item, and large enough that the longest sequence is cut into no more
      // pieces than the scratch has slots per sequence (a sequence of n units meets at most
      // (n - 1) / C + 2 ranges).  Even, see above.
      const long long U = (long long)hsubs * total;
      const long long W = (long long)gridDim.x * nwarps;
      long long C = (U + W - 1) / W;
      C = max(C, (long long)p.min_chunk);
      C = max(C, (long long)((n_max - 1) / max(1, p.max_partitions - 1) + 1));
      C = (C + 1) & ~1ll;
      s_plan[0] = int(min(C, (long long)INT32_MAX - 1));
      s_plan[1] = total;
      s_plan[2] = int((U + C - 1) / C);
    }
  }
  __syncthreads();

  const unsigned grid_warps = gridDim.x * unsigned(nwarps);
  // work items of an unsplit launch / ranges of a split one
  const unsigned total_items = flat ? unsigned(s_plan[2]) : unsigned(p.num_seqs) * unsigned(hsubs);
  // Ranges and the first items are numbered SM-first: warp w of CTA b has number
  // w * gridDim.x + b, so a launch with fewer of them than warps leaves the
  // highest-numbered warps of every CTA idle.
  const unsigned my_number = unsigned(warp) * gridDim.x + blockIdx.x;

  // Ring of this warp.  The host sizes warps and slots without knowing the lengths; when the
  // batch turns out to have fewer ranges / items than the grid has warps, the warps without
  // one leave their slots and barriers to the others: fewer busy warps, each with more pages
  // in flight, which is what a launch bound by the latency of one item needs.
  int NSLOT = slots_per_warp;
  if (total_items < grid_warps) {
    const int busy = max(1, int((total_items + gridDim.x - 1) / gridDim.x));  // per CTA, at most
    NSLOT = min(8, nwarps * slots_per_warp / busy);
  }
  const uint32_t my_slot0 = smem_u32(slots) + uint32_t(warp) * NSLOT * slot_bytes;
  const uint32_t my_bar0 = smem_u32(bars) + uint32_t(warp) * NSLOT * 8;
  unsigned char* my_slots = slots + size_t(warp) * NSLOT * slot_bytes;
  const bool has_ring = (warp + 1) * NSLOT <= nwarps * slots_per_warp;
  if (lane == 0 && has_ring) {
    // the barriers are private to the warp: no CTA-wide synchronisation after their set-up
    for (int s = 0; s < NSLOT; ++s) mbar_init(my_bar0 + s * 8, 1);
    fence_barrier_init();
  }
  // where range r starts: head, sequence (binary search), block offset
  auto start_range = [&](unsigned r) -> int4 {
    int4 st = make_int4(0, 0, 0, 0);
    if (r < total_items) {
      const int C = s_plan[0], TP = s_plan[1];
      const long long U = (long long)hsubs * TP;
      const long long u0 = (long long)r * C;
      st.x = int(min((long long)C, U - u0));
      // (64-bit divisions cost a few hundred cycles each; lists below 2^31 units use 32-bit ones)
      st.w = U <= INT32_MAX ? int(unsigned(u0) / unsigned(TP)) : int(u0 / TP);
      const int rem = int(u0 - (long long)st.w * TP);
      int lo = 0, hi = p.num_seqs;  // cum[lo] <= rem < cum[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cum[mid] <= rem) lo = mid; else hi = mid;
      }
      st.z = lo;
      st.y = rem - cum[lo];
    }
    return st;
  };
  if (flat) {
    const int4 st = start_range(my_number);
    if (lane == 0) s_iter[warp] = st;
  }
  if (lane == 0) s_ntodo[warp] = 0;
  __syncwarp();
  const uint64_t policy = policy_evict_first();
  const char* kc_base = static_cast<const char*>(p.kc);
  const char* vc_base = static_cast<const char*>(p.vc);

  // Unsplit launches: up to three items per resident warp are dealt out by a fixed stride
  // (warp number, + W, + 2W; W = warps in the grid): no ticket round trips, and nobody holds a
  // second item while another warp idles.  Larger launches pull tickets from the global
  // counter, which balances items of unequal length.
  const bool strided = !flat && total_items <= 3u * grid_warps;
  unsigned next_strided = my_number;

  auto fetch = [&]() -> unsigned {
    if (strided) {
      const unsigned v = next_strided;
      next_strided += grid_warps;
      return v;
    }
    unsigned v = 0;
    if (lane == 0) v = atomicAdd(p.sched, 1u);
    return __shfl_sync(0xffffffffu, v, 0);
  };

  auto blank_item = [&]() -> WorkItem {
    WorkItem it;
    it.valid = false;
    it.seq = it.kvh = it.hg = it.part = it.tok_begin = it.tok_end = it.first_page = it.npages = 0;
    it.nparts = 1;
    it.win = 0;
    it.bt = 0;
    return it;
  };

  // unsplit: item number -> (sequence, head), the whole sequence
  auto decode = [&](unsigned raw) -> WorkItem {
    WorkItem it = blank_item();
    it.valid = raw < total_items;
    if (!it.valid) return it;
    const int hsub = int(raw % unsigned(hsubs));
    it.seq = int(raw / unsigned(hsubs));
    it.kvh = hsub / p.head_groups;
    it.hg = hsub % p.head_groups;
    it.tok_end = max(p.seq_lens[it.seq], 0);
    it.npages = (it.tok_end + B - 1) / B;
    it.bt = load_bt(p, it, 0, lane);
    return it;
  };

  // split: the next piece of this warp's range.  The iterator lives in shared memory so that
  // the page loop carries no registers for it.
  auto next_piece = [&]() -> WorkItem {
    WorkItem it = blank_item();
    int4 st = s_iter[warp];
    it.valid = st.x > 0;
    if (!it.valid) return it;
    const int C = s_plan[0], TP = s_plan[1];
    const int c0 = cum[st.z];
    const int n = cum[st.z + 1] - c0;      // units of this sequence
    const int take = min(n - st.y, st.x);  // units of it that fall into the range
    const int len = min(max(p.seq_lens[st.z], 0), p.len_cap);
    it.seq = st.z;
    it.kvh = st.w / p.head_groups;
    it.hg = st.w % p.head_groups;
    // the ranges that meet this (head, sequence) are consecutive; each delivers one partial
    const long long base = (long long)st.w * TP + c0;
    if (base + n <= INT32_MAX) {  // (32-bit divisions: see start_range)
      const unsigned b32 = unsigned(base), c32 = unsigned(C);
      const int w_lo = int(b32 / c32);
      it.nparts = int((b32 + unsigned(n) - 1u) / c32) - w_lo + 1;
      it.part = int((b32 + unsigned(st.y)) / c32) - w_lo;
    } else {
      const int w_lo = int(base / C);
      it.nparts = int((base + n - 1) / C) - w_lo + 1;
      it.part = int((base + st.y) / C) - w_lo;
    }
    it.first_page = st.y;
    it.tok_begin = st.y * B;
    it.tok_end = max(it.tok_begin, min(len, (st.y + take) * B));
    it.npages = (it.tok_end - it.tok_begin + B - 1) / B;
    it.bt = load_bt(p, it, 0, lane);
    st.x -= take;
    st.y += take;
    if (st.y == n) {
      st.y = 0;
      if (++st.z == p.num_seqs) {
        st.z = 0;
        ++st.w;
      }
    }
    __syncwarp();
    if (lane == 0) s_iter[warp] = st;
    __syncwarp();
    return it;
  };

  // A warp always knows its current item and the next one (decoded, block ids loaded); an
  // unsplit launch also the number of the one after.  With tickets, the second and third are
  // requested as soon as the first has arrived and their round trips overlap with the
  // decoding of the first.
  WorkItem cur, nxt;
  unsigned nn_raw = 0;
  if (flat) {
    cur = next_piece();
    nxt = next_piece();
  } else {
    const unsigned raw0 = fetch();
    unsigned raw1 = 0, raw2 = 0;
    if (strided) {
      raw1 = fetch();
      raw2 = fetch();
    } else if (lane == 0) {
      raw1 = atomicAdd(p.sched, 1u);
      raw2 = atomicAdd(p.sched, 1u);
    }
    cur = decode(raw0);
    if (!strided) {
      raw1 = __shfl_sync(0xffffffffu, raw1, 0);
      raw2 = __shfl_sync(0xffffffffu, raw2, 0);
    }
    nxt = decode(raw1);
    nn_raw = raw2;
  }
  if (!has_ring && cur.valid) {
    // cannot happen with the numbering above; never touch slots that are not this warp's
    if (lane == 0) atomicExch(p.status, kStatusNoRing);
    cur.valid = false;
  }

  // ---- producer state.  The ring is filled in the order K(page 0), V(page 0), K(page 1), ...
  int prod_sel = 0;   // 0: producing pages of `cur`, 1: of `nxt`
  int prod_pg = 0;
  int prod_half = 0;  // 0: the K page is next, 1: the V page of the same block
  int prod_blk[PP] = {};  // block ids of the step being requested
  int prod_n = 0;         // blocks in that step (the last step of an item may be short)
  int prod_slot = 0;
  int inflight = 0;
  int cons_slot = 0;
  uint32_t cons_phase = 0;
  // the producer's own copy of the item it is loading (no cur/nxt selects in the hot path)
  int pi_npages = cur.npages, pi_bt = cur.bt, pi_win = 0;
  int64_t pi_kvoff = int64_t(cur.kvh) * p.kv_head_stride * ES;
  const int64_t blk_stride_bytes = p.kv_block_stride * ES;

  auto producer_take = [&](const WorkItem& it) {
    pi_npages = it.npages;
    pi_bt = it.bt;
    pi_win = 0;
    pi_kvoff = int64_t(it.kvh) * p.kv_head_stride * ES;
    prod_pg = 0;
  };

  auto produce_one = [&]() -> bool {
    if (!split_kv || prod_half == 0) {
      if (prod_pg >= pi_npages) {
        // the item is fully requested: move on to the next one, if it is known
        if (prod_sel == 1 || !nxt.valid) return false;
        prod_sel = 1;
        producer_take(nxt);
        if (pi_npages == 0) return false;
      }
      const int win = prod_pg >> 5;
      if (win != pi_win) {
        pi_win = win;
        pi_bt = load_bt(p, prod_sel ? nxt : cur, win, lane);
      }
      // items start on an even page and a window holds 32: both ids are in this window
#pragma unroll
      for (int i = 0; i < PP; ++i) prod_blk[i] = __shfl_sync(0xffffffffu, pi_bt, (prod_pg + i) & 31);
      if constexpr (PP > 1) prod_n = min(PP, pi_npages - prod_pg);
    }
    if (lane == 0) {
      const uint32_t bar = my_bar0 + prod_slot * 8;
      const uint32_t dst = my_slot0 + prod_slot * slot_bytes;
      const int nblk = PP > 1 ? prod_n : 1;  // blocks in this step
      mbar_expect_tx(bar, (split_kv ? 1u : 2u) * uint32_t(nblk) * page_bytes);
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        if (i < nblk) {
          const int64_t off = int64_t(prod_blk[i]) * blk_stride_bytes + pi_kvoff;
          if constexpr (split_kv) {
            bulk_g2s(dst + i * page_bytes, (prod_half ? vc_base : kc_base) + off, page_bytes, bar,
                     policy);
          } else {
            bulk_g2s(dst + i * page_bytes, kc_base + off, page_bytes, bar, policy);
            bulk_g2s(dst + step_bytes + i * page_bytes, vc_base + off, page_bytes, bar, policy);
          }
        }
      }
    }
    prod_slot = (prod_slot + 1 == NSLOT) ? 0 : prod_slot + 1;
    if constexpr (split_kv) {
      prod_pg += PP * prod_half;
      prod_half ^= 1;
    } else {
      prod_pg += PP;
    }
    ++inflight;
    return true;
  };

  while (inflight < NSLOT && produce_one()) {}

  // fold the per-tensor scales of an fp8 cache into the logit scale and the output scale
  const float kv_qk = kFp8 ? *p.k_scale : 1.f;
  const float kv_o = kFp8 ? *p.v_scale : 1.f;
  const float qk_scale = p.scale * kLog2e * kv_qk;
  bool failed = false;
  const bool has_alibi = p.alibi != nullptr;

  while (cur.valid && !failed) {
    const int hq0 = cur.kvh * p.group + cur.hg * TR::kHeadsPerItem;
    const int nheads = min(TR::kHeadsPerItem, p.group - cur.hg * TR::kHeadsPerItem);
    const int seq_len = p.seq_lens[cur.seq];

    // ---- Q fragments (B operand), head = nt*8 + g
    uint32_t qf[GP][KS][2];
#pragma unroll
    for (int nt = 0; nt < GP; ++nt) {
      const int hl = nt * 8 + g;
      const QT* qrow = static_cast<const QT*>(p.q) + int64_t(cur.seq) * p.q_stride +
                       int64_t(hq0 + hl) * D;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t v0 = 0, v1 = 0;
        if (hl < nheads) {
          if constexpr (!kFp8) {
            v0 = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * c);
            v1 = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * c);
          } else {
            // k index 2c+i <-> d 4c+i ; k index 2c+8+i <-> d 4c+2+i ; operands in f16
            const uint2 raw = *reinterpret_cast<const uint2*>(qrow + 16 * ks + 4 * c);
            const QT* e = reinterpret_cast<const QT*>(&raw);
            v0 = pack2<false>(to_f32(e[0]), to_f32(e[1]));
            v1 = pack2<false>(to_f32(e[2]), to_f32(e[3]));
          }
        }
        qf[nt][ks][0] = v0;
        qf[nt][ks][1] = v1;
      }
    }
    float slope[GP][2];
#pragma unroll
    for (int nt = 0; nt < GP; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int hl = nt * 8 + 2 * c + j;
        slope[nt][j] = (has_alibi && hl < nheads) ? p.alibi[hq0 + hl] * kLog2e : 0.f;
      }

    float o[KS][GP][4];
#pragma unroll
    for (int mt = 0; mt < KS; ++mt)
#pragma unroll
      for (int nt = 0; nt < GP; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[mt][nt][i] = 0.f;
    float m_run[GP][2], l_run[GP][2];
#pragma unroll
    for (int nt = 0; nt < GP; ++nt) {
      m_run[nt][0] = m_run[nt][1] = -INFINITY;
      l_run[nt][0] = l_run[nt][1] = 0.f;
    }

    const int nsteps = (cur.npages + PP - 1) / PP;
    for (int st = 0; st < nsteps; ++st) {
      const int page_tok0 = (cur.first_page + st * PP) * B;  // first token of the step
      // tiles of this step that hold at least one valid token (warp-uniform)
      const int ntiles = min(NT, (cur.tok_end - page_tok0 + 15) >> 4);

      // ================= K half: S^T = K . Q^T for every tile of the page
      if (!__all_sync(0xffffffffu, mbar_wait(my_bar0 + cons_slot * 8, cons_phase))) {
        if (lane == 0) atomicExch(p.status, kStatusMbarTimeout);
        failed = true;
        break;
      }
      const uint32_t sk = my_slot0 + cons_slot * slot_bytes;
      float s[NT][GP][4];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        constexpr int kZero = 0;
        float s2[GP][4];  // second accumulation chain: halves the dependent-MMA latency
#pragma unroll
        for (int nt = 0; nt < GP; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) s[t][nt][i] = s2[nt][i] = float(kZero);
        if (NT == 1 || t < ntiles) {
          const int tt = 16 * (t % BT);                        // tile's first token in its block
          const uint32_t skt = sk + (t / BT) * page_bytes;     // that block's K page
          if constexpr (!kFp8) {
            const uint32_t kaddr =
                skt + uint32_t(((lane >> 4) * B + tt + ((lane >> 3) & 1) * 8 + (lane & 7)) * 16);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
              uint32_t a0, a1, a2, a3;
              ldsm_x4(kaddr + uint32_t(2 * ks * B * 16), a0, a1, a2, a3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt) {
                if (ks & 1) mma16816<kBf>(s2[nt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
                else mma16816<kBf>(s[t][nt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
              }
            }
          } else {
            // A row rho of half h <-> token 4*(rho/2) + 2*h + rho%2
            const int rho = lane & 7, hsel = (lane >> 3) & 1;
            const int tok = 4 * (rho >> 1) + 2 * hsel + (rho & 1);
            const uint32_t kaddr = skt + uint32_t(((lane >> 4) * B + tt + tok) * 16);
#pragma unroll
            for (int ks = 0; ks + 1 < KS; ks += 2) {
              uint32_t r0, r1, r2, r3, a0, a1, a2, a3, b0, b1, b2, b3;
              ldsm_x4(kaddr + uint32_t(ks * B * 16), r0, r1, r2, r3);
              fp8x4_to_f16<kE5>(r0, a0, a2);
              fp8x4_to_f16<kE5>(r1, a1, a3);
              fp8x4_to_f16<kE5>(r2, b0, b2);
              fp8x4_to_f16<kE5>(r3, b1, b3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt) {
                mma16816<false>(s[t][nt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
                mma16816<false>(s2[nt], b0, b1, b2, b3, qf[nt][ks + 1][0], qf[nt][ks + 1][1]);
              }
            }
            if constexpr (KS & 1) {
              constexpr int ks = KS - 1;
              uint32_t r0, r1, a0, a1, a2, a3;
              // lanes 0-15 supply the addresses of the two matrices (lanes 16-31 ignored)
              ldsm_x2(skt + uint32_t((ks * B + tt + tok) * 16), r0, r1);
              fp8x4_to_f16<kE5>(r0, a0, a2);
              fp8x4_to_f16<kE5>(r1, a1, a3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt)
                mma16816<false>(s[t][nt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
            }
          }
#pragma unroll
          for (int nt = 0; nt < GP; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[t][nt][i] += s2[nt][i];
        }
      }
      if constexpr (split_kv) {
        // the K slot is free: refill it while the softmax runs
        __syncwarp();
        cons_slot = (cons_slot + 1 == NSLOT) ? 0 : cons_slot + 1;
        if (cons_slot == 0) cons_phase ^= 1;
        --inflight;
        produce_one();
      }

      // ================= scale, ALiBi, mask; online softmax over the whole page
      const bool need_mask = page_tok0 + ST > cur.tok_end;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        int tok_lo, tok_hi;  // absolute token of accumulator rows g and g+8
        if constexpr (!kFp8) {
          tok_lo = page_tok0 + 16 * t + g;
          tok_hi = tok_lo + 8;
        } else {
          tok_lo = page_tok0 + 16 * t + 4 * (g >> 1) + (g & 1);
          tok_hi = tok_lo + 2;
        }
#pragma unroll
        for (int nt = 0; nt < GP; ++nt) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            float v_lo = s[t][nt][j] * qk_scale;
            float v_hi = s[t][nt][2 + j] * qk_scale;
            if (has_alibi) {
              v_lo += slope[nt][j] * float(tok_lo - seq_len + 1);
              v_hi += slope[nt][j] * float(tok_hi - seq_len + 1);
            }
            if (need_mask) {
              if (tok_lo >= cur.tok_end) v_lo = -INFINITY;
              if (tok_hi >= cur.tok_end) v_hi = -INFINITY;
            }
            s[t][nt][j] = v_lo;
            s[t][nt][2 + j] = v_hi;
          }
        }
      }
      float alpha[GP][2];
      bool rescale = false;
#pragma unroll
      for (int nt = 0; nt < GP; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float tmax = fmaxf(s[0][nt][j], s[0][nt][2 + j]);
#pragma unroll
          for (int t = 1; t < NT; ++t) tmax = fmaxf(tmax, fmaxf(s[t][nt][j], s[t][nt][2 + j]));
          tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
          tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
          tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
          const float m_old = m_run[nt][j];
          const float m_new = fmaxf(m_old, tmax);
          // m_new is finite here: every processed page holds at least one valid token
          alpha[nt][j] = fast_exp2(m_old - m_new);
          rescale |= (m_new != m_old);
          m_run[nt][j] = m_new;
          float psum = 0.f;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const float p_lo = fast_exp2(s[t][nt][j] - m_new);
            const float p_hi = fast_exp2(s[t][nt][2 + j] - m_new);
            psum += p_lo + p_hi;
            s[t][nt][j] = p_lo;
            s[t][nt][2 + j] = p_hi;
          }
          l_run[nt][j] = l_run[nt][j] * alpha[nt][j] + psum;
        }
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int mt = 0; mt < KS; ++mt)
#pragma unroll
          for (int nt = 0; nt < GP; ++nt) {
            o[mt][nt][0] *= alpha[nt][0];
            o[mt][nt][1] *= alpha[nt][1];
            o[mt][nt][2] *= alpha[nt][0];
            o[mt][nt][3] *= alpha[nt][1];
          }
      }

      // ================= V half: O^T += V^T . P^T
      if (split_kv && !__all_sync(0xffffffffu, mbar_wait(my_bar0 + cons_slot * 8, cons_phase))) {
        if (lane == 0) atomicExch(p.status, kStatusMbarTimeout);
        failed = true;
        break;
      }
      const uint32_t sv = my_slot0 + cons_slot * slot_bytes + (split_kv ? 0u : step_bytes);
      // zero V columns of tokens past the end of the sequence (stale cache bytes
      // could be NaN/Inf; the reference zeroes them too, attention_kernels.cuh:415-425).
      // Only the block holding the last valid token needs it: tiles beyond are skipped.
      if (need_mask) {
        const int rem = cur.tok_end - page_tok0;  // valid tokens of this step, 1 .. ST-1
        const int pl = (rem - 1) / B;             // block of the step that holds the last one
        const int r = rem - pl * B;               // valid tokens in that block
        unsigned char* vpage = my_slots + size_t(cons_slot) * slot_bytes +
                               (split_kv ? 0u : step_bytes) + pl * page_bytes;
        for (int d = lane; d < D; d += 32) {
          for (int tk = r; tk < B; ++tk) {
            if constexpr (ES == 1) vpage[d * B + tk] = 0;
            else reinterpret_cast<uint16_t*>(vpage)[d * B + tk] = 0;
          }
        }
        __syncwarp();
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (NT == 1 || t < ntiles) {
          const int tt = 16 * (t % BT);
          const uint32_t svt = sv + (t / BT) * page_bytes;
          uint32_t pf[GP][2];  // P^T as B operand
#pragma unroll
          for (int nt = 0; nt < GP; ++nt) {
            pf[nt][0] = movm_trans(pack2<kBf>(s[t][nt][0], s[t][nt][1]));
            pf[nt][1] = movm_trans(pack2<kBf>(s[t][nt][2], s[t][nt][3]));
          }
          if constexpr (!kFp8) {
            const uint32_t vaddr =
                svt + uint32_t(((((lane >> 3) & 1) * 8 + (lane & 7)) * B + tt + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
              uint32_t a0, a1, a2, a3;
              ldsm_x4(vaddr + uint32_t(16 * mt * B * 2), a0, a1, a2, a3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt)
                mma16816<kBf>(o[mt][nt], a0, a1, a2, a3, pf[nt][0], pf[nt][1]);
            }
          } else {
            const uint32_t vaddr =
                svt + uint32_t((16 * (lane >> 4) + ((lane >> 3) & 1) * 8 + (lane & 7)) * B + tt);
#pragma unroll
            for (int mt = 0; mt + 1 < KS; mt += 2) {
              uint32_t r0, r1, r2, r3, a0, a1, a2, a3, b0, b1, b2, b3;
              ldsm_x4(vaddr + uint32_t(16 * mt * B), r0, r1, r2, r3);
              fp8x4_to_f16<kE5>(r0, a0, a2);
              fp8x4_to_f16<kE5>(r1, a1, a3);
              fp8x4_to_f16<kE5>(r2, b0, b2);
              fp8x4_to_f16<kE5>(r3, b1, b3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt) {
                mma16816<false>(o[mt][nt], a0, a1, a2, a3, pf[nt][0], pf[nt][1]);
                mma16816<false>(o[mt + 1][nt], b0, b1, b2, b3, pf[nt][0], pf[nt][1]);
              }
            }
            if constexpr (KS & 1) {
              constexpr int mt = KS - 1;
              uint32_t r0, r1, a0, a1, a2, a3;
              ldsm_x2(svt + uint32_t((16 * mt + ((lane >> 3) & 1) * 8 + (lane & 7)) * B + tt), r0, r1);
              fp8x4_to_f16<kE5>(r0, a0, a2);
              fp8x4_to_f16<kE5>(r1, a1, a3);
#pragma unroll
              for (int nt = 0; nt < GP; ++nt)
                mma16816<false>(o[mt][nt], a0, a1, a2, a3, pf[nt][0], pf[nt][1]);
            }
          }
        }
      }
      // ---- release the V slot and refill it
      __syncwarp();
      if (need_mask) fence_proxy_async();  // generic writes above vs. the next bulk copy
      cons_slot = (cons_slot + 1 == NSLOT) ? 0 : cons_slot + 1;
      if (cons_slot == 0) cons_phase ^= 1;
      --inflight;
      produce_one();
    }  // pages
    if (failed) break;

    // ---- finalise the item: l over the 8 row groups, normalise, write
    const bool direct = cur.nparts == 1;
    QT* obase;
    int64_t ohead_stride;
    if (direct) {
      obase = static_cast<QT*>(p.out) + (int64_t(cur.seq) * p.num_heads + hq0) * D;
      ohead_stride = D;
    } else {
      obase = static_cast<QT*>(p.tmp_out) +
              ((int64_t(cur.seq) * p.num_heads + hq0) * p.max_partitions + cur.part) * D;
      ohead_stride = int64_t(p.max_partitions) * D;
    }
#pragma unroll
    for (int nt = 0; nt < GP; ++nt) {
      float inv[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float l = l_run[nt][j];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        inv[j] = kv_o * __fdividef(1.f, l + 1e-6f);
        const int hl = nt * 8 + 2 * c + j;
        if (!direct && g == 0 && hl < nheads) {
          const int64_t idx =
              (int64_t(cur.seq) * p.num_heads + hq0 + hl) * p.max_partitions + cur.part;
          p.max_logits[idx] = m_run[nt][j];
          p.exp_sums[idx] = l;
        }
        if (direct && p.lse != nullptr && g == 0 && hl < nheads)
          p.lse[int64_t(hq0 + hl) * p.num_seqs + cur.seq] =
              l > 0.f ? (m_run[nt][j] + log2f(l)) * kLn2 : -INFINITY;
      }
      const int hl_t = nt * 8 + g;  // head owned after the transpose
#pragma unroll
      for (int mt = 0; mt < KS; ++mt) {
        // transposes are warp-collective: executed by all lanes, stores predicated
        const uint32_t lo = movm_trans(pack2<kOutBf>(o[mt][nt][0] * inv[0],
                                                                      o[mt][nt][1] * inv[1]));
        const uint32_t hi = movm_trans(pack2<kOutBf>(o[mt][nt][2] * inv[0],
                                                                      o[mt][nt][3] * inv[1]));
        if (hl_t < nheads) {
          QT* orow = obase + hl_t * ohead_stride + 16 * mt + 2 * c;
          *reinterpret_cast<uint32_t*>(orow) = lo;
          *reinterpret_cast<uint32_t*>(orow + 8) = hi;
        }
      }
    }

    // ---- split sequences: the warp that delivers the LAST partial of a (sequence, kv head,
    // head group) merges all of them into `out` (replaces the reference's separate
    // paged_attention_v2_reduce_kernel launch, attention_kernels.cuh:559-664).  Nobody waits:
    // earlier arrivers just leave.  The arrival is counted here; the merge itself is noted down
    // and done after the page loop (below), where it costs the loop no registers.  A range has
    // at most two pieces of sequences that continue in other ranges (its first and its last),
    // so two notes per warp are enough.
    if (!direct && p.arrive != nullptr) {
      __threadfence();  // partials visible before the arrival is counted
      __syncwarp();
      const size_t unit = (size_t(cur.seq) * p.num_kv_heads + cur.kvh) * p.head_groups + cur.hg;
      int level = -1;  // 1: this warp completed its group, 0: it completed the sequence
      if (p.arrive2 != nullptr && cur.nparts > kMergeDirectMax &&
          min(kMergeFan, cur.nparts - (cur.part / kMergeFan) * kMergeFan) > 1) {
        const int gidx = cur.part / kMergeFan;
        const int gsize = min(kMergeFan, cur.nparts - gidx * kMergeFan);
        unsigned* cnt2 = p.arrive2 + unit * p.groups_max + gidx;
        unsigned old2 = 0;
        if (lane == 0) old2 = atomicAdd(cnt2, 1u);
        old2 = __shfl_sync(0xffffffffu, old2, 0);
        if (old2 == unsigned(gsize - 1)) {
          if (lane == 0) *cnt2 = 0;  // re-arm for the next launch
          level = 1;
        }
      } else {
        const int np_top = (p.arrive2 != nullptr && cur.nparts > kMergeDirectMax)
                               ? (cur.nparts + kMergeFan - 1) / kMergeFan
                               : cur.nparts;
        unsigned* cnt = p.arrive + unit;
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(cnt, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == unsigned(np_top - 1)) {
          if (lane == 0) *cnt = 0;  // re-arm for the next launch
          level = 0;
        }
      }
      if (level >= 0) {
        const int n = s_ntodo[warp];
        if (n < 2) {
          if (lane == 0) {
            s_todo[warp][n] = make_int4(cur.seq, cur.kvh * p.head_groups + cur.hg, cur.nparts,
                                        cur.part | (level << 30));
            s_ntodo[warp] = n + 1;
          }
          __syncwarp();
        } else {
          // cannot happen (see above); never drop a merge silently
          if (lane == 0) atomicExch(p.status, kStatusMergeNotes);
        }
      }
    }

    // ---- advance to the next item
    cur = nxt;
    if (flat) {
      nxt = next_piece();
    } else {
      nxt = decode(nn_raw);
      nn_raw = fetch();
    }
    // the producer either already works on the new `cur` (keep its state) or starts it now
    if (prod_sel == 1) prod_sel = 0; else producer_take(cur);
    while (inflight < NSLOT && produce_one()) {}
  }

  // ---- the merges this warp owes (noted above)
  if (!failed) {
    const int ntodo = s_ntodo[warp];
    for (int k = 0; k < ntodo; ++k) {
      const int4 td = s_todo[warp][k];
      const int seq = td.x, kvh = td.y / p.head_groups, hg = td.y % p.head_groups, nparts = td.z;
      const int part = td.w & 0x3fffffff;
      const bool group_first = (td.w >> 30) != 0;
      const int hq0 = kvh * p.group + hg * TR::kHeadsPerItem;
      const int nheads = min(TR::kHeadsPerItem, p.group - hg * TR::kHeadsPerItem);
      const size_t unit = (size_t(seq) * p.num_kv_heads + kvh) * p.head_groups + hg;
      const int64_t rowbase = (int64_t(seq) * p.num_heads + hq0) * p.max_partitions;
      QT* tmp_q = static_cast<QT*>(p.tmp_out);
      const bool two_level = p.arrive2 != nullptr && nparts > kMergeDirectMax;
      const int np_top = two_level ? (nparts + kMergeFan - 1) / kMergeFan : nparts;
      const int stride_top = two_level ? kMergeFan : 1;
      bool go_top = true;
      if (group_first) {
        // two levels: this piece's group first, then the group arrives for the sequence
        const int gidx = part / kMergeFan;
        const int gsize = min(kMergeFan, nparts - gidx * kMergeFan);
        __threadfence();  // order the loads below after the observed arrivals
        const int64_t g0 = rowbase + gidx * kMergeFan;
        merge_partials<QT, D>(p.exp_sums, p.max_logits, tmp_q, tmp_q + g0 * D,
                              int64_t(p.max_partitions) * D, g0, gsize, p.max_partitions, 1, nheads,
                              lane, nullptr, 0, true);
        __threadfence();
        __syncwarp();
        unsigned* cnt = p.arrive + unit;
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(cnt, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        go_top = old == unsigned(np_top - 1);
        if (go_top && lane == 0) *cnt = 0;  // re-arm for the next launch
      }
      if (go_top) {
        __threadfence();  // order the loads below after the observed arrivals
        merge_partials<QT, D>(p.exp_sums, p.max_logits, tmp_q,
                              static_cast<QT*>(p.out) + (int64_t(seq) * p.num_heads + hq0) * D, D, rowbase,
                              np_top, p.max_partitions, stride_top, nheads, lane,
                              p.lse ? p.lse + int64_t(hq0) * p.num_seqs + seq : nullptr, p.num_seqs, false);
      }
    }
  }

  if (failed) {
    // give copies already in flight a bounded chance to land before the CTA's
    // shared memory is released
    for (int i = 0; i < inflight; ++i) {
      mbar_wait(my_bar0 + cons_slot * 8, cons_phase);
      cons_slot = (cons_slot + 1 == NSLOT) ? 0 : cons_slot + 1;
      if (cons_slot == 0) cons_phase ^= 1;
    }
  }

  // ---- last CTA out re-arms the scheduler words for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(p.sched + 1, 1u);
    if (prev == gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace b200pa
