// Parameter block and small PTX wrappers shared by the decode kernels.
#pragma once

#include "common.cuh"

namespace b200pa {

constexpr int kPartitionTokens = 512;  // split-KV partition, same as the reference's PARTITION_SIZE
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Status codes written to the device status word.
enum : int { kStatusOk = 0, kStatusMbarTimeout = 1, kStatusNoRing = 2, kStatusMergeNotes = 3 };

struct DecodeParams {
  void* out;
  const void* q;
  const void* kc;
  const void* vc;
  const int* block_tables;
  const int* seq_lens;
  const float* alibi;
  const float* k_scale;
  const float* v_scale;
  float* exp_sums;    // [S, Hq, P]  (l per partition)
  float* max_logits;  // [S, Hq, P]  (m per partition, log2 domain)
  void* tmp_out;      // [S, Hq, P, D] query dtype, normalised partials
  unsigned* sched;    // [0] work ticket, [1] CTAs done (self-resetting)
  unsigned* arrive;   // per (seq, kv head, head group) count of delivered partials, or nullptr
  unsigned* arrive2;  // [that][groups_max]: counts per group of pieces (two-level merge), or nullptr
  int* status;
  int64_t q_stride;
  int64_t kv_block_stride;
  int64_t kv_head_stride;
  int num_seqs;
  int num_heads;
  int num_kv_heads;
  int block_size;
  int max_blocks_per_seq;
  int max_partitions;  // P: partial slots per (sequence, head) in the scratch; 0 = unsplit
  int part_tokens;     // generic kernel: tokens per partition (512)
  int len_cap;         // sequence lengths are clamped to this
  int group;           // query heads per kv head
  int head_groups;     // ceil(group / heads per item)
  int nstages;         // ring slots per warp
  int groups_max;      // ceil(max_partitions / pieces per merge group)
  int use_table;       // 1: split launch (per-sequence unit prefix table in shared memory)
  int min_chunk;       // split launch: smallest range worth a work item, in cache blocks (even)
  float scale;
  // block-sparse attention of the reference signature (generic kernel only); enabled when
  // bs_vert_stride > 1 (attention_kernels.cuh:204-251)
  int tp_rank;
  float* lse;  // optional [num_heads, num_seqs] log-sum-exp output (natural log), or nullptr
  int bs_local_blocks;
  int bs_vert_stride;
  int bs_block_size;
  int bs_head_sliding_step;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: false if the phase did not complete within ~2^32 SM cycles (about two
// seconds).  The clock is read only every 64 polls to keep waiting warps cheap.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (int outer = 0; outer < (1 << 20); ++outer) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > (1ll << 32)) break;
  }
  return false;
}

// 1-D bulk async copy global -> shared, completion counted in bytes on `bar`.
// No cluster multicast: every CTA fetches its own pages.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}

__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(addr)
               : "memory");
}

__device__ __forceinline__ uint32_t movm_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// D(16x8,f32) += A(16x16) * B(16x8); kBf16 selects bf16 operands, else f16.
template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Four fp8 bytes -> two packed f16x2 (lo = bytes 0,1; hi = bytes 2,3), exact.
// One asm block, so that the assembler can read the two halves of `x` in place.
// (Unpacking with integer ALU ops instead, or feeding the bytes to the legacy fp8
// mma.sync, were both measured slower on B200.)
template <bool kE5M2>
__device__ __forceinline__ void fp8x4_to_f16(uint32_t x, uint32_t& lo, uint32_t& hi) {
  if constexpr (kE5M2) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e5m2x2 %0, l;\n\tcvt.rn.f16x2.e5m2x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(x));
  } else {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(x));
  }
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

}  // namespace b200pa
