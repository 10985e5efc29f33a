// Host entry points of paged_attention_v1 / v2, the split-KV reduce kernel and
// the generic (any dtype / head size / block size) SIMT decode kernel.
//
// Replaces: csrc/attention/paged_attention_v1.cu:160-182, paged_attention_v2.cu:167-192
// (host entries and launchers) and attention_kernels.cuh:559-664 (reduce) of the
// reference.
#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cstdint>
#include <cstdlib>
#include <iterator>

#include "decode_inst.cuh"

namespace b200pa {

// ------------------------------------------------------------------ reduce
// out[s,h,:] = sum_j tmp_out[s,h,j,:] * w_j / (sum_j w_j + 1e-6),
// w_j = l_j * 2^(m_j - max_j m_j); one warp per (sequence, head).
// Sequences with <= 1 partition were written to `out` by the decode kernel.
template <typename QT>
__global__ void pa_reduce_kernel(QT* __restrict__ out, const QT* __restrict__ tmp_out,
                                 const float* __restrict__ exp_sums,
                                 const float* __restrict__ max_logits,
                                 const int* __restrict__ seq_lens, int num_seqs, int num_heads,
                                 int head_size, int max_partitions, int part_tokens,
                                 float* __restrict__ lse) {
  extern __shared__ float s_w[];  // [warps][max_partitions]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int item = blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= num_seqs * num_heads) return;
  const int seq = item / num_heads;
  const int len = seq_lens[seq];
  const int np = min((len + part_tokens - 1) / part_tokens, max_partitions);
  if (np <= 1) return;
  float* w = s_w + warp * max_partitions;
  const float* ml = max_logits + int64_t(item) * max_partitions;
  const float* es = exp_sums + int64_t(item) * max_partitions;
  float mx = -INFINITY;
  for (int j = lane; j < np; j += 32) mx = fmaxf(mx, ml[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int j = lane; j < np; j += 32) {
    const float v = es[j] * exp2f(ml[j] - mx);
    w[j] = v;
    sum += v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  const float inv = __fdividef(1.f, sum + 1e-6f);
  if (lse != nullptr && lane == 0)
    lse[int64_t(item % num_heads) * num_seqs + seq] = (mx + log2f(sum)) * kLn2;
  const QT* tp = tmp_out + int64_t(item) * max_partitions * head_size;
  QT* op = out + int64_t(item) * head_size;
  for (int d = lane; d < head_size; d += 32) {
    float acc = 0.f;
    for (int j = 0; j < np; ++j) acc += to_f32(tp[int64_t(j) * head_size + d]) * w[j];
    op[d] = from_f32<QT>(acc * inv);
  }
}

// ------------------------------------------------------------------ generic decode
// Fallback for every combination the tensor-core kernel is not built for
// (fp32 tensors, head size 120, block size 8, unaligned strides, G > 32).
// One warp per (head, sequence, partition); fp32 math throughout.
template <typename CT, int KV>
__device__ __forceinline__ float cache_to_f32(CT v) {
  if constexpr (KV == kCache16) return to_f32(v);
  else return fp8_to_f32<KV == kCacheE5M2>(v);
}

constexpr int kGenericWarps = 4;

template <typename QT, typename CT, int KV>
__global__ void __launch_bounds__(kGenericWarps * 32)
pa_generic_kernel(const DecodeParams p, int head_size, int x) {
  extern __shared__ float s_gen[];  // per warp: q[head_size] + logits[512]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int per_warp = head_size + kPartitionTokens;
  float* sq = s_gen + warp * per_warp;
  float* sl = sq + head_size;

  const int P = p.max_partitions > 0 ? p.max_partitions : 1;
  const int64_t item = int64_t(blockIdx.x) * kGenericWarps + warp;
  if (item >= int64_t(p.num_seqs) * p.num_heads * P) return;
  const int part = int(item % P);
  const int head = int((item / P) % p.num_heads);
  const int seq = int(item / (int64_t(P) * p.num_heads));
  const bool split = p.max_partitions > 0;
  const int len = split ? min(p.seq_lens[seq], p.max_partitions * p.part_tokens) : p.seq_lens[seq];
  const int PT = p.part_tokens;
  const int nparts = split ? max(1, (len + PT - 1) / PT) : 1;
  if (part >= nparts) return;
  const int t0 = split ? part * PT : 0;
  const int t1 = split ? min(len, t0 + PT) : len;
  const int B = p.block_size;
  const int kvh = head / p.group;
  const float kq = KV == kCache16 ? 1.f : *p.k_scale;
  const float vo = KV == kCache16 ? 1.f : *p.v_scale;
  const float qk_scale = p.scale * kLog2e * kq;
  const float slope = p.alibi ? p.alibi[head] * kLog2e : 0.f;
  // block-sparse pattern: a KV block is attended when it is "local" (among the last
  // bs_local_blocks sparse blocks of the sequence) or "remote" (every bs_vert_stride-th,
  // shifted per head); attention_kernels.cuh:204-251
  const bool sparse = p.bs_vert_stride > 1;
  const int q_bs_block = sparse ? (len - 1) / p.bs_block_size : 0;
  const int bs_offset =
      !sparse ? 0
              : (p.bs_head_sliding_step >= 0
                     ? (p.tp_rank * p.num_heads + head) * p.bs_head_sliding_step + 1
                     : (p.tp_rank * p.num_kv_heads + kvh) * (-p.bs_head_sliding_step) + 1);
  auto attended = [&](int tok) -> bool {
    if (!sparse) return true;
    const int kb = (tok / B) * B / p.bs_block_size;
    return ((kb + bs_offset) % p.bs_vert_stride == 0) || (kb > q_bs_block - p.bs_local_blocks);
  };

  const QT* q = static_cast<const QT*>(p.q) + int64_t(seq) * p.q_stride + int64_t(head) * head_size;
  for (int d = lane; d < head_size; d += 32) sq[d] = to_f32(q[d]);
  __syncwarp();

  const CT* kc = static_cast<const CT*>(p.kc);
  const CT* vc = static_cast<const CT*>(p.vc);
  const int* bt = p.block_tables + int64_t(seq) * p.max_blocks_per_seq;
  constexpr int kMaxAcc = 8;  // head_size <= 256
  float acc[kMaxAcc];
#pragma unroll
  for (int i = 0; i < kMaxAcc; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int ts = t0; ts < t1; ts += kPartitionTokens) {
    const int n = min(kPartitionTokens, t1 - ts);
    float lmax = -INFINITY;
    for (int i = lane; i < n; i += 32) {
      const int tok = ts + i;
      const int64_t blk = bt[tok / B];
      const int off = tok % B;
      const CT* kp = kc + blk * p.kv_block_stride + int64_t(kvh) * p.kv_head_stride + off * x;
      float dot = 0.f;
      for (int d0 = 0; d0 < head_size; d0 += x) {
        const CT* kk = kp + int64_t(d0 / x) * B * x;
        for (int e = 0; e < x; ++e) dot += sq[d0 + e] * cache_to_f32<CT, KV>(kk[e]);
      }
      float s = dot * qk_scale;
      if (p.alibi) s += slope * float(tok - len + 1);
      if (!attended(tok)) s = -FLT_MAX;  // skipped block: no weight, as in the reference
      sl[i] = s;
      lmax = fmaxf(lmax, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    const float m_new = fmaxf(m, lmax);
    const float alpha = exp2f(m - m_new);
    float lsum = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float pv = exp2f(sl[i] - m_new);
      sl[i] = attended(ts + i) ? pv : 0.f;  // skipped blocks never reach the P.V product
      lsum += pv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    l = l * alpha + lsum;
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) acc[i] *= alpha;
    __syncwarp();
    for (int i = 0; i < n; ++i) {
      const int tok = ts + i;
      const int64_t blk = bt[tok / B];
      const int off = tok % B;
      const float pv = sl[i];
      const CT* vp = vc + blk * p.kv_block_stride + int64_t(kvh) * p.kv_head_stride + off;
#pragma unroll
      for (int j = 0; j < kMaxAcc; ++j) {
        const int d = lane + 32 * j;
        if (d < head_size) acc[j] += pv * cache_to_f32<CT, KV>(vp[int64_t(d) * B]);
      }
    }
    __syncwarp();
  }

  const float inv = vo * __fdividef(1.f, l + 1e-6f);
  const bool direct = nparts == 1;
  QT* o;
  if (direct) {
    o = static_cast<QT*>(p.out) + (int64_t(seq) * p.num_heads + head) * head_size;
    if (p.lse != nullptr && lane == 0)
      p.lse[int64_t(head) * p.num_seqs + seq] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
  } else {
    const int64_t idx = (int64_t(seq) * p.num_heads + head) * p.max_partitions + part;
    o = static_cast<QT*>(p.tmp_out) + idx * head_size;
    if (lane == 0) {
      p.max_logits[idx] = m;
      p.exp_sums[idx] = l;
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxAcc; ++j) {
    const int d = lane + 32 * j;
    if (d < head_size) o[d] = from_f32<QT>(acc[j] * inv);
  }
}

// ------------------------------------------------------------------ host side
__device__ unsigned g_sched_words[256][2];  // zero-initialised; self-resetting per launch
// Arrival counters of the fused split-KV merge: one per (sequence, kv head, head
// group); zero-initialised and re-armed by the warp that performs the merge.
constexpr int kArriveRegions = 8;
constexpr int kArrivePerRegion = 16384;
__device__ unsigned g_arrive[kArriveRegions][kArrivePerRegion];

// Split-KV workspace of the library.  The reference's v1 has no scratch argument, so a
// sequence could only be handled by one work item; with a small batch that leaves most of
// the GPU idle.  v1 therefore splits sequences into partitions of 64..512 tokens when the
// partials fit this buffer, exactly like v2 does with the caller's scratch; v2 switches to
// it as well when the caller's 512-token partitions are too coarse to fill the GPU.
// Shared by all such calls on a device (one stream at a time).
constexpr size_t kV1ScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_v1_scratch[kV1ScratchBytes];

static unsigned char* v1_scratch_ptr() {
  constexpr int kMaxDev = 64;
  static unsigned char* cache[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  unsigned char* ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_v1_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  }
  return ptr;
}

// Picks the scheduler words (256 rotating slots) and the arrival-counter region
// (8 rotating regions) of one launch.  Rotation keeps launches that overlap on
// different streams apart; launches on one stream are ordered anyway.
static bool launch_slots(unsigned** sched, unsigned** arrive) {
  constexpr int kMaxDev = 64;
  static unsigned* sbase[kMaxDev] = {};
  static unsigned* abase[kMaxDev] = {};
  static std::atomic<unsigned> rr{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return false;
  unsigned* sb = __atomic_load_n(&sbase[dev], __ATOMIC_ACQUIRE);
  unsigned* ab = __atomic_load_n(&abase[dev], __ATOMIC_ACQUIRE);
  if (sb == nullptr || ab == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&sb), g_sched_words) != cudaSuccess ||
        cudaGetSymbolAddress(reinterpret_cast<void**>(&ab), g_arrive) != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    __atomic_store_n(&abase[dev], ab, __ATOMIC_RELEASE);
    __atomic_store_n(&sbase[dev], sb, __ATOMIC_RELEASE);
  }
  const unsigned slot = rr.fetch_add(1, std::memory_order_relaxed);
  *sched = sb + 2 * (slot & 255u);
  *arrive = ab + size_t(slot % kArriveRegions) * kArrivePerRegion;
  return true;
}

static int sm_count() {
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

static DecodeKernelInfo find_decode(int d, int qdt, int kv, int gp, int nt) {
  switch (d) {
    case 32: return find_decode_d32(qdt, kv, gp, nt);
    case 64: return find_decode_d64(qdt, kv, gp, nt);
    case 80: return find_decode_d80(qdt, kv, gp, nt);
    case 96: return find_decode_d96(qdt, kv, gp, nt);
    case 112: return find_decode_d112(qdt, kv, gp, nt);
    case 128: return find_decode_d128(qdt, kv, gp, nt);
    case 192: return find_decode_d192(qdt, kv, gp, nt);
    case 256: return find_decode_d256(qdt, kv, gp, nt);
  }
  return {nullptr, 0, 1};
}

template <typename QT>
static int launch_generic(const DecodeParams& p, const b200pa_attn_args& a, cudaStream_t s) {
  const int P = p.max_partitions > 0 ? p.max_partitions : 1;
  const int64_t items = int64_t(p.num_seqs) * p.num_heads * P;
  const int grid = int((items + kGenericWarps - 1) / kGenericWarps);
  const size_t smem = size_t(kGenericWarps) * (a.head_size + kPartitionTokens) * sizeof(float);
  const int x_wide = 16 / int(sizeof(QT));
  switch (a.kv_dtype) {
    case B200PA_KV_AUTO:
      pa_generic_kernel<QT, QT, kCache16><<<grid, kGenericWarps * 32, smem, s>>>(p, a.head_size, x_wide);
      break;
    case B200PA_KV_FP8_E4M3:
      pa_generic_kernel<QT, uint8_t, kCacheE4M3><<<grid, kGenericWarps * 32, smem, s>>>(p, a.head_size, 16);
      break;
    case B200PA_KV_FP8_E5M2:
      pa_generic_kernel<QT, uint8_t, kCacheE5M2><<<grid, kGenericWarps * 32, smem, s>>>(p, a.head_size, 16);
      break;
    default:
      set_error("Unsupported data type of kv cache: %d", a.kv_dtype);
      return B200PA_EUNSUPPORTED;
  }
  count_launch();
  B200PA_CHECK_CUDA(cudaGetLastError());
  return B200PA_OK;
}

template <typename QT>
static int launch_reduce(const DecodeParams& p, int head_size, cudaStream_t s) {
  const int warps = 4;
  const int items = p.num_seqs * p.num_heads;
  const int grid = (items + warps - 1) / warps;
  const size_t smem = size_t(warps) * p.max_partitions * sizeof(float);
  pa_reduce_kernel<QT><<<grid, warps * 32, smem, s>>>(
      static_cast<QT*>(p.out), static_cast<const QT*>(p.tmp_out), p.exp_sums, p.max_logits,
      p.seq_lens, p.num_seqs, p.num_heads, head_size, p.max_partitions, p.part_tokens, p.lse);
  count_launch();
  B200PA_CHECK_CUDA(cudaGetLastError());
  return B200PA_OK;
}

// Environment switch for tests: B200PA_FORCE_GENERIC=1 routes everything through
// the SIMT kernel so the two implementations can be compared on a GPU.
static bool force_generic() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200PA_FORCE_GENERIC");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

static int attention_entry(const b200pa_attn_args* a, void* stream, bool v2) {
  B200PA_CHECK_ARG(a != nullptr, "args is NULL");
  B200PA_CHECK_ARG(a->num_seqs >= 0 && a->num_heads > 0 && a->num_kv_heads > 0 && a->head_size > 0,
                   "bad sizes: num_seqs=%d num_heads=%d num_kv_heads=%d head_size=%d", a->num_seqs,
                   a->num_heads, a->num_kv_heads, a->head_size);
  B200PA_CHECK_ARG(a->num_heads % a->num_kv_heads == 0,
                   "num_heads %d is not a multiple of num_kv_heads %d", a->num_heads,
                   a->num_kv_heads);
  // same dispatch tables as the reference launchers (paged_attention_v1.cu:90-158)
  static const int kHeadSizes[] = {32, 64, 80, 96, 112, 120, 128, 192, 256};
  bool head_ok = false;
  for (int hs : kHeadSizes) head_ok |= (hs == a->head_size);
  if (!head_ok) {
    set_error("Unsupported head size: %d", a->head_size);
    return B200PA_EUNSUPPORTED;
  }
  if (a->block_size != 8 && a->block_size != 16 && a->block_size != 32) {
    set_error("Unsupported block size: %d", a->block_size);
    return B200PA_EUNSUPPORTED;
  }
  const bool sparse = a->blocksparse_vert_stride > 1;
  if (sparse) {
    B200PA_CHECK_ARG(a->blocksparse_block_size > 0 &&
                         a->blocksparse_block_size % a->block_size == 0,
                     "blocksparse_block_size=%d needs to be a positive multiple of block_size=%d",
                     a->blocksparse_block_size, a->block_size);
  }
  if (a->q_dtype != B200PA_F32 && a->q_dtype != B200PA_F16 && a->q_dtype != B200PA_BF16) {
    set_error("Unsupported input type of kv cache: %d", a->q_dtype);
    return B200PA_EUNSUPPORTED;
  }
  if (a->kv_dtype != B200PA_KV_AUTO && a->kv_dtype != B200PA_KV_FP8_E4M3 &&
      a->kv_dtype != B200PA_KV_FP8_E5M2) {
    set_error("Unsupported data type of kv cache: %d", a->kv_dtype);
    return B200PA_EUNSUPPORTED;
  }
  if (a->num_seqs == 0) return B200PA_OK;
  B200PA_CHECK_ARG(a->out && a->query && a->key_cache && a->value_cache && a->block_tables &&
                       a->seq_lens,
                   "null tensor pointer");
  B200PA_CHECK_ARG(a->kv_dtype == B200PA_KV_AUTO || (a->k_scale && a->v_scale),
                   "fp8 kv cache needs k_scale and v_scale");
  B200PA_CHECK_ARG(a->max_num_blocks_per_seq > 0, "max_num_blocks_per_seq must be positive");
  if (v2) {
    B200PA_CHECK_ARG(a->exp_sums && a->max_logits && a->tmp_out, "v2 needs exp_sums/max_logits/tmp_out");
    B200PA_CHECK_ARG(a->max_num_partitions >= 1 &&
                         int64_t(a->max_num_partitions) * kPartitionTokens >= a->max_seq_len,
                     "max_num_partitions=%d does not cover max_seq_len=%d", a->max_num_partitions,
                     a->max_seq_len);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  DecodeParams p{};
  p.out = a->out;
  p.q = a->query;
  p.kc = a->key_cache;
  p.vc = a->value_cache;
  p.block_tables = a->block_tables;
  p.seq_lens = a->seq_lens;
  p.alibi = a->alibi_slopes;
  p.k_scale = a->k_scale;
  p.v_scale = a->v_scale;
  p.exp_sums = a->exp_sums;
  p.max_logits = a->max_logits;
  p.tmp_out = a->tmp_out;
  p.q_stride = a->q_stride;
  p.kv_block_stride = a->kv_block_stride;
  p.kv_head_stride = a->kv_head_stride;
  p.num_seqs = a->num_seqs;
  p.num_heads = a->num_heads;
  p.num_kv_heads = a->num_kv_heads;
  p.block_size = a->block_size;
  p.max_blocks_per_seq = a->max_num_blocks_per_seq;
  // a single partition needs no scratch and no reduce: run it unsplit
  bool split = v2 && a->max_num_partitions > 1;
  p.max_partitions = split ? a->max_num_partitions : 0;
  p.part_tokens = kPartitionTokens;
  p.group = a->num_heads / a->num_kv_heads;
  p.scale = a->scale;
  p.tp_rank = a->tp_rank;
  p.lse = a->out_lse;
  p.bs_local_blocks = a->blocksparse_local_blocks;
  p.bs_vert_stride = a->blocksparse_vert_stride;
  p.bs_block_size = a->blocksparse_block_size;
  p.bs_head_sliding_step = a->blocksparse_head_sliding_step;

  // ---- can the tensor-core kernel take it?
  const int es = a->kv_dtype == B200PA_KV_AUTO ? 2 : 1;
  auto aligned = [](const void* ptr, uintptr_t n) { return reinterpret_cast<uintptr_t>(ptr) % n == 0; };
  const int gp = p.group <= 8 ? 1 : 2;
  DecodeKernelInfo ki{nullptr, 0, 1};
  // block-sparse attention (unused by any in-tree caller of the reference) runs on the
  // generic kernel only
  bool fast = !force_generic() && !sparse && a->q_dtype != B200PA_F32 &&
              (a->block_size == 16 || a->block_size == 32) && a->head_size % 16 == 0 &&
              aligned(a->key_cache, 16) && aligned(a->value_cache, 16) && aligned(a->query, 16) &&
              aligned(a->out, 16) && (!split || aligned(a->tmp_out, 16)) &&
              (a->kv_block_stride * es) % 16 == 0 && (a->kv_head_stride * es) % 16 == 0 &&
              a->q_stride % 8 == 0;
  if (fast) ki = find_decode(a->head_size, a->q_dtype, a->kv_dtype, gp, a->block_size / 16);
  DecodeLaunchFn fn = ki.fn;
  int rc;
  bool fused = false;
  if (fn != nullptr) {
    p.head_groups = (p.group + 8 * gp - 1) / (8 * gp);
    const size_t page_bytes = size_t(a->head_size) * a->block_size * es;
    // Ring geometry.  Warps hide the latency of the per-page instruction chain, ring slots
    // the latency of HBM; measured on B200 the first matters more and a shallow ring (about
    // 100-130 KiB in flight per SM) beats a deep one when there is work for every warp.
    // A pipeline step is one cache block, or two when blocks are small.  Steps of 4 KiB and
    // more get separate K and V slots; smaller ones share one slot and one barrier.
    const size_t step_bytes = page_bytes * ki.pages_per_step;  // K (or V) bytes per pipeline step
    const int split_kv = step_bytes >= 4096 ? 1 : 0;           // same rule as in the kernel
    const size_t slot_bytes = split_kv ? step_bytes : 2 * step_bytes;
    const size_t min_slots = split_kv ? 2 : 1;
    const size_t budget_total = 227 * 1024 - 1024;  // static smem + slack
    auto ring_budget = [&](bool with_table) {
      const size_t table = with_table ? size_t((p.num_seqs + 1 + 3) & ~3) * 4 : 0;
      return budget_total - std::min(budget_total - 2048, table) - 1024 /* mbarriers */;
    };
    auto warps_for = [&](size_t budget) {
      int w = int(std::min<size_t>(size_t(ki.max_warps), budget / (min_slots * slot_bytes)));
      if (es == 2 && w > 12) w = 12;  // 16-bit caches: 12 warps measured best
      if (w >= 8) w &= ~3;            // same number of warps on each of the 4 schedulers
      return std::max(w, 1);
    };
    // The partition prefix table lives in shared memory; very large batches run
    // without it (one work item per sequence and kv head).
    if (a->max_seq_len > 64 && p.num_seqs <= 12000 && !getenv("B200PA_TUNE_NO_V1_SPLIT")) {
      // Split-KV into the library's own workspace when the caller gave no scratch (v1, or v2
      // with a single 512-token partition) or when the caller's 512-token partitions are too
      // coarse for the batch.  Two regimes, measured on B200:
      //  - fewer work items than resident warps: the launch lasts as long as one item, so take
      //    the finest partition that still gives every item its own warp;
      //  - more: warps pull several items each and a few items per warp balance the load, so
      //    refine while there are at most ~4 per warp.
      // Either way the partitions of one (sequence, kv head) are merged by a single warp,
      // which bounds how many are worth having (fewer when an item carries many heads).
      const int64_t warps_total = int64_t(sm_count()) * warps_for(ring_budget(true));
      const int64_t units = int64_t(p.num_seqs) * p.num_kv_heads * p.head_groups;
      const int heads_per_item = std::min(p.group, 8 * gp);
      int max_parts = std::max(16, 64 / heads_per_item);
      if (const char* e = getenv("B200PA_TUNE_MAX_PARTS")) max_parts = atoi(e);
      auto parts_of = [&](int t) { return (int64_t(a->max_seq_len) + t - 1) / t; };
      int pt = kPartitionTokens;
      const int64_t per_warp = units * parts_of(pt) <= warps_total ? 1 : 4;
      while (pt > 64 && parts_of(pt / 2) <= max_parts &&
             units * parts_of(pt / 2) <= per_warp * warps_total)
        pt /= 2;
      // fp8 caches: a warp's time goes into its own instruction chain (every cache byte is
      // converted before the MMA), not into waiting for HBM, so the fixed cost of an item
      // (~7 us of round trips that nothing overlaps) counts.  Measured on B200 with sequences
      // of equal length, about 1.7 items per warp is the optimum (config 3: 0.376 ms with
      // 512-token partitions, 0.345 ms with 2048); with mixed lengths the count estimated from
      // max_seq_len is about twice the real one and that point is already too coarse.  So:
      // coarsen while the estimate keeps at least `kMinItemsPerWarp` items per warp, and never
      // beyond 2048 tokens (larger items of unequal length lengthen the tail of big batches).
      // 16-bit caches stay at 512 (config 2 loses 5 % with 1024).
      if (es == 1 && pt == kPartitionTokens) {
        int min_items_per_warp = 3;
        if (const char* e = getenv("B200PA_TUNE_FP8_ITEMS")) min_items_per_warp = atoi(e);
        while (pt < 2048 && parts_of(pt) > 1 &&
               units * parts_of(2 * pt) >= min_items_per_warp * warps_total)
          pt *= 2;
      }
      if (const char* e = getenv("B200PA_TUNE_PT")) pt = atoi(e);  // 0: no library split
      if (split && pt > kPartitionTokens) {
        // the caller's scratch has a partition slot per 512 tokens: coarser partitions use the
        // first ceil(len / pt) of them
        p.part_tokens = pt;
      }
      if (pt > 0 && (!split || pt < kPartitionTokens)) {
        auto up = [](int64_t v) { return (v + 255) & ~int64_t(255); };
        auto need_of = [&](int t) {
          const int64_t n = int64_t(p.num_seqs) * p.num_heads * parts_of(t);
          return 2 * up(n * 4) + up(n * a->head_size * 2);
        };
        while (pt < kPartitionTokens && need_of(pt) > int64_t(kV1ScratchBytes)) pt *= 2;
        // fp8 (see above): rather fewer, larger partitions than none at all
        while (es == 1 && parts_of(pt) > 1 && need_of(pt) > int64_t(kV1ScratchBytes)) pt *= 2;
        const int64_t parts = parts_of(pt);
        const int64_t stat = up(int64_t(p.num_seqs) * p.num_heads * parts * 4);
        unsigned char* ws = ((!split || pt < kPartitionTokens) && parts > 1 &&
                             need_of(pt) <= int64_t(kV1ScratchBytes) && units <= kArrivePerRegion)
                                ? v1_scratch_ptr() : nullptr;
        if (ws != nullptr) {
          split = true;
          p.part_tokens = pt;
          p.max_partitions = int(parts);
          p.exp_sums = reinterpret_cast<float*>(ws);
          p.max_logits = reinterpret_cast<float*>(ws + stat);
          p.tmp_out = ws + 2 * stat;
        }
      }
    }
    // The partition table of a split launch lives in shared memory (4 bytes per sequence).
    // Batches it cannot hold have more than enough sequences to fill the GPU unsplit.
    if (split && size_t((p.num_seqs + 1 + 3) & ~3) * 4 > 48 * 1024) {
      split = false;
      p.max_partitions = 0;
    }
    // lengths beyond what the scratch has partitions for are ignored, like the reference's v2
    // grid ignores partitions beyond max_num_partitions
    // (the caller's scratch covers max_partitions * 512 tokens whatever the partition size)
    const int slot_tokens = p.exp_sums == a->exp_sums ? std::min(p.part_tokens, kPartitionTokens)
                                                      : p.part_tokens;
    p.len_cap = split ? int(std::min<int64_t>(int64_t(p.max_partitions) * slot_tokens, INT32_MAX))
                      : INT32_MAX;
    p.use_table = split ? 1 : 0;
    const size_t table_bytes = p.use_table ? size_t((p.num_seqs + 1 + 3) & ~3) * 4 : 0;
    if (table_bytes > 48 * 1024) {
      set_error("num_seqs=%d is too large for the split-KV partition table", a->num_seqs);
      return B200PA_EUNSUPPORTED;
    }
    const size_t budget = ring_budget(p.use_table != 0);
    // B200PA_TUNE_WARPS / B200PA_TUNE_STAGES override (STAGES = slots per warp).
    int nwarps = warps_for(budget);
    if (const char* e = getenv("B200PA_TUNE_WARPS"))
      nwarps = std::max(1, std::min(ki.max_warps, atoi(e)));
    // Launches with fewer work items than warps are bound by the latency of one item, not by
    // bandwidth: run just enough warps to give every item its own (a multiple of 4, at least
    // 4) and spend the shared memory on a deeper ring (<= 8 slots) so that one warp keeps
    // many pages in flight.
    int ns = 2;
    {
      const int64_t parts_ub =
          split ? std::max<int64_t>(1, (int64_t(a->max_seq_len) + p.part_tokens - 1) / p.part_tokens) : 1;
      const int64_t items_ub = int64_t(p.num_seqs) * p.num_kv_heads * p.head_groups * parts_ub;
      if (items_ub <= int64_t(sm_count()) * nwarps && !getenv("B200PA_TUNE_WARPS")) {
        const int need = int((items_ub + sm_count() - 1) / sm_count());
        nwarps = std::min(nwarps, std::max(4, (need + 3) & ~3));
        ns = 8;
      }
    }
    ns = int(std::min<size_t>(size_t(ns), budget / (size_t(nwarps) * slot_bytes)));
    if (const char* e = getenv("B200PA_TUNE_STAGES"))
      ns = std::max(int(min_slots), std::min(int(budget / (size_t(nwarps) * slot_bytes)), atoi(e)));
    if (ns < int(min_slots)) {
      set_error("head_size=%d block_size=%d does not fit the shared-memory pipeline", a->head_size,
                a->block_size);
      return B200PA_EUNSUPPORTED;
    }
    p.nstages = ns;
    unsigned* arrive = nullptr;
    p.status = device_status_ptr();
    if (!launch_slots(&p.sched, &arrive) || p.status == nullptr) {
      set_error("could not resolve device-side scheduler/status words");
      return B200PA_ECUDA;
    }
    // merge the partials inside the decode kernel when the counters cover the batch
    fused = split && int64_t(p.num_seqs) * p.num_kv_heads * p.head_groups <= kArrivePerRegion;
    p.arrive = fused ? arrive : nullptr;
    const size_t bars_bytes = (size_t(nwarps) * ns * 8 + 127) & ~size_t(127);
    const size_t smem = table_bytes + bars_bytes + size_t(nwarps) * ns * slot_bytes;
    const int grid = sm_count();
    cudaError_t e = fn(p, grid, nwarps * 32, smem, s);
    count_launch();
    if (e != cudaSuccess) {
      set_error("decode kernel launch failed: %s", cudaGetErrorString(e));
      return B200PA_ECUDA;
    }
    rc = B200PA_OK;
  } else {
    if (a->head_size > 256) {
      set_error("Unsupported head size: %d", a->head_size);
      return B200PA_EUNSUPPORTED;
    }
    switch (a->q_dtype) {
      case B200PA_F32: rc = launch_generic<float>(p, *a, s); break;
      case B200PA_F16: rc = launch_generic<__half>(p, *a, s); break;
      default: rc = launch_generic<__nv_bfloat16>(p, *a, s); break;
    }
  }
  if (rc != B200PA_OK) return rc;
  if (split && !fused) {
    switch (a->q_dtype) {
      case B200PA_F32: return launch_reduce<float>(p, a->head_size, s);
      case B200PA_F16: return launch_reduce<__half>(p, a->head_size, s);
      default: return launch_reduce<__nv_bfloat16>(p, a->head_size, s);
    }
  }
  return B200PA_OK;
}

}  // namespace b200pa

extern "C" int b200pa_paged_attention_v1(const b200pa_attn_args* args, void* stream) {
  return b200pa::attention_entry(args, stream, false);
}

extern "C" int b200pa_paged_attention_v2(const b200pa_attn_args* args, void* stream) {
  return b200pa::attention_entry(args, stream, true);
}

// ------------------------------------------------------------------ v2 without caller scratch
// Split-KV scratch (exp_sums, max_logits, tmp_out) for callers that cannot
// provide device memory of their own: a plain C host that binds this library
// has no allocator to ask, and a serving process that has already handed all
// free HBM to its KV-cache pool can see cudaMalloc fail late.  The buffer is a
// file-scope device array: every GPU that loads the library holds these 32 MiB
// until the process exits.  All calls on a device share it and it keeps the
// previous call's contents; nothing in it has to start at zero, because the
// decode kernel writes every partial (m, l, O) that the reduce kernel reads.
namespace b200pa {

constexpr size_t kBuiltinScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// `g_builtin_scratch` names a host-side stand-in in host code, not a device
// address: resolve the device address once per device, with that device current.
static unsigned char* builtin_scratch_ptr() {
  constexpr int kMaxDev = 64;
  static unsigned char* cache[kMaxDev] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    set_error("cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  unsigned char* p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_builtin_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      set_error("cudaGetSymbolAddress(built-in scratch) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
  }
  return p;
}

}  // namespace b200pa

extern "C" int b200pa_paged_attention_v2_noalloc(const b200pa_attn_args* args, void* stream) {
  using namespace b200pa;
  B200PA_CHECK_ARG(args != nullptr, "args is NULL");
  B200PA_CHECK_ARG(args->num_seqs >= 0 && args->num_heads > 0 && args->head_size > 0 &&
                       args->max_seq_len >= 0,
                   "bad sizes: num_seqs=%d num_heads=%d head_size=%d max_seq_len=%d", args->num_seqs,
                   args->num_heads, args->head_size, args->max_seq_len);
  const int64_t parts = std::max<int64_t>(
      1, (int64_t(args->max_seq_len) + kPartitionTokens - 1) / kPartitionTokens);
  const int64_t n = int64_t(args->num_seqs) * args->num_heads * parts;
  const int64_t esize = args->q_dtype == B200PA_F32 ? 4 : 2;
  auto up = [](int64_t v) { return (v + 255) & ~int64_t(255); };
  const int64_t stat_bytes = up(n * 4);
  const int64_t need = 2 * stat_bytes + up(n * args->head_size * esize);
  if (need > int64_t(kBuiltinScratchBytes)) {
    set_error("paged_attention_v2_noalloc: num_seqs=%d x num_heads=%d x %lld partitions needs %lld "
              "bytes of split-KV scratch, the built-in buffer holds %lld; use "
              "b200pa_paged_attention_v2 with caller scratch",
              args->num_seqs, args->num_heads, (long long)parts, (long long)need,
              (long long)kBuiltinScratchBytes);
    return B200PA_EINVAL;
  }
  unsigned char* base = builtin_scratch_ptr();
  if (base == nullptr) return B200PA_ECUDA;
  b200pa_attn_args a = *args;
  a.exp_sums = reinterpret_cast<float*>(base);
  a.max_logits = reinterpret_cast<float*>(base + stat_bytes);
  a.tmp_out = base + 2 * stat_bytes;
  a.max_num_partitions = static_cast<int32_t>(parts);
  return attention_entry(&a, stream, true);
}

extern "C" int b200pa_reset_device_state(void* stream) {
  using namespace b200pa;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned* sched = nullptr;
  unsigned* arrive = nullptr;
  int* status = device_status_ptr();
  if (!launch_slots(&sched, &arrive) || status == nullptr) {
    set_error("could not resolve device-side scheduler/status words");
    return B200PA_ECUDA;
  }
  void* sbase = nullptr;
  void* abase = nullptr;
  B200PA_CHECK_CUDA(cudaGetSymbolAddress(&sbase, g_sched_words));
  B200PA_CHECK_CUDA(cudaGetSymbolAddress(&abase, g_arrive));
  B200PA_CHECK_CUDA(cudaMemsetAsync(sbase, 0, sizeof(g_sched_words), s));
  B200PA_CHECK_CUDA(cudaMemsetAsync(abase, 0, sizeof(g_arrive), s));
  B200PA_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int), s));
  return B200PA_OK;
}
