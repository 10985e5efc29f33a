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
#include <mutex>

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
constexpr int kStreamSlots = 8;
constexpr int kArrivePerRegion = 32768;
__device__ unsigned g_arrive[kStreamSlots][kArrivePerRegion];
// ... and one per group of pieces of a sequence that is merged in two levels
constexpr int kArrive2PerRegion = 65536;
__device__ unsigned g_arrive2[kStreamSlots][kArrive2PerRegion];

// Split-KV workspace of the library.  The reference's v1 has no scratch argument, so a
// sequence could only be handled by one work item; with a small batch that leaves most of
// the GPU idle.  v1 therefore splits sequences across warps through this buffer exactly
// like v2 does through the caller's scratch, and v2 switches to it when the caller's
// scratch has too few partition slots per sequence for the batch (few, long sequences).
//
// Calls on different streams may overlap on the GPU, so every stream gets a region of its
// own (and its own arrival counters): the first stream seen on a device - the one stream of
// a typical engine - the large region, up to seven more a small one each.  Calls on one
// stream are ordered by the stream and share its region.
constexpr size_t kBigRegionBytes = size_t(32) << 20;
constexpr size_t kSmallRegionBytes = size_t(4) << 20;
constexpr size_t kWorkspaceBytes = kBigRegionBytes + (kStreamSlots - 1) * kSmallRegionBytes;
static __device__ __align__(256) unsigned char g_workspace[kWorkspaceBytes];

struct StreamRegion {
  unsigned char* ws;   // split-KV workspace of this stream
  size_t ws_bytes;
  unsigned* arrive;    // arrival counters of this stream
  unsigned* arrive2;   // ... of its merge groups
};

// Developer knobs, read from the environment once per process (B200PA_TUNE_RELOAD=1 at
// that first read makes every call read them again, for parameter sweeps in one process).
struct Tuning {
  int no_split = 0;      // B200PA_TUNE_NO_SPLIT=1: never use the library workspace
  int max_parts = 0;     // B200PA_TUNE_MAX_PARTS: cap on partial slots per sequence (>= 2)
  int min_tokens = 0;    // B200PA_TUNE_MIN_TOKENS: smallest range, in tokens (multiple of 32)
  int warps = 0;         // B200PA_TUNE_WARPS: warps per CTA
  int stages = 0;        // B200PA_TUNE_STAGES: ring slots per warp
  int reload = 0;
};

static int env_int(const char* name, int lo, int hi) {
  const char* e = getenv(name);
  if (e == nullptr || *e == 0) return 0;
  const long v = strtol(e, nullptr, 10);
  return (v < lo || v > hi) ? 0 : int(v);  // out of range: ignored
}

static Tuning read_tuning() {
  Tuning t;
  t.no_split = env_int("B200PA_TUNE_NO_SPLIT", 0, 1);
  t.max_parts = env_int("B200PA_TUNE_MAX_PARTS", 2, 1024);
  t.min_tokens = env_int("B200PA_TUNE_MIN_TOKENS", 32, 1 << 20) & ~31;
  t.warps = env_int("B200PA_TUNE_WARPS", 1, 16);
  t.stages = env_int("B200PA_TUNE_STAGES", 1, 8);
  t.reload = env_int("B200PA_TUNE_RELOAD", 0, 1);
  return t;
}

static Tuning tuning() {
  static const Tuning first = read_tuning();
  return first.reload ? read_tuning() : first;
}

// Region of the calling stream on the current device, or false when the device's eight
// stream slots are taken by other streams (the caller then runs without the library's
// scratch and counters).  A slot whose stream has not been used for the longest time is
// handed to a new stream, so streams that have been destroyed do not use the slots up;
// more than eight streams calling concurrently are not kept apart.
static bool stream_region(cudaStream_t stream, StreamRegion* out) {
  constexpr int kMaxDev = 64;
  struct DevState {
    unsigned char* ws = nullptr;
    unsigned* arrive = nullptr;
    unsigned* arrive2 = nullptr;
    uintptr_t key[kStreamSlots] = {};
    uint64_t used[kStreamSlots] = {};
    int n = 0;
    uint64_t clock = 0;
  };
  static DevState state[kMaxDev];
  static std::mutex mu;
  static thread_local char thread_tag;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return false;
  // the legacy default stream has two handles; the per-thread default stream is one handle
  // for a different stream in every host thread
  uintptr_t key = reinterpret_cast<uintptr_t>(stream);
  if (stream == cudaStreamLegacy) key = 0;
  if (stream == cudaStreamPerThread) key = reinterpret_cast<uintptr_t>(&thread_tag) | 1u;
  key += 16;  // 0 marks a free entry
  std::lock_guard<std::mutex> lock(mu);
  DevState& d = state[dev];
  if (d.ws == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&d.ws), g_workspace) != cudaSuccess ||
        cudaGetSymbolAddress(reinterpret_cast<void**>(&d.arrive), g_arrive) != cudaSuccess ||
        cudaGetSymbolAddress(reinterpret_cast<void**>(&d.arrive2), g_arrive2) != cudaSuccess) {
      (void)cudaGetLastError();
      d.ws = nullptr;
      return false;
    }
  }
  int idx = -1;
  for (int i = 0; i < d.n; ++i)
    if (d.key[i] == key) idx = i;
  if (idx < 0) {
    if (d.n < kStreamSlots) {
      idx = d.n++;
    } else {
      idx = 1;  // the large region stays with the first stream
      for (int i = 2; i < kStreamSlots; ++i)
        if (d.used[i] < d.used[idx]) idx = i;
    }
    d.key[idx] = key;
  }
  d.used[idx] = ++d.clock;
  out->ws = idx == 0 ? d.ws : d.ws + kBigRegionBytes + size_t(idx - 1) * kSmallRegionBytes;
  out->ws_bytes = idx == 0 ? kBigRegionBytes : kSmallRegionBytes;
  out->arrive = d.arrive + size_t(idx) * kArrivePerRegion;
  out->arrive2 = d.arrive2 + size_t(idx) * kArrive2PerRegion;
  return true;
}

// Scheduler words of one launch (256 rotating slots; only unsplit launches with more than
// three items per warp use them).
static unsigned* sched_words() {
  constexpr int kMaxDev = 64;
  static unsigned* sbase[kMaxDev] = {};
  static std::atomic<unsigned> rr{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  unsigned* sb = __atomic_load_n(&sbase[dev], __ATOMIC_ACQUIRE);
  if (sb == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&sb), g_sched_words) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    __atomic_store_n(&sbase[dev], sb, __ATOMIC_RELEASE);
  }
  return sb + 2 * (rr.fetch_add(1, std::memory_order_relaxed) & 255u);
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

// How an attention call may use scratch memory.
enum class Scratch {
  kNone,      // paged_attention_v1: no scratch argument; the library workspace if it helps
  kCaller,    // paged_attention_v2: the caller's exp_sums / max_logits / tmp_out, one partial
              // slot per 512 tokens of max_seq_len; the library workspace if that is too coarse
  kOwnArray   // the scratch pointers are an array of the library with `max_num_partitions`
              // slots per (sequence, head), not tied to 512 tokens; nothing else is used
};

static int attention_entry(const b200pa_attn_args* a, void* stream, Scratch mode) {
  const bool v2 = mode != Scratch::kNone;
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
  // The K cache keeps x = 16 / sizeof(cache element) consecutive head dimensions together,
  // so the head size has to be a multiple of x: an fp8 cache (x = 16) cannot hold head size
  // 120 (the reference's cache factory asserts the same, vllm/utils/torch_utils.py:259-262).
  {
    const int x = a->kv_dtype != B200PA_KV_AUTO ? 16 : 16 / dtype_size(a->q_dtype);
    if (a->head_size % x != 0) {
      set_error("Unsupported head size %d for this kv cache type: it is not a multiple of x = %d",
                a->head_size, x);
      return B200PA_EUNSUPPORTED;
    }
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
    B200PA_CHECK_ARG(a->max_num_partitions >= 1, "max_num_partitions=%d", a->max_num_partitions);
    B200PA_CHECK_ARG(mode == Scratch::kOwnArray ||
                         int64_t(a->max_num_partitions) * kPartitionTokens >= a->max_seq_len,
                     "max_num_partitions=%d does not cover max_seq_len=%d", a->max_num_partitions,
                     a->max_seq_len);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Tuning tune = tuning();

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
  p.len_cap = INT32_MAX;
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
    const size_t budget_total = 227 * 1024 - 2048;  // static smem + slack
    const size_t table_full = size_t((p.num_seqs + 1 + 3) & ~3) * 4;
    auto ring_budget = [&](bool with_table) {
      const size_t table = with_table ? table_full : 0;
      return budget_total - std::min(budget_total - 2048, table) - 1024 /* mbarriers */;
    };
    auto warps_for = [&](size_t budget) {
      int w = int(std::min<size_t>(size_t(ki.max_warps), budget / (min_slots * slot_bytes)));
      if (es == 2 && w > 12) w = 12;  // 16-bit caches: 12 warps measured best
      if (w >= 8) w &= ~3;            // same number of warps on each of the 4 schedulers
      return std::max(w, 1);
    };

    // ---- split-KV plan.  The kernel cuts the flat list of (head, sequence, cache block)
    // units into equal ranges by itself, from the real lengths; what the host decides is
    // where the partials go and how many slots P a (sequence, head) has there, which bounds
    // how finely the longest sequence can be cut.
    const int64_t units_hs = int64_t(p.num_seqs) * p.num_kv_heads * p.head_groups;
    const int64_t pages_max = (int64_t(std::max(a->max_seq_len, 1)) + a->block_size - 1) / a->block_size;
    const int min_tokens = tune.min_tokens ? tune.min_tokens : 64;
    const int min_chunk = std::max(2, (min_tokens / a->block_size + 1) & ~1);
    const int64_t warps_total = int64_t(sm_count()) * warps_for(ring_budget(true));
    StreamRegion region{};
    // the unit table lives in shared memory (4 bytes per sequence) and the merge needs one
    // arrival counter per (sequence, head); batches beyond either have more than enough
    // sequences to fill the GPU unsplit
    const bool can_split = table_full <= 48 * 1024 && units_hs <= kArrivePerRegion &&
                           pages_max > min_chunk && stream_region(s, &region);
    bool own_ws = false;
    if (!can_split) {
      split = false;
    } else {
      // slots worth having: the finest cut the kernel would make if the sequences were a
      // quarter as long as max_seq_len on average (it only knows the bound; skewed batches
      // have a few long sequences and many short ones)
      const int64_t c_est = std::max<int64_t>(min_chunk, units_hs * pages_max / 4 / warps_total);
      const int64_t p_need = std::min<int64_t>(pages_max / c_est + 2, pages_max / min_chunk + 2);
      const int p_cap = tune.max_parts ? tune.max_parts : 128;
      // what the stream's region of the library workspace can hold
      const int64_t per_slot = int64_t(p.num_seqs) * p.num_heads * (8 + int64_t(a->head_size) * 2);
      int64_t p_ws = (int64_t(region.ws_bytes) - 3 * 256) / std::max<int64_t>(per_slot, 1);
      p_ws = std::min<int64_t>({p_ws, int64_t(p_cap), pages_max / min_chunk + 2});
      if (tune.no_split || mode == Scratch::kOwnArray) p_ws = 0;
      const int64_t p_caller = split ? std::min<int64_t>(a->max_num_partitions, p_cap) : 0;
      if (p_caller >= 2 && (p_caller >= p_need || p_caller >= p_ws)) {
        // the layout inside the caller's scratch is the library's business: rows of
        // p_caller slots (no more than the caller's own row length)
        p.max_partitions = int(p_caller);
      } else if (p_ws >= 2) {
        own_ws = true;
        split = true;
        auto up = [](int64_t v) { return (v + 255) & ~int64_t(255); };
        const int64_t stat = up(int64_t(p.num_seqs) * p.num_heads * p_ws * 4);
        p.max_partitions = int(p_ws);
        p.exp_sums = reinterpret_cast<float*>(region.ws);
        p.max_logits = reinterpret_cast<float*>(region.ws + stat);
        p.tmp_out = region.ws + 2 * stat;
      } else {
        split = false;
      }
    }
    if (split) {
      // lengths beyond what the caller's scratch was sized for are ignored, like the
      // reference's v2 grid ignores partitions beyond max_num_partitions
      if (!own_ws && mode == Scratch::kCaller)
        p.len_cap = int(std::min<int64_t>(int64_t(a->max_num_partitions) * kPartitionTokens, INT32_MAX));
    } else {
      p.max_partitions = 0;
    }
    p.use_table = split ? 1 : 0;
    p.min_chunk = min_chunk;
    const size_t table_bytes = split ? table_full : 0;
    const size_t budget = ring_budget(split);
    int nwarps = warps_for(budget);
    if (tune.warps)  // (never more than the shared memory has ring slots for)
      nwarps = std::max(1, std::min({ki.max_warps, tune.warps, int(budget / (min_slots * slot_bytes))}));
    // Ring slots per warp: two.  Measured on B200, a launch with work for every warp is 3-5 %
    // slower when the CTA is given shared memory for four slots per warp, even if only two of
    // them are kept in flight; a split launch whose batch turns out to have fewer ranges than
    // the grid has warps deepens the rings of its busy warps by itself with the slots of the
    // idle ones.  Unsplit launches with fewer work items than warps are bound by the latency of
    // one item: just enough warps to give every item its own (a multiple of 4, at least 4) and
    // the shared memory spent on a deeper ring (<= 8 slots).
    int ns = 2;
    if (!split) {
      const int64_t items = units_hs;
      if (items <= int64_t(sm_count()) * nwarps && !tune.warps) {
        const int need = int((items + sm_count() - 1) / sm_count());
        nwarps = std::min(nwarps, std::max(4, (need + 3) & ~3));
        ns = 8;
      }
    }
    ns = int(std::min<size_t>(size_t(ns), budget / (size_t(nwarps) * slot_bytes)));
    if (tune.stages)
      ns = std::max(int(min_slots), std::min(int(budget / (size_t(nwarps) * slot_bytes)), tune.stages));
    if (ns < int(min_slots)) {
      set_error("head_size=%d block_size=%d does not fit the shared-memory pipeline", a->head_size,
                a->block_size);
      return B200PA_EUNSUPPORTED;
    }
    p.nstages = ns;
    p.status = device_status_ptr();
    p.sched = sched_words();
    if (p.sched == nullptr || p.status == nullptr) {
      set_error("could not resolve device-side scheduler/status words");
      return B200PA_ECUDA;
    }
    // the partials are merged inside the decode kernel
    fused = split;
    p.arrive = fused ? region.arrive : nullptr;
    // sequences cut into many pieces are merged in two levels when there are counters for the
    // groups of every (sequence, head)
    p.groups_max = (p.max_partitions + kMergeFan - 1) / kMergeFan;
    p.arrive2 = (fused && p.max_partitions > kMergeDirectMax &&
                 units_hs * p.groups_max <= kArrive2PerRegion) ? region.arrive2 : nullptr;
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
  return b200pa::attention_entry(args, stream, b200pa::Scratch::kNone);
}

extern "C" int b200pa_paged_attention_v2(const b200pa_attn_args* args, void* stream) {
  return b200pa::attention_entry(args, stream, b200pa::Scratch::kCaller);
}

// ------------------------------------------------------------------ v2 without caller scratch
// Split-KV scratch (exp_sums, max_logits, tmp_out) for callers that cannot
// provide device memory of their own: a plain C host that binds this library
// has no allocator to ask, and a serving process that has already handed all
// free HBM to its KV-cache pool can see cudaMalloc fail late.  The buffer is a
// file-scope device array: every GPU that loads the library holds these 32 MiB
// until the process exits.  All calls on a device share it and it keeps the
// previous call's contents; nothing in it has to start at zero, because the
// decode kernel writes every partial (m, l, O) that the merge reads.
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
  // the documented limit: one partial slot per 512 tokens of max_seq_len has to fit
  const int64_t parts = std::max<int64_t>(
      1, (int64_t(args->max_seq_len) + kPartitionTokens - 1) / kPartitionTokens);
  const int64_t rows = int64_t(args->num_seqs) * args->num_heads;
  const int64_t esize = args->q_dtype == B200PA_F32 ? 4 : 2;
  auto up = [](int64_t v) { return (v + 255) & ~int64_t(255); };
  auto need_of = [&](int64_t slots) {
    return 2 * up(rows * slots * 4) + up(rows * slots * args->head_size * esize);
  };
  if (need_of(parts) > int64_t(kBuiltinScratchBytes)) {
    set_error("paged_attention_v2_noalloc: num_seqs=%d x num_heads=%d x %lld partitions needs %lld "
              "bytes of split-KV scratch, the built-in buffer holds %lld; use "
              "b200pa_paged_attention_v2 with caller scratch",
              args->num_seqs, args->num_heads, (long long)parts, (long long)need_of(parts),
              (long long)kBuiltinScratchBytes);
    return B200PA_EINVAL;
  }
  unsigned char* base = builtin_scratch_ptr();
  if (base == nullptr) return B200PA_ECUDA;
  // Room left in the array becomes more slots per (sequence, head): a small batch of long
  // sequences can then be cut finer than one piece per 512 tokens.
  int64_t slots = parts;
  while (slots < 128 && need_of(slots * 2) <= int64_t(kBuiltinScratchBytes)) slots *= 2;
  const int64_t stat_bytes = up(rows * slots * 4);
  b200pa_attn_args a = *args;
  a.exp_sums = reinterpret_cast<float*>(base);
  a.max_logits = reinterpret_cast<float*>(base + stat_bytes);
  a.tmp_out = base + 2 * stat_bytes;
  a.max_num_partitions = static_cast<int32_t>(slots);
  return attention_entry(&a, stream, Scratch::kOwnArray);
}

extern "C" int b200pa_reset_device_state(void* stream) {
  using namespace b200pa;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = device_status_ptr();
  if (status == nullptr) {
    set_error("could not resolve the device-side status word");
    return B200PA_ECUDA;
  }
  void* sbase = nullptr;
  void* abase = nullptr;
  B200PA_CHECK_CUDA(cudaGetSymbolAddress(&sbase, g_sched_words));
  void* a2base = nullptr;
  B200PA_CHECK_CUDA(cudaGetSymbolAddress(&abase, g_arrive));
  B200PA_CHECK_CUDA(cudaGetSymbolAddress(&a2base, g_arrive2));
  B200PA_CHECK_CUDA(cudaMemsetAsync(sbase, 0, sizeof(g_sched_words), s));
  B200PA_CHECK_CUDA(cudaMemsetAsync(abase, 0, sizeof(g_arrive), s));
  B200PA_CHECK_CUDA(cudaMemsetAsync(a2base, 0, sizeof(g_arrive2), s));
  B200PA_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int), s));
  return B200PA_OK;
}
