// Operators next to the decode path that work on the same tensors:
//   merge_attn_states  - LSE-weighted merge of two partial attention results
//                        (reference csrc/attention/merge_attn_states.cu:14-212)
//   copy_blocks        - copy whole cache blocks inside every layer's K and V cache
//                        (reference csrc/cache_kernels.cu:73-171)
//   swap_blocks        - copy whole blocks between two caches, host or device
//                        (reference csrc/cache_kernels.cu:26-69)
// All are pure data movement / elementwise work: 16-byte accesses, grids sized
// from the SM count.
#include <cmath>
#include <limits>

#include "common.cuh"

namespace b200pa {

// One thread per 16-byte pack of one (token, head) row.
// output [T, H, D]; lse tensors [H, T] fp32.
template <typename T>
__global__ void merge_attn_states_kernel(T* __restrict__ output, float* __restrict__ output_lse,
                                         const T* __restrict__ prefix_output,
                                         const float* __restrict__ prefix_lse,
                                         const T* __restrict__ suffix_output,
                                         const float* __restrict__ suffix_lse, uint32_t num_tokens,
                                         uint32_t num_heads, uint32_t head_size) {
  constexpr uint32_t PACK = 16 / sizeof(T);
  const uint32_t packs_per_head = head_size / PACK;
  const uint64_t total = uint64_t(num_tokens) * num_heads * packs_per_head;
  const uint64_t idx = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint32_t pack = uint32_t(idx % packs_per_head);
  const uint64_t th = idx / packs_per_head;
  const uint32_t token = uint32_t(th / num_heads);
  const uint32_t head = uint32_t(th % num_heads);
  const uint64_t off = th * head_size + uint64_t(pack) * PACK;

  float p_lse = prefix_lse[uint64_t(head) * num_tokens + token];
  float s_lse = suffix_lse[uint64_t(head) * num_tokens + token];
  // +inf is treated like -inf ("no contribution"), as the reference does
  if (isinf(p_lse)) p_lse = -INFINITY;
  if (isinf(s_lse)) s_lse = -INFINITY;
  const float max_lse = fmaxf(p_lse, s_lse);

  const uint4 pv = *reinterpret_cast<const uint4*>(prefix_output + off);
  if (isinf(max_lse)) {
    // neither side attended to anything: pass the prefix through
    *reinterpret_cast<uint4*>(output + off) = pv;
    if (output_lse != nullptr && pack == 0) output_lse[uint64_t(head) * num_tokens + token] = max_lse;
    return;
  }
  const uint4 sv = *reinterpret_cast<const uint4*>(suffix_output + off);
  const float p_se = expf(p_lse - max_lse);
  const float s_se = expf(s_lse - max_lse);
  const float out_se = p_se + s_se;
  const float p_scale = p_se / out_se;
  const float s_scale = s_se / out_se;
  uint4 ov;
  const T* pe = reinterpret_cast<const T*>(&pv);
  const T* se = reinterpret_cast<const T*>(&sv);
  T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
  for (uint32_t i = 0; i < PACK; ++i)
    oe[i] = from_f32<T>(to_f32(pe[i]) * p_scale + (to_f32(se[i]) * s_scale));
  *reinterpret_cast<uint4*>(output + off) = ov;
  if (output_lse != nullptr && pack == 0)
    output_lse[uint64_t(head) * num_tokens + token] = logf(out_se) + max_lse;
}

// Cache base pointers travel as kernel parameters, so the op needs no device
// allocation, no host-to-device copy and no synchronisation (the reference
// builds pointer tensors on the device inside the op, cache_kernels.cu:150-160).
constexpr int kCopyLayersPerLaunch = 64;
struct CopyBlocksArgs {
  char* key[kCopyLayersPerLaunch];
  char* value[kCopyLayersPerLaunch];
};

// grid = (layers, pairs); 16-byte copies when vec16 != 0.
__global__ void __launch_bounds__(256)
copy_blocks_kernel(const CopyBlocksArgs a, const int64_t* __restrict__ block_mapping,
                   int64_t block_bytes, int vec16) {
  const int layer = blockIdx.x;
  const int64_t src = block_mapping[2 * blockIdx.y] * block_bytes;
  const int64_t dst = block_mapping[2 * blockIdx.y + 1] * block_bytes;
  char* kc = a.key[layer];
  char* vc = a.value[layer];
  if (vec16) {
    const int64_t n = block_bytes / 16;
    const uint4* ks = reinterpret_cast<const uint4*>(kc + src);
    const uint4* vs = reinterpret_cast<const uint4*>(vc + src);
    uint4* kd = reinterpret_cast<uint4*>(kc + dst);
    uint4* vd = reinterpret_cast<uint4*>(vc + dst);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      const uint4 k = ks[i];
      const uint4 v = vs[i];
      kd[i] = k;
      vd[i] = v;
    }
  } else {
    for (int64_t i = threadIdx.x; i < block_bytes; i += blockDim.x) {
      kc[dst + i] = kc[src + i];
      vc[dst + i] = vc[src + i];
    }
  }
}

template <typename T>
static int launch_merge(void* out, float* out_lse, const void* p, const float* pl, const void* s,
                        const float* sl, int64_t nt, int nh, int hs, cudaStream_t stream) {
  constexpr int PACK = 16 / sizeof(T);
  B200PA_CHECK_ARG(hs % PACK == 0, "headsize must be multiple of pack_size:%d", PACK);
  const uint64_t total = uint64_t(nt) * nh * (hs / PACK);
  if (total == 0) return B200PA_OK;
  const int threads = 128;
  const uint64_t blocks = (total + threads - 1) / threads;
  B200PA_CHECK_ARG(blocks < (1ull << 31), "merge_attn_states: problem too large");
  merge_attn_states_kernel<T><<<unsigned(blocks), threads, 0, stream>>>(
      static_cast<T*>(out), out_lse, static_cast<const T*>(p), pl, static_cast<const T*>(s), sl,
      uint32_t(nt), uint32_t(nh), uint32_t(hs));
  count_launch();
  B200PA_CHECK_CUDA(cudaGetLastError());
  return B200PA_OK;
}

}  // namespace b200pa

extern "C" int b200pa_merge_attn_states(void* output, float* output_lse, const void* prefix_output,
                                        const float* prefix_lse, const void* suffix_output,
                                        const float* suffix_lse, int64_t num_tokens,
                                        int32_t num_heads, int32_t head_size, int32_t dtype,
                                        void* stream) {
  using namespace b200pa;
  B200PA_CHECK_ARG(num_tokens >= 0 && num_heads > 0 && head_size > 0, "bad sizes");
  if (num_tokens == 0) return B200PA_OK;
  B200PA_CHECK_ARG(output && prefix_output && prefix_lse && suffix_output && suffix_lse,
                   "null tensor pointer");
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  B200PA_CHECK_ARG(al(output) && al(prefix_output) && al(suffix_output),
                   "output / prefix_output / suffix_output must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200PA_F32:
      return launch_merge<float>(output, output_lse, prefix_output, prefix_lse, suffix_output,
                                 suffix_lse, num_tokens, num_heads, head_size, s);
    case B200PA_F16:
      return launch_merge<__half>(output, output_lse, prefix_output, prefix_lse, suffix_output,
                                  suffix_lse, num_tokens, num_heads, head_size, s);
    case B200PA_BF16:
      return launch_merge<__nv_bfloat16>(output, output_lse, prefix_output, prefix_lse,
                                         suffix_output, suffix_lse, num_tokens, num_heads,
                                         head_size, s);
  }
  set_error("Unsupported data type of O: %d", dtype);
  return B200PA_EUNSUPPORTED;
}

extern "C" int b200pa_copy_blocks(void* const* key_caches, void* const* value_caches,
                                  int32_t num_layers, const int64_t* block_mapping,
                                  int64_t num_pairs, int64_t block_bytes, void* stream) {
  using namespace b200pa;
  B200PA_CHECK_ARG(num_layers >= 0 && num_pairs >= 0 && block_bytes > 0, "bad sizes");
  if (num_layers == 0 || num_pairs == 0) return B200PA_OK;
  B200PA_CHECK_ARG(key_caches && value_caches && block_mapping, "null pointer");
  B200PA_CHECK_ARG(num_pairs <= 65535, "at most 65535 block pairs per call");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int l0 = 0; l0 < num_layers; l0 += kCopyLayersPerLaunch) {
    const int n = num_layers - l0 < kCopyLayersPerLaunch ? num_layers - l0 : kCopyLayersPerLaunch;
    CopyBlocksArgs a{};
    int vec = block_bytes % 16 == 0;
    for (int i = 0; i < n; ++i) {
      a.key[i] = static_cast<char*>(key_caches[l0 + i]);
      a.value[i] = static_cast<char*>(value_caches[l0 + i]);
      B200PA_CHECK_ARG(a.key[i] && a.value[i], "null cache pointer for layer %d", l0 + i);
      if ((reinterpret_cast<uintptr_t>(a.key[i]) | reinterpret_cast<uintptr_t>(a.value[i])) & 15) vec = 0;
    }
    copy_blocks_kernel<<<dim3(n, unsigned(num_pairs)), 256, 0, s>>>(a, block_mapping, block_bytes, vec);
    count_launch();
    B200PA_CHECK_CUDA(cudaGetLastError());
  }
  return B200PA_OK;
}

extern "C" int b200pa_swap_blocks(const void* src, void* dst, const int64_t* block_mapping_host,
                                  int64_t num_pairs, int64_t block_bytes, void* stream) {
  using namespace b200pa;
  B200PA_CHECK_ARG(num_pairs >= 0 && block_bytes > 0, "bad sizes");
  if (num_pairs == 0) return B200PA_OK;
  B200PA_CHECK_ARG(src && dst && block_mapping_host, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one asynchronous copy per block; direction is inferred from the pointers
  for (int64_t i = 0; i < num_pairs; ++i) {
    const int64_t so = block_mapping_host[2 * i] * block_bytes;
    const int64_t d_o = block_mapping_host[2 * i + 1] * block_bytes;
    B200PA_CHECK_CUDA(cudaMemcpyAsync(static_cast<char*>(dst) + d_o,
                                      static_cast<const char*>(src) + so, size_t(block_bytes),
                                      cudaMemcpyDefault, s));
  }
  return B200PA_OK;
}
