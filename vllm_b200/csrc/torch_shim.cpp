// PyTorch registration shim: the only file of the product that includes torch
// headers.  It unwraps tensors into the POD argument blocks of include/b200pa.h,
// sets the device guard, fetches the current stream, calls the C-ABI launcher
// and turns a non-zero return into a c10::Error (Python RuntimeError), like the
// reference's TORCH_CHECKs.
//
// Operator schemas are byte-for-byte those of the reference
// (csrc/torch_bindings.cpp:52-76, :687-704, :716-719).  The ops are always
// registered as torch.ops._C_b200.* / torch.ops._C_b200_cache_ops.*; on request
// (b200_claim_reference_names) also under the reference's own names
// (_C / _C_cache_ops), so code written against vllm._custom_ops runs unchanged.
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/all.h>
#include <torch/library.h>

#include <cstdio>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "../../include/b200pa.h"

namespace {

int dtype_code(at::ScalarType t, const char* what) {
  switch (t) {
    case at::ScalarType::Float: return B200PA_F32;
    case at::ScalarType::Half: return B200PA_F16;
    case at::ScalarType::BFloat16: return B200PA_BF16;
    default: TORCH_CHECK(false, "Unsupported input type of ", what, ": ", t);
  }
  return -1;
}

int kv_code(const std::string& s) {
  const int v = b200pa_kv_dtype_from_string(s.c_str());
  TORCH_CHECK(v >= 0, "Unsupported data type of kv cache: ", s);
  return v;
}

void check_rc(int rc) { TORCH_CHECK(rc == 0, "b200pa: ", b200pa_last_error()); }

void check_cuda(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

void fill_attn(b200pa_attn_args& a, torch::Tensor& out, torch::Tensor& query,
               torch::Tensor& key_cache, torch::Tensor& value_cache, int64_t num_kv_heads,
               double scale, torch::Tensor& block_tables, torch::Tensor& seq_lens,
               int64_t block_size, int64_t max_seq_len,
               const std::optional<torch::Tensor>& alibi_slopes, const std::string& kv_cache_dtype,
               torch::Tensor& k_scale, torch::Tensor& v_scale, int64_t tp_rank,
               int64_t bs_local, int64_t bs_vert, int64_t bs_block, int64_t bs_step) {
  check_cuda(out, "out");
  check_cuda(query, "query");
  check_cuda(key_cache, "key_cache");
  check_cuda(value_cache, "value_cache");
  check_cuda(block_tables, "block_tables");
  check_cuda(seq_lens, "seq_lens");
  TORCH_CHECK(query.dim() == 3, "query must be [num_seqs, num_heads, head_size]");
  TORCH_CHECK(out.is_contiguous(), "out must be contiguous");
  TORCH_CHECK(out.scalar_type() == query.scalar_type(), "out and query dtypes differ");
  TORCH_CHECK(query.stride(2) == 1 && query.stride(1) == query.size(2),
              "query heads must be contiguous");
  TORCH_CHECK(block_tables.scalar_type() == at::ScalarType::Int && block_tables.is_contiguous(),
              "block_tables must be a contiguous int32 tensor");
  TORCH_CHECK(seq_lens.scalar_type() == at::ScalarType::Int && seq_lens.is_contiguous(),
              "seq_lens must be a contiguous int32 tensor");
  TORCH_CHECK(key_cache.dim() == 5 && value_cache.dim() == 4, "caches must be 5-D (K) and 4-D (V)");
  std::memset(&a, 0, sizeof(a));
  a.q_dtype = dtype_code(query.scalar_type(), "kv cache");
  a.kv_dtype = kv_code(kv_cache_dtype);
  if (a.kv_dtype == B200PA_KV_AUTO) {
    TORCH_CHECK(key_cache.scalar_type() == query.scalar_type() &&
                    value_cache.scalar_type() == query.scalar_type(),
                "kv_cache_dtype 'auto' needs caches of the query dtype");
  } else {
    TORCH_CHECK(key_cache.element_size() == 1 && value_cache.element_size() == 1,
                "fp8 kv cache tensors must have 1-byte elements");
    TORCH_CHECK(k_scale.is_cuda() && v_scale.is_cuda() &&
                    k_scale.scalar_type() == at::ScalarType::Float &&
                    v_scale.scalar_type() == at::ScalarType::Float,
                "k_scale / v_scale must be float32 CUDA tensors");
  }
  a.out = out.data_ptr();
  a.query = query.data_ptr();
  a.key_cache = key_cache.data_ptr();
  a.value_cache = value_cache.data_ptr();
  a.block_tables = block_tables.data_ptr<int>();
  a.seq_lens = seq_lens.data_ptr<int>();
  if (alibi_slopes.has_value()) {
    TORCH_CHECK(alibi_slopes->scalar_type() == at::ScalarType::Float && alibi_slopes->is_cuda(),
                "alibi_slopes must be a float32 CUDA tensor");
    a.alibi_slopes = alibi_slopes->data_ptr<float>();
  }
  a.k_scale = k_scale.defined() && k_scale.is_cuda() ? static_cast<const float*>(k_scale.data_ptr()) : nullptr;
  a.v_scale = v_scale.defined() && v_scale.is_cuda() ? static_cast<const float*>(v_scale.data_ptr()) : nullptr;
  a.q_stride = query.stride(0);
  a.kv_block_stride = key_cache.stride(0);
  a.kv_head_stride = key_cache.stride(1);
  a.num_seqs = static_cast<int32_t>(query.size(0));
  a.num_heads = static_cast<int32_t>(query.size(1));
  a.num_kv_heads = static_cast<int32_t>(num_kv_heads);
  a.head_size = static_cast<int32_t>(query.size(2));
  a.block_size = static_cast<int32_t>(block_size);
  a.max_seq_len = static_cast<int32_t>(max_seq_len);
  a.max_num_blocks_per_seq = static_cast<int32_t>(block_tables.size(1));
  a.scale = static_cast<float>(scale);
  a.tp_rank = static_cast<int32_t>(tp_rank);
  a.blocksparse_local_blocks = static_cast<int32_t>(bs_local);
  a.blocksparse_vert_stride = static_cast<int32_t>(bs_vert);
  a.blocksparse_block_size = static_cast<int32_t>(bs_block);
  a.blocksparse_head_sliding_step = static_cast<int32_t>(bs_step);
}

void paged_attention_v1(torch::Tensor& out, torch::Tensor& query, torch::Tensor& key_cache,
                        torch::Tensor& value_cache, int64_t num_kv_heads, double scale,
                        torch::Tensor& block_tables, torch::Tensor& seq_lens, int64_t block_size,
                        int64_t max_seq_len, const std::optional<torch::Tensor>& alibi_slopes,
                        const std::string& kv_cache_dtype, torch::Tensor& k_scale,
                        torch::Tensor& v_scale, const int64_t tp_rank,
                        const int64_t blocksparse_local_blocks,
                        const int64_t blocksparse_vert_stride,
                        const int64_t blocksparse_block_size,
                        const int64_t blocksparse_head_sliding_step) {
  b200pa_attn_args a;
  fill_attn(a, out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
            block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale, tp_rank,
            blocksparse_local_blocks, blocksparse_vert_stride, blocksparse_block_size,
            blocksparse_head_sliding_step);
  const at::cuda::OptionalCUDAGuard device_guard(device_of(query));
  check_rc(b200pa_paged_attention_v1(&a, at::cuda::getCurrentCUDAStream().stream()));
}

// paged_attention_v1 that also returns the log-sum-exp of every (head, sequence), the
// quantity merge_attn_states needs to combine attention over disjoint token ranges.  Not
// an op of the reference: registered under the _C_b200 namespace only.
void paged_attention_with_lse(torch::Tensor& out, torch::Tensor& lse, torch::Tensor& query,
                              torch::Tensor& key_cache, torch::Tensor& value_cache,
                              int64_t num_kv_heads, double scale, torch::Tensor& block_tables,
                              torch::Tensor& seq_lens, int64_t block_size, int64_t max_seq_len,
                              const std::optional<torch::Tensor>& alibi_slopes,
                              const std::string& kv_cache_dtype, torch::Tensor& k_scale,
                              torch::Tensor& v_scale) {
  b200pa_attn_args a;
  fill_attn(a, out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
            block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale, 0, 0, 0, 64, 0);
  check_cuda(lse, "lse");
  TORCH_CHECK(lse.scalar_type() == at::ScalarType::Float && lse.is_contiguous() && lse.dim() == 2 &&
                  lse.size(0) == query.size(1) && lse.size(1) == query.size(0),
              "lse must be a contiguous float32 tensor [num_heads, num_seqs]");
  a.out_lse = lse.data_ptr<float>();
  const at::cuda::OptionalCUDAGuard device_guard(device_of(query));
  check_rc(b200pa_paged_attention_v1(&a, at::cuda::getCurrentCUDAStream().stream()));
}

void paged_attention_v2(torch::Tensor& out, torch::Tensor& exp_sums, torch::Tensor& max_logits,
                        torch::Tensor& tmp_out, torch::Tensor& query, torch::Tensor& key_cache,
                        torch::Tensor& value_cache, int64_t num_kv_heads, double scale,
                        torch::Tensor& block_tables, torch::Tensor& seq_lens, int64_t block_size,
                        int64_t max_seq_len, const std::optional<torch::Tensor>& alibi_slopes,
                        const std::string& kv_cache_dtype, torch::Tensor& k_scale,
                        torch::Tensor& v_scale, const int64_t tp_rank,
                        const int64_t blocksparse_local_blocks,
                        const int64_t blocksparse_vert_stride,
                        const int64_t blocksparse_block_size,
                        const int64_t blocksparse_head_sliding_step) {
  b200pa_attn_args a;
  fill_attn(a, out, query, key_cache, value_cache, num_kv_heads, scale, block_tables, seq_lens,
            block_size, max_seq_len, alibi_slopes, kv_cache_dtype, k_scale, v_scale, tp_rank,
            blocksparse_local_blocks, blocksparse_vert_stride, blocksparse_block_size,
            blocksparse_head_sliding_step);
  check_cuda(exp_sums, "exp_sums");
  check_cuda(max_logits, "max_logits");
  check_cuda(tmp_out, "tmp_out");
  TORCH_CHECK(exp_sums.dim() == 3 && exp_sums.is_contiguous() && max_logits.is_contiguous() &&
                  tmp_out.is_contiguous(),
              "exp_sums / max_logits / tmp_out must be contiguous");
  TORCH_CHECK(exp_sums.scalar_type() == at::ScalarType::Float &&
                  max_logits.scalar_type() == at::ScalarType::Float &&
                  tmp_out.scalar_type() == query.scalar_type(),
              "exp_sums / max_logits must be float32 and tmp_out of the query dtype");
  TORCH_CHECK(max_logits.sizes() == exp_sums.sizes() && exp_sums.size(0) == query.size(0) &&
                  exp_sums.size(1) == query.size(1) && tmp_out.numel() == exp_sums.numel() * query.size(2),
              "v2 scratch tensors have inconsistent shapes");
  a.exp_sums = exp_sums.data_ptr<float>();
  a.max_logits = max_logits.data_ptr<float>();
  a.tmp_out = tmp_out.data_ptr();
  a.max_num_partitions = static_cast<int32_t>(exp_sums.size(2));
  const at::cuda::OptionalCUDAGuard device_guard(device_of(query));
  check_rc(b200pa_paged_attention_v2(&a, at::cuda::getCurrentCUDAStream().stream()));
}

void fill_cache(b200pa_cache_args& a, torch::Tensor& key, torch::Tensor& value,
                torch::Tensor& key_cache, torch::Tensor& value_cache, torch::Tensor& slot_mapping,
                const std::string& kv_cache_dtype, torch::Tensor& k_scale, torch::Tensor& v_scale) {
  check_cuda(key, "key");
  check_cuda(value, "value");
  check_cuda(key_cache, "key_cache");
  check_cuda(value_cache, "value_cache");
  check_cuda(slot_mapping, "slot_mapping");
  TORCH_CHECK(key.dim() == 3 && value.dim() == 3, "key/value must be [num_tokens, num_heads, head_size]");
  TORCH_CHECK(key.stride(2) == 1 && key.stride(1) == key.size(2) && value.stride(2) == 1 &&
                  value.stride(1) == value.size(2),
              "key/value heads must be contiguous");
  TORCH_CHECK(slot_mapping.scalar_type() == at::ScalarType::Long && slot_mapping.is_contiguous(),
              "slot_mapping must be a contiguous int64 tensor");
  std::memset(&a, 0, sizeof(a));
  a.in_dtype = dtype_code(key.scalar_type(), "kv cache");
  TORCH_CHECK(value.scalar_type() == key.scalar_type(), "key and value dtypes differ");
  a.kv_dtype = kv_code(kv_cache_dtype);
  if (a.kv_dtype == B200PA_KV_AUTO) {
    TORCH_CHECK(key_cache.scalar_type() == key.scalar_type() &&
                    value_cache.scalar_type() == key.scalar_type(),
                "kv_cache_dtype 'auto' needs caches of the key dtype");
  } else {
    TORCH_CHECK(key_cache.element_size() == 1 && value_cache.element_size() == 1,
                "fp8 kv cache tensors must have 1-byte elements");
    TORCH_CHECK(k_scale.is_cuda() && v_scale.is_cuda() &&
                    k_scale.scalar_type() == at::ScalarType::Float &&
                    v_scale.scalar_type() == at::ScalarType::Float,
                "k_scale / v_scale must be float32 CUDA tensors");
  }
  a.key = key.data_ptr();
  a.value = value.data_ptr();
  a.key_cache = key_cache.data_ptr();
  a.value_cache = value_cache.data_ptr();
  a.slot_mapping = slot_mapping.data_ptr<int64_t>();
  a.k_scale = k_scale.defined() && k_scale.is_cuda() ? static_cast<const float*>(k_scale.data_ptr()) : nullptr;
  a.v_scale = v_scale.defined() && v_scale.is_cuda() ? static_cast<const float*>(v_scale.data_ptr()) : nullptr;
  a.key_stride = key.stride(0);
  a.value_stride = value.stride(0);
  a.num_tokens = static_cast<int32_t>(slot_mapping.size(0));
  a.num_heads = static_cast<int32_t>(key.size(1));
  a.head_size = static_cast<int32_t>(key.size(2));
}

void reshape_and_cache(torch::Tensor& key, torch::Tensor& value, torch::Tensor& key_cache,
                       torch::Tensor& value_cache, torch::Tensor& slot_mapping,
                       const std::string& kv_cache_dtype, torch::Tensor& k_scale,
                       torch::Tensor& v_scale) {
  b200pa_cache_args a;
  fill_cache(a, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  TORCH_CHECK(key_cache.dim() == 5 && value_cache.dim() == 4,
              "key_cache must be [num_blocks, num_heads, head_size/x, block_size, x] and "
              "value_cache [num_blocks, num_heads, head_size, block_size]");
  TORCH_CHECK(key_cache.is_contiguous() && value_cache.is_contiguous(),
              "reshape_and_cache needs contiguous caches");
  a.block_size = static_cast<int32_t>(key_cache.size(3));
  a.x = static_cast<int32_t>(key_cache.size(4));
  const at::cuda::OptionalCUDAGuard device_guard(device_of(key));
  check_rc(b200pa_reshape_and_cache(&a, at::cuda::getCurrentCUDAStream().stream()));
}

void reshape_and_cache_flash(torch::Tensor& key, torch::Tensor& value, torch::Tensor& key_cache,
                             torch::Tensor& value_cache, torch::Tensor& slot_mapping,
                             const std::string& kv_cache_dtype, torch::Tensor& k_scale,
                             torch::Tensor& v_scale) {
  b200pa_cache_args a;
  fill_cache(a, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale);
  TORCH_CHECK(key_cache.dim() == 4 && value_cache.dim() == 4,
              "caches must be [num_blocks, block_size, num_heads, head_size] (possibly strided)");
  TORCH_CHECK(key_cache.stride(0) == value_cache.stride(0));
  TORCH_CHECK(key_cache.stride(3) == 1 && value_cache.stride(3) == 1,
              "the head_size dimension of the caches must be contiguous");
  a.block_size = static_cast<int32_t>(key_cache.size(1));
  a.block_stride = key_cache.stride(0);
  a.page_stride = key_cache.stride(1);
  a.head_stride = key_cache.stride(2);
  const at::cuda::OptionalCUDAGuard device_guard(device_of(key));
  check_rc(b200pa_reshape_and_cache_flash(&a, at::cuda::getCurrentCUDAStream().stream()));
}

void convert_fp8(torch::Tensor& dst_cache, torch::Tensor& src_cache, const double scale,
                 const std::string& kv_cache_dtype) {
  TORCH_CHECK(src_cache.is_cuda(), "src must be on a GPU");
  TORCH_CHECK(dst_cache.is_cuda(), "dst must be on a GPU");
  TORCH_CHECK(src_cache.device() == dst_cache.device(), "src and dst must be on the same GPU");
  TORCH_CHECK(src_cache.is_contiguous() && dst_cache.is_contiguous() &&
                  src_cache.numel() == dst_cache.numel(),
              "convert_fp8 needs contiguous tensors of equal size");
  int kv;
  if (kv_cache_dtype == "auto" || kv_cache_dtype == "fp8" || kv_cache_dtype == "fp8_e4m3") {
    kv = B200PA_KV_FP8_E4M3;
  } else if (kv_cache_dtype == "fp8_e5m2") {
    kv = B200PA_KV_FP8_E5M2;
  } else {
    TORCH_CHECK(false, "Unsupported data type: ", kv_cache_dtype);
  }
  const bool to_fp8 = dst_cache.element_size() == 1;
  TORCH_CHECK(to_fp8 != (src_cache.element_size() == 1),
              "exactly one of src / dst must be a 1-byte (fp8) tensor");
  const int wide = dtype_code(to_fp8 ? src_cache.scalar_type() : dst_cache.scalar_type(), "convert_fp8");
  const at::cuda::OptionalCUDAGuard device_guard(src_cache.device());
  check_rc(b200pa_convert_fp8(dst_cache.data_ptr(), src_cache.data_ptr(), src_cache.numel(),
                              static_cast<float>(scale), wide, kv, to_fp8 ? 1 : 0,
                              at::cuda::getCurrentCUDAStream().stream()));
}

void merge_attn_states(torch::Tensor& output, std::optional<torch::Tensor> output_lse,
                       const torch::Tensor& prefix_output, const torch::Tensor& prefix_lse,
                       const torch::Tensor& suffix_output, const torch::Tensor& suffix_lse) {
  check_cuda(output, "output");
  TORCH_CHECK(output.dim() == 3, "output must be [num_tokens, num_heads, head_size]");
  const int dt = [&]() -> int {
    switch (output.scalar_type()) {
      case at::ScalarType::Float: return B200PA_F32;
      case at::ScalarType::Half: return B200PA_F16;
      case at::ScalarType::BFloat16: return B200PA_BF16;
      default: TORCH_CHECK(false, "Unsupported data type of O: ", output.scalar_type());
    }
    return -1;
  }();
  const int64_t head_size = output.size(2);
  TORCH_CHECK(output.stride(-2) == head_size && output.stride(-1) == 1,
              "output heads must be contiguous");
  TORCH_CHECK(prefix_output.stride(-2) == head_size && prefix_output.stride(-1) == 1,
              "prefix_output heads must be contiguous");
  TORCH_CHECK(suffix_output.stride(-2) == head_size && suffix_output.stride(-1) == 1,
              "suffix_output heads must be contiguous");
  TORCH_CHECK(output.is_contiguous() && prefix_output.is_contiguous() &&
                  suffix_output.is_contiguous() && prefix_lse.is_contiguous() &&
                  suffix_lse.is_contiguous(),
              "merge_attn_states needs contiguous tensors");
  TORCH_CHECK(prefix_output.scalar_type() == output.scalar_type() &&
                  suffix_output.scalar_type() == output.scalar_type(),
              "prefix/suffix/output dtypes differ");
  TORCH_CHECK(prefix_lse.scalar_type() == at::ScalarType::Float &&
                  suffix_lse.scalar_type() == at::ScalarType::Float,
              "lse tensors must be float32");
  float* olse = nullptr;
  if (output_lse.has_value()) {
    TORCH_CHECK(output_lse->scalar_type() == at::ScalarType::Float && output_lse->is_contiguous(),
                "output_lse must be a contiguous float32 tensor");
    olse = output_lse->data_ptr<float>();
  }
  const at::cuda::OptionalCUDAGuard device_guard(device_of(output));
  check_rc(b200pa_merge_attn_states(output.data_ptr(), olse, prefix_output.data_ptr(),
                                    prefix_lse.data_ptr<float>(), suffix_output.data_ptr(),
                                    suffix_lse.data_ptr<float>(), output.size(0),
                                    static_cast<int32_t>(output.size(1)),
                                    static_cast<int32_t>(head_size), dt,
                                    at::cuda::getCurrentCUDAStream().stream()));
}

void copy_blocks(std::vector<torch::Tensor> const& key_caches,
                 std::vector<torch::Tensor> const& value_caches,
                 const torch::Tensor& block_mapping) {
  const size_t num_layers = key_caches.size();
  TORCH_CHECK(num_layers == value_caches.size());
  if (num_layers == 0) return;
  TORCH_CHECK(key_caches[0].is_cuda());
  TORCH_CHECK(block_mapping.is_cuda() && block_mapping.scalar_type() == at::ScalarType::Long &&
                  block_mapping.is_contiguous() && block_mapping.dim() == 2 &&
                  block_mapping.size(1) == 2,
              "block_mapping must be a contiguous int64 CUDA tensor of shape [num_pairs, 2]");
  std::vector<void*> kp(num_layers), vp(num_layers);
  for (size_t i = 0; i < num_layers; ++i) {
    kp[i] = key_caches[i].data_ptr();
    vp[i] = value_caches[i].data_ptr();
  }
  const int64_t block_bytes = key_caches[0][0].numel() * key_caches[0].element_size();
  const at::cuda::OptionalCUDAGuard device_guard(key_caches[0].device());
  check_rc(b200pa_copy_blocks(kp.data(), vp.data(), static_cast<int32_t>(num_layers),
                              block_mapping.data_ptr<int64_t>(), block_mapping.size(0),
                              block_bytes, at::cuda::getCurrentCUDAStream().stream()));
}

void swap_blocks(torch::Tensor& src, torch::Tensor& dst, const torch::Tensor& block_mapping) {
  const bool sc = src.is_cuda(), dc = dst.is_cuda();
  if (sc && dc) {
    TORCH_CHECK(src.device() == dst.device(), "src and dst must be on the same GPU");
  } else {
    TORCH_CHECK((sc && dst.is_cpu()) || (src.is_cpu() && dc), "Invalid device combination");
  }
  TORCH_CHECK(block_mapping.device().is_cpu(), "block_mapping must be on CPU");
  TORCH_CHECK(block_mapping.scalar_type() == at::ScalarType::Long && block_mapping.dim() == 2 &&
                  block_mapping.size(1) == 2,
              "block_mapping must be an int64 tensor of shape [num_pairs, 2]");
  const torch::Tensor bm = block_mapping.contiguous();
  // the stride, not numel, so that padded blocks are copied whole (as the reference does)
  const int64_t block_bytes = src.element_size() * src.stride(0);
  const at::cuda::OptionalCUDAGuard device_guard(sc ? src.device() : dst.device());
  check_rc(b200pa_swap_blocks(src.data_ptr(), dst.data_ptr(), bm.data_ptr<int64_t>(), bm.size(0),
                              block_bytes, at::cuda::getCurrentCUDAStream().stream()));
}

constexpr const char* kMergeSchema =
    "merge_attn_states("
    "    Tensor! output,"
    "    Tensor!? output_lse,"
    "    Tensor prefix_output,"
    "    Tensor prefix_lse,"
    "    Tensor suffix_output,"
    "    Tensor suffix_lse) -> ()";
constexpr const char* kSwapSchema = "swap_blocks(Tensor src, Tensor! dst, Tensor block_mapping) -> ()";
constexpr const char* kCopySchema =
    "copy_blocks(Tensor(a!)[] key_caches, Tensor[](b!) value_caches, "
    "Tensor block_mapping) -> ()";
constexpr const char* kV1Schema =
    "paged_attention_v1("
    "    Tensor! out, Tensor query, Tensor key_cache,"
    "    Tensor value_cache, int num_kv_heads, float scale,"
    "    Tensor block_tables, Tensor seq_lens, int block_size,"
    "    int max_seq_len, Tensor? alibi_slopes,"
    "    str kv_cache_dtype, Tensor k_scale, Tensor v_scale,"
    "    int tp_rank, int blocksparse_local_blocks,"
    "    int blocksparse_vert_stride, int blocksparse_block_size,"
    "    int blocksparse_head_sliding_step) -> ()";
constexpr const char* kV2Schema =
    "paged_attention_v2("
    "    Tensor! out, Tensor! exp_sums, Tensor! max_logits,"
    "    Tensor! tmp_out, Tensor query, Tensor key_cache,"
    "    Tensor value_cache, int num_kv_heads, float scale,"
    "    Tensor block_tables, Tensor seq_lens, int block_size,"
    "    int max_seq_len, Tensor? alibi_slopes,"
    "    str kv_cache_dtype, Tensor k_scale, Tensor v_scale,"
    "    int tp_rank, int blocksparse_local_blocks,"
    "    int blocksparse_vert_stride, int blocksparse_block_size,"
    "    int blocksparse_head_sliding_step) -> ()";
constexpr const char* kReshapeSchema =
    "reshape_and_cache(Tensor key, Tensor value,"
    "                  Tensor! key_cache, Tensor! value_cache,"
    "                  Tensor slot_mapping,"
    "                  str kv_cache_dtype,"
    "                  Tensor k_scale, Tensor v_scale) -> ()";
constexpr const char* kReshapeFlashSchema =
    "reshape_and_cache_flash(Tensor key, Tensor value,"
    "                        Tensor! key_cache,"
    "                        Tensor! value_cache,"
    "                        Tensor slot_mapping,"
    "                        str kv_cache_dtype,"
    "                        Tensor k_scale, Tensor v_scale) -> ()";
constexpr const char* kConvertSchema =
    "convert_fp8(Tensor! dst_cache, Tensor src_cache, float scale, "
    "str kv_cache_dtype) -> ()";

bool op_exists(const char* qualified) {
  return c10::Dispatcher::singleton().findSchema({qualified, ""}).has_value();
}

}  // namespace

TORCH_LIBRARY(_C_b200, ops) {
  ops.def(kV1Schema);
  ops.impl("paged_attention_v1", torch::kCUDA, &paged_attention_v1);
  ops.def(kV2Schema);
  ops.impl("paged_attention_v2", torch::kCUDA, &paged_attention_v2);
  ops.def(kMergeSchema);
  ops.impl("merge_attn_states", torch::kCUDA, &merge_attn_states);
  ops.def(
      "paged_attention_with_lse(Tensor! out, Tensor! lse, Tensor query, Tensor key_cache,"
      " Tensor value_cache, int num_kv_heads, float scale, Tensor block_tables, Tensor seq_lens,"
      " int block_size, int max_seq_len, Tensor? alibi_slopes, str kv_cache_dtype,"
      " Tensor k_scale, Tensor v_scale) -> ()");
  ops.impl("paged_attention_with_lse", torch::kCUDA, &paged_attention_with_lse);
}

TORCH_LIBRARY(_C_b200_cache_ops, cache_ops) {
  cache_ops.def(kSwapSchema);
  cache_ops.impl("swap_blocks", torch::kCUDA, &swap_blocks);
  cache_ops.def(kCopySchema);
  cache_ops.impl("copy_blocks", torch::kCUDA, &copy_blocks);
  cache_ops.def(kReshapeSchema);
  cache_ops.impl("reshape_and_cache", torch::kCUDA, &reshape_and_cache);
  cache_ops.def(kReshapeFlashSchema);
  cache_ops.impl("reshape_and_cache_flash", torch::kCUDA, &reshape_and_cache_flash);
  cache_ops.def(kConvertSchema);
  cache_ops.impl("convert_fp8", torch::kCUDA, &convert_fp8);
}

// The reference's own operator names (_C / _C_cache_ops) are claimed on request only, never
// while this library loads: if they were defined here first, a vLLM `_C` extension imported
// afterwards would fail on the duplicate definitions.  A stand-alone user (the reference's
// own tests and benchmarks run without vLLM's extension) asks for them once with
// vllm_b200.claim_reference_names(); names that somebody has defined already are left alone.
// Returns how many names were claimed by this call, or -1 with `err` filled in.
extern "C" int b200_claim_reference_names(char* err, int err_len) {
  static std::vector<std::unique_ptr<torch::Library>> keep;  // registrations live as long as these
  try {
    int n = 0;
    auto ops = std::make_unique<torch::Library>(torch::Library::FRAGMENT, "_C", std::nullopt,
                                                __FILE__, __LINE__);
    auto cache_ops = std::make_unique<torch::Library>(torch::Library::FRAGMENT, "_C_cache_ops",
                                                      std::nullopt, __FILE__, __LINE__);
    if (!op_exists("_C::paged_attention_v1")) {
      ops->def(kV1Schema);
      ops->impl("paged_attention_v1", torch::kCUDA, &paged_attention_v1);
      ++n;
    }
    if (!op_exists("_C::paged_attention_v2")) {
      ops->def(kV2Schema);
      ops->impl("paged_attention_v2", torch::kCUDA, &paged_attention_v2);
      ++n;
    }
    if (!op_exists("_C::merge_attn_states")) {
      ops->def(kMergeSchema);
      ops->impl("merge_attn_states", torch::kCUDA, &merge_attn_states);
      ++n;
    }
    if (!op_exists("_C_cache_ops::reshape_and_cache")) {
      cache_ops->def(kReshapeSchema);
      cache_ops->impl("reshape_and_cache", torch::kCUDA, &reshape_and_cache);
      ++n;
    }
    if (!op_exists("_C_cache_ops::reshape_and_cache_flash")) {
      cache_ops->def(kReshapeFlashSchema);
      cache_ops->impl("reshape_and_cache_flash", torch::kCUDA, &reshape_and_cache_flash);
      ++n;
    }
    if (!op_exists("_C_cache_ops::swap_blocks")) {
      cache_ops->def(kSwapSchema);
      cache_ops->impl("swap_blocks", torch::kCUDA, &swap_blocks);
      ++n;
    }
    if (!op_exists("_C_cache_ops::copy_blocks")) {
      cache_ops->def(kCopySchema);
      cache_ops->impl("copy_blocks", torch::kCUDA, &copy_blocks);
      ++n;
    }
    if (!op_exists("_C_cache_ops::convert_fp8")) {
      cache_ops->def(kConvertSchema);
      cache_ops->impl("convert_fp8", torch::kCUDA, &convert_fp8);
      ++n;
    }
    keep.push_back(std::move(ops));
    keep.push_back(std::move(cache_ops));
    return n;
  } catch (const std::exception& e) {
    if (err != nullptr && err_len > 0) snprintf(err, size_t(err_len), "%s", e.what());
    return -1;
  }
}
