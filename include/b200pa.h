/*
 * b200pa.h — C ABI of the B200-native PagedAttention decode path.
 *
 * One shared library (libb200pa.so) exports the functions declared here.  They
 * are the drop-in boundary for four operators of the reference project (vLLM):
 *
 *   torch.ops._C.paged_attention_v1            csrc/torch_bindings.cpp:52-63
 *   torch.ops._C.paged_attention_v2            csrc/torch_bindings.cpp:65-77
 *   torch.ops._C_cache_ops.reshape_and_cache   csrc/torch_bindings.cpp:687-694
 *   torch.ops._C_cache_ops.reshape_and_cache_flash          ... :696-705
 *   torch.ops._C_cache_ops.convert_fp8         csrc/torch_bindings.cpp:716-719
 * and, next to that path, torch.ops._C.merge_attn_states (csrc/torch_bindings.cpp:83-90),
 * torch.ops._C_cache_ops.copy_blocks / swap_blocks (csrc/torch_bindings.cpp:672-685).
 *
 * Conventions
 *   - Plain C: raw device pointers, sizes and element strides; no framework
 *     types.  `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  The current CUDA device must be the one that owns the pointers.
 *   - Every function returns 0 on success or a negative B200PA_E* code; it never
 *     throws and never aborts.  b200pa_last_error() returns a thread-local,
 *     human-readable message for the last non-zero return on this thread.
 *   - Like the reference ops they replace, the launchers do not synchronise, do
 *     not allocate device memory and do not read device data on the host, so
 *     those ops may be recorded into a CUDA graph as the reference's are.
 *   - No bounds checks on block-table or slot indices (same contract as the
 *     reference kernels, csrc/attention/attention_kernels.cuh:252-253).
 *   - All strides are in ELEMENTS of the tensor they describe.
 */
#ifndef B200PA_H_
#define B200PA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200PA_VERSION 2

/* Error codes (negative). */
#define B200PA_OK 0
#define B200PA_EINVAL (-1)      /* bad argument (null pointer, bad size, bad stride)     */
#define B200PA_EUNSUPPORTED (-2)/* head size / block size / dtype combination not built  */
#define B200PA_ECUDA (-3)       /* a CUDA runtime call failed at launch time             */
#define B200PA_EDEVICE (-4)     /* a kernel reported a bounded wait that ran out         */

/* Element type of query / out / key / value (the reference dispatches on
 * at::ScalarType Float / Half / BFloat16, quant_utils.cuh:545-593). */
typedef enum b200pa_dtype {
  B200PA_F32 = 0,
  B200PA_F16 = 1,
  B200PA_BF16 = 2
} b200pa_dtype;

/* Storage type of the paged KV cache; the reference passes this as the string
 * kv_cache_dtype ("auto" | "fp8" | "fp8_e4m3" | "fp8_e5m2" | "fp8_ds_mla"). */
typedef enum b200pa_kv_dtype {
  B200PA_KV_AUTO = 0,     /* cache holds the same 16/32-bit type as query/key */
  B200PA_KV_FP8_E4M3 = 1, /* 1 byte per element, OCP e4m3fn                   */
  B200PA_KV_FP8_E5M2 = 2  /* 1 byte per element, e5m2                         */
} b200pa_kv_dtype;

/* Maps the reference's kv_cache_dtype string to b200pa_kv_dtype
 * (DISPATCH_BY_KV_CACHE_DTYPE, quant_utils.cuh:545-593); -1 if unknown. */
int b200pa_kv_dtype_from_string(const char* kv_cache_dtype);

/*
 * Arguments of paged_attention_v1 / paged_attention_v2.
 * Replaces: csrc/ops.h:32-53, launchers csrc/attention/paged_attention_v1.cu:43-125
 * and paged_attention_v2.cu:43-131.
 *
 * Layouts (x = 16 / sizeof(cache element)):
 *   out          [num_seqs, num_heads, head_size]               contiguous
 *   query        [num_seqs, num_heads, head_size]               row stride q_stride
 *   key_cache    [num_blocks, num_kv_heads, head_size/x, block_size, x]
 *   value_cache  [num_blocks, num_kv_heads, head_size, block_size]
 *                block stride kv_block_stride, head stride kv_head_stride
 *                (K's strides address V too, as in the reference)
 *   block_tables [num_seqs, max_num_blocks_per_seq] int32
 *   seq_lens     [num_seqs] int32
 *   alibi_slopes [num_heads] float32 or NULL
 *   k_scale, v_scale : device pointers to ONE float each (may be NULL when
 *                kv_dtype == B200PA_KV_AUTO)
 * v2 scratch, owned by the caller, contents unspecified after the call (the library lays its
 * partial results out in it as it sees fit):
 *   exp_sums, max_logits [num_seqs, num_heads, max_num_partitions] float32
 *   tmp_out              [num_seqs, num_heads, max_num_partitions, head_size] (query dtype)
 *   max_num_partitions = ceil(max_seq_len / 512)
 */
typedef struct b200pa_attn_args {
  void* out;
  const void* query;
  const void* key_cache;
  const void* value_cache;
  const int32_t* block_tables;
  const int32_t* seq_lens;
  const float* alibi_slopes;
  const float* k_scale;
  const float* v_scale;
  float* exp_sums;
  float* max_logits;
  void* tmp_out;

  int64_t q_stride;
  int64_t kv_block_stride;
  int64_t kv_head_stride;

  int32_t num_seqs;
  int32_t num_heads;
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t block_size;
  int32_t max_seq_len;
  int32_t max_num_blocks_per_seq;
  int32_t max_num_partitions; /* v2 only; ignored by v1 */

  float scale;
  int32_t q_dtype;  /* b200pa_dtype    */
  int32_t kv_dtype; /* b200pa_kv_dtype */

  /* Block-sparse arguments of the reference signature
   * (attention_kernels.cuh:187-262): blocksparse_vert_stride <= 1 is dense
   * attention; larger values keep the last blocksparse_local_blocks sparse
   * blocks plus every vert_stride-th one (shifted per head by
   * head_sliding_step).  The sparse case runs on the generic kernel. */
  int32_t tp_rank;
  int32_t blocksparse_local_blocks;
  int32_t blocksparse_vert_stride;
  int32_t blocksparse_block_size;
  int32_t blocksparse_head_sliding_step;

  /* Optional extra output, NULL in the reference's calls (its ops have no such
   * argument): out_lse[head * num_seqs + seq] = natural log of the sum over the
   * sequence's tokens of exp(scaled logit + ALiBi bias), float32, -inf for an empty
   * sequence.  Layout [num_heads, num_seqs] as merge_attn_states takes it
   * (csrc/attention/merge_attn_states.cu:14-30), so that attention over disjoint
   * token ranges of a sequence - on one GPU or one range per rank - can be combined
   * with b200pa_merge_attn_states. */
  float* out_lse;
} b200pa_attn_args;

/* Replaces paged_attention_v1 (csrc/attention/paged_attention_v1.cu:160-182).  No scratch
 * argument, as in the reference; sequences are nevertheless cut into pieces that different
 * warps process (by equal numbers of cache blocks, from the real lengths), with the partial
 * results kept in a workspace inside the library (60 MiB per GPU that loads it) and merged in
 * the same launch.  Calls may overlap on the GPU like the reference's: every stream gets its
 * own part of that workspace - 32 MiB for the first stream used on a device, 4 MiB for each of
 * up to seven more (a least-recently-used slot is reassigned after that; more than eight
 * streams calling concurrently are not kept apart).  A batch whose partials do not fit its
 * stream's part is cut more coarsely, or not at all.  A kernel node captured into a CUDA graph
 * keeps the workspace part of the stream it was captured on. */
int b200pa_paged_attention_v1(const b200pa_attn_args* args, void* stream);

/* Replaces paged_attention_v2 + its reduce kernel
 * (csrc/attention/paged_attention_v2.cu:167-192, attention_kernels.cuh:559-664):
 * split-KV with the partial results in the caller's scratch, merged inside the same kernel.
 * The scratch is used as max_num_partitions slots per (sequence, head); which tokens a slot
 * covers is decided in the kernel (equal numbers of cache blocks per warp), not fixed at 512.
 * Few, long sequences need more slots per sequence than ceil(max_seq_len / 512) to occupy the
 * GPU; such calls keep their partials in the workspace described at b200pa_paged_attention_v1
 * instead and leave the caller's scratch untouched. */
int b200pa_paged_attention_v2(const b200pa_attn_args* args, void* stream);

/*
 * paged_attention_v2 for callers that cannot hand over scratch memory.  It has no
 * counterpart in the reference, whose caller always allocates exp_sums,
 * max_logits and tmp_out (vllm/attention/ops/paged_attn.py:164-174).
 *
 * Who needs it: a host that binds this C ABI directly and owns no device
 * allocator, and serving processes that gave all free HBM to the KV-cache pool
 * at start-up, where a later cudaMalloc can fail.  This entry point allocates
 * nothing (no cudaMalloc / cudaFree, no allocating library call): the split-KV
 * scratch is a 32 MiB array built into the library, resident on every GPU that
 * loads it until the process exits (in addition to the 60 MiB workspace of
 * b200pa_paged_attention_v1, which this entry point does not use).
 *
 *   - args->exp_sums, max_logits, tmp_out and max_num_partitions are ignored
 *     (may be NULL / 0); everything else is as for b200pa_paged_attention_v2.
 *   - Limit: num_seqs * num_heads * ceil(max_seq_len/512) * (8 + head_size *
 *     sizeof(query element)) bytes, each of the three regions rounded up to
 *     256 bytes, must fit 32 MiB; larger problems return B200PA_EINVAL with a
 *     message and launch nothing.  Room that a smaller problem leaves is used for
 *     more partial slots per sequence.
 *   - The first call on a device resolves the array's device address; make that
 *     call before any stream capture.
 *   - All calls on one device share the array.  Calls that may overlap on the
 *     GPU (different streams without an ordering between them) race on it; keep
 *     them on one stream or order them with events.  Nothing in the array has
 *     to be cleared between calls.
 */
int b200pa_paged_attention_v2_noalloc(const b200pa_attn_args* args, void* stream);

/*
 * Arguments of reshape_and_cache / reshape_and_cache_flash.
 * Replaces: csrc/cache.h:21-32, launchers csrc/cache_kernels.cu:656-683 and :700-738.
 *
 *   key, value   [num_tokens, num_heads, head_size]  row strides key_stride/value_stride
 *   slot_mapping [num_tokens] int64; slot < 0 = padded token, skipped
 * reshape_and_cache ("x-layout", contiguous caches):
 *   key_cache    [num_blocks, num_heads, head_size/x, block_size, x]
 *   value_cache  [num_blocks, num_heads, head_size, block_size]
 *   (x is given explicitly, as the reference reads it from key_cache.size(4))
 * reshape_and_cache_flash (strided caches, NHD or HND):
 *   key_cache/value_cache viewed as [num_blocks, block_size, num_heads, head_size]
 *   with element strides (block_stride, page_stride, head_stride).
 * fp8: bits = cvt_rn_satfinite(float(v) / scale) with IEEE division
 *   (quant_utils.cuh:469-502).
 */
typedef struct b200pa_cache_args {
  const void* key;
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;
  const float* k_scale;
  const float* v_scale;

  int64_t key_stride;
  int64_t value_stride;
  int64_t block_stride; /* flash only */
  int64_t page_stride;  /* flash only */
  int64_t head_stride;  /* flash only */

  int32_t num_tokens;
  int32_t num_heads;
  int32_t head_size;
  int32_t block_size;
  int32_t x;        /* x-layout only */
  int32_t in_dtype; /* b200pa_dtype    */
  int32_t kv_dtype; /* b200pa_kv_dtype */
} b200pa_cache_args;

int b200pa_reshape_and_cache(const b200pa_cache_args* args, void* stream);
int b200pa_reshape_and_cache_flash(const b200pa_cache_args* args, void* stream);

/*
 * Replaces convert_fp8 (csrc/cache_kernels.cu:826-899): elementwise
 * quantise (src 16/32-bit -> dst fp8) or dequantise (src fp8 -> dst 16/32-bit)
 * of `numel` contiguous elements with a host-side scalar scale.
 * wide_dtype is the b200pa_dtype of the non-fp8 side; kv_dtype selects e4m3/e5m2.
 * to_fp8 != 0: dst is fp8.
 */
int b200pa_convert_fp8(void* dst, const void* src, int64_t numel, float scale,
                       int32_t wide_dtype, int32_t kv_dtype, int32_t to_fp8,
                       void* stream);

/*
 * Replaces merge_attn_states (csrc/attention/merge_attn_states.cu:14-212, schema
 * csrc/torch_bindings.cpp:83-90): merges two partial attention results with their
 * log-sum-exp,
 *   out = (prefix * e^(p_lse-m) + suffix * e^(s_lse-m)) / (e^(p_lse-m) + e^(s_lse-m)),
 *   out_lse = log(sum) + m,  m = max(p_lse, s_lse);  infinite LSEs count as -inf and
 *   if both are, prefix_output is passed through.
 * output / prefix_output / suffix_output: [num_tokens, num_heads, head_size] contiguous,
 * 16-byte aligned, of `dtype` (b200pa_dtype); *_lse: [num_heads, num_tokens] float32;
 * output_lse may be NULL.  head_size must be a multiple of 16 / sizeof(element).
 */
int b200pa_merge_attn_states(void* output, float* output_lse, const void* prefix_output,
                             const float* prefix_lse, const void* suffix_output,
                             const float* suffix_lse, int64_t num_tokens, int32_t num_heads,
                             int32_t head_size, int32_t dtype, void* stream);

/*
 * Replaces copy_blocks (csrc/cache_kernels.cu:73-171): for every layer l and every
 * pair (src, dst) in block_mapping, copies block src to block dst inside
 * key_caches[l] and inside value_caches[l].  key_caches / value_caches are HOST
 * arrays of num_layers device pointers; block_mapping is a DEVICE array of
 * num_pairs (src, dst) int64 pairs; block_bytes is the size of one block of one
 * cache in bytes.  The pointers are passed to the kernel as parameters: no device
 * allocation, no host-device copy, no synchronisation.
 */
int b200pa_copy_blocks(void* const* key_caches, void* const* value_caches, int32_t num_layers,
                       const int64_t* block_mapping, int64_t num_pairs, int64_t block_bytes,
                       void* stream);

/*
 * Replaces swap_blocks (csrc/cache_kernels.cu:26-69): copies block src -> dst for
 * every (src, dst) int64 pair of the HOST array block_mapping_host, between two
 * caches that may live on the host or on the current device (one asynchronous copy
 * per block on `stream`; pinned host memory is needed for true asynchrony).
 */
int b200pa_swap_blocks(const void* src, void* dst, const int64_t* block_mapping_host,
                       int64_t num_pairs, int64_t block_bytes, void* stream);

/* Thread-local message for the last non-zero return on this thread ("" if none). */
const char* b200pa_last_error(void);

/* B200PA_VERSION of the loaded library. */
int b200pa_version(void);

/*
 * Reads (and clears) the device-side status word of the current device.  The
 * kernels' mbarrier waits are bounded; a wait that runs out records a code here
 * and the warp returns instead of spinning.  Codes: 0 healthy, 1 a wait ran out,
 * 2 a warp was handed work without shared-memory ring slots, 3 a warp owed more
 * split-KV merges than it can note down (2 and 3 guard invariants of the work
 * distribution and are not expected to occur).  This call synchronises the
 * device; it is meant for tests and debugging, never for the hot path.
 * Returns 0 and stores the word in *status.
 */
int b200pa_device_status(int32_t* status);

/*
 * Puts the library's device-side bookkeeping of the current device back to its initial state:
 * the work-distribution words and split-KV arrival counters of the decode kernel (which every
 * healthy launch leaves zeroed by itself) and the status word.  Only needed after a launch
 * reported a non-zero status, whose warps may have left early; enqueued on `stream`, which
 * must be ordered after every attention call still in flight.  No counterpart in the reference.
 */
int b200pa_reset_device_state(void* stream);

/* Number of kernel launches issued by this library on the calling thread since
 * the last call with reset != 0 (host-side counter, for benchmark bookkeeping). */
int64_t b200pa_launch_count(int reset);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* B200PA_H_ */
