// Definitions of the reference's three decode dispatchers and of its GQA prefill dispatcher on top
// of the C ABI.
//
// The reference signatures carry neither the number of pages in the pool nor a workspace, so:
//  * block-table entries are bounds-checked against INT32_MAX only (the reference does not check
//    them at all, paged_attention_kernel.cuh:76);
//  * scratch comes from cudaMallocAsync / cudaFreeAsync on the caller's stream (stream-ordered,
//    served from the driver's pool after the first call).
#include <cstdio>
#include <climits>
#include <type_traits>

#include "kernels_api.h"
#include "cuda_llm_b200.h"

namespace {
template <typename T> constexpr int dtype_of() {
  return std::is_same<T, float>::value ? CUDA_LLM_F32 : std::is_same<T, __half>::value ? CUDA_LLM_F16 : CUDA_LLM_BF16;
}
void report(const char* who, int rc) {
  if (rc != CUDA_LLM_OK) fprintf(stderr, "%s: error %d: %s\n", who, rc, cuda_llm_last_cuda_error());
}
void* scratch(size_t bytes, cudaStream_t st) {
  void* p = nullptr;
  if (bytes == 0 || cudaMallocAsync(&p, bytes, st) != cudaSuccess) return nullptr;
  return p;
}
}  // namespace

template <typename T>
void dispatch_paged_attention(const T* query, const T* key_cache, const T* value_cache,
                              const int32_t* block_tables, const int32_t* context_lens, T* out,
                              int num_seqs, int num_heads, int head_dim, int max_blocks_per_seq,
                              float softmax_scale, cudaStream_t stream) {
  const int page = 16;  // the reference dispatcher instantiates PAGE_SIZE = 16 only (paged_attention_kernel.cuh:169-181)
  const size_t bytes = cuda_llm_dense_decode_workspace_bytes(num_seqs, num_heads, num_heads, head_dim,
                                                             max_blocks_per_seq * page);
  void* ws = scratch(bytes, stream);
  report("dispatch_paged_attention",
         cuda_llm_paged_attention(query, key_cache, value_cache, block_tables, context_lens, out, num_seqs,
                                  num_heads, num_heads, head_dim, page, max_blocks_per_seq, INT_MAX,
                                  softmax_scale, dtype_of<T>(), ws, bytes, stream));
  if (ws) cudaFreeAsync(ws, stream);
}

template <typename T>
void dispatch_async_flash_decode(const T* q, const T* k, const T* v, T* o, int batch_size,
                                 int num_heads, int seq_len, int head_dim, float softmax_scale,
                                 cudaStream_t stream) {
  const size_t bytes = cuda_llm_dense_decode_workspace_bytes(batch_size, num_heads, num_heads, head_dim, seq_len);
  void* ws = scratch(bytes, stream);
  report("dispatch_async_flash_decode",
         cuda_llm_flash_decode(q, k, v, o, batch_size, num_heads, num_heads, seq_len, head_dim, softmax_scale,
                               dtype_of<T>(), ws, bytes, stream));
  if (ws) cudaFreeAsync(ws, stream);
}

template <typename T>
void dispatch_fused_gqa(const T* q, const T* k, const T* v, T* o, int batch_size, int num_q_heads,
                        int num_kv_heads, int seq_len, int head_dim, float softmax_scale, bool is_causal,
                        cudaStream_t stream) {
  report("dispatch_fused_gqa",
         cuda_llm_gqa_prefill(q, k, v, o, batch_size, num_q_heads, num_kv_heads, seq_len, head_dim, softmax_scale,
                              is_causal ? 1 : 0, dtype_of<T>(), nullptr, stream));
}

template <typename T_OUT, typename T_Q>
void dispatch_fp8_paged_attention(const T_Q* query, const int8_t* key_cache_fp8,
                                  const int8_t* value_cache_fp8, const float* k_scale,
                                  const float* v_scale, const int32_t* block_tables,
                                  const int32_t* context_lens, T_OUT* out, int num_seqs,
                                  int num_heads, int head_dim, int max_blocks_per_seq, int page_size,
                                  float softmax_scale, bool per_block_scales, cudaStream_t stream) {
  CudaLlmPagedDecodeParams p = {};
  p.query = query;
  p.key_cache = key_cache_fp8;
  p.value_cache = value_cache_fp8;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.out = out;
  p.num_seqs = num_seqs;
  p.num_q_heads = p.num_kv_heads = num_heads;  // the reference path is MHA
  p.head_dim = head_dim;
  p.page_size = page_size;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.num_blocks = INT_MAX;
  p.max_q_len = 1;
  p.q_dtype = dtype_of<T_Q>();
  p.out_dtype = dtype_of<T_OUT>();
  p.k_format = p.v_format = CUDA_LLM_KV_FP8_E4M3;
  p.scale_mode = per_block_scales ? CUDA_LLM_SCALE_PER_BLOCK : CUDA_LLM_SCALE_PER_HEAD;
  p.softmax_scale = softmax_scale;
  p.workspace_bytes = cuda_llm_paged_decode_workspace_bytes(num_seqs, num_heads, num_heads, head_dim, page_size, 1, 0);
  p.workspace = scratch(p.workspace_bytes, stream);
  int rc = p.workspace ? cuda_llm_workspace_init(p.workspace, 256, stream) : CUDA_LLM_EWORKSPACE;
  if (rc == CUDA_LLM_OK) rc = cuda_llm_paged_decode(&p, stream);
  report("dispatch_fp8_paged_attention", rc);
  if (p.workspace) cudaFreeAsync(p.workspace, stream);
}

template <typename T_OUT>
void dispatch_fused_microscaled_attention(const int8_t* q, const float* q_scale, const int8_t* k,
                                          const float* k_scale, const int8_t* v, const float* v_scale, T_OUT* out,
                                          int batch_size, int num_heads, int seq_len, int head_dim,
                                          float softmax_scale, bool is_causal, cudaStream_t stream) {
  const size_t bytes = cuda_llm_mx_attention_workspace_bytes(batch_size, num_heads, num_heads, seq_len, head_dim);
  void* ws = scratch(bytes, stream);
  report("dispatch_fused_microscaled_attention",
         cuda_llm_mx_attention_ws(q, q_scale, k, k_scale, v, v_scale, out, batch_size, num_heads, num_heads, seq_len,
                                  head_dim, softmax_scale, is_causal ? 1 : 0, dtype_of<T_OUT>(), ws, ws ? bytes : 0, stream));
  if (ws) cudaFreeAsync(ws, stream);
}

#define INSTANTIATE(T)                                                                                        \
  template void dispatch_paged_attention<T>(const T*, const T*, const T*, const int32_t*, const int32_t*, T*, \
                                            int, int, int, int, float, cudaStream_t);                         \
  template void dispatch_async_flash_decode<T>(const T*, const T*, const T*, T*, int, int, int, int, float,   \
                                               cudaStream_t);                                                 \
  template void dispatch_fused_gqa<T>(const T*, const T*, const T*, T*, int, int, int, int, int, float, bool,           \
                                      cudaStream_t);                                                          \
  template void dispatch_fused_microscaled_attention<T>(const int8_t*, const float*, const int8_t*, const float*,   \
                                                        const int8_t*, const float*, T*, int, int, int, int, float, \
                                                        bool, cudaStream_t);                                        \
  template void dispatch_fp8_paged_attention<T, T>(const T*, const int8_t*, const int8_t*, const float*,      \
                                                   const float*, const int32_t*, const int32_t*, T*, int, int, \
                                                   int, int, int, float, bool, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(__half)
INSTANTIATE(__nv_bfloat16)
