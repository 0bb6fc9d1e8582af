#pragma once
// Host-side C++ entry points of the decode path and of the prefill that fills its cache, with the
// exact signatures the reference declares for them (kernels_api.h:35-41, 52-56, 58-62, 94-101, 103-108 in
// the reference project), so that the reference's
// PyTorch binding (fused_softmax_binding.cpp) links against libcuda_llm_b200.so unchanged.  They are
// explicitly instantiated for float, __half and __nv_bfloat16 as in the reference
// (paged_attention_instantiations.cu, fused_gqa_instantiations.cu,
// async_flash_decode_instantiations.cu, fp8_paged_attention_instantiations.cu).  No default arguments: the caller always passes the stream.
//
// Differences in behaviour, all on the side of saying more: the 8-bit cache bytes are E4M3 codes;
// page sizes 32 and 64 work; an unsupported shape or a CUDA error is reported on stderr instead of
// silently launching nothing (the signatures return void, as the reference's do).  Scratch memory
// for split partials comes from cudaMallocAsync on the caller's stream.
#include <cstdint>
#include <cuda_runtime_api.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

template <typename T>
void dispatch_paged_attention(const T* query, const T* key_cache, const T* value_cache,
                              const int32_t* block_tables, const int32_t* context_lens, T* out,
                              int num_seqs, int num_heads, int head_dim, int max_blocks_per_seq,
                              float softmax_scale, cudaStream_t stream);

template <typename T>
void dispatch_fused_gqa(const T* q, const T* k, const T* v, T* o, int batch_size, int num_q_heads,
                        int num_kv_heads, int seq_len, int head_dim, float softmax_scale,
                        bool is_causal, cudaStream_t stream);

template <typename T>
void dispatch_async_flash_decode(const T* q, const T* k, const T* v, T* o, int batch_size,
                                 int num_heads, int seq_len, int head_dim, float softmax_scale,
                                 cudaStream_t stream);

template <typename T_OUT, typename T_Q>
void dispatch_fp8_paged_attention(const T_Q* query, const int8_t* key_cache_fp8,
                                  const int8_t* value_cache_fp8, const float* k_scale,
                                  const float* v_scale, const int32_t* block_tables,
                                  const int32_t* context_lens, T_OUT* out, int num_seqs,
                                  int num_heads, int head_dim, int max_blocks_per_seq, int page_size,
                                  float softmax_scale, bool per_block_scales, cudaStream_t stream);

// Declared by the reference (kernels_api.h:103-108) without a definition; here: E4M3 codes with one
// fp32 scale per 32 elements of head_dim, scales laid out [batch, heads, seq_len, head_dim / 32].
template <typename T_OUT>
void dispatch_fused_microscaled_attention(const int8_t* q, const float* q_scale, const int8_t* k,
                                          const float* k_scale, const int8_t* v, const float* v_scale,
                                          T_OUT* out, int batch_size, int num_heads, int seq_len,
                                          int head_dim, float softmax_scale, bool is_causal,
                                          cudaStream_t stream);
