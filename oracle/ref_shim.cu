// TEST INFRASTRUCTURE.  C entry points around the REFERENCE's own paged decode dispatchers, compiled
// from the reference's sources where they lie (see oracle/Makefile); nothing of the reference is
// copied into this repository.  Used to check the unquantised path against the real reference
// kernel and to time the reference kernels on the same GPU.
#include "paged_attention_kernel.cuh"      // reference: paged_attention_kernel.cuh:20-182
#include "fp8_paged_attention_kernel.cuh"  // reference: fp8_paged_attention_kernel.cuh:24-191

extern "C" {

// dtype: 0 fp32, 1 fp16, 2 bf16
int ref_paged_attention(const void* q, const void* kc, const void* vc, const int32_t* bt, const int32_t* ctx,
                        void* out, int num_seqs, int num_heads, int head_dim, int max_blocks, float scale,
                        int dtype, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0)
    dispatch_paged_attention<float>((const float*)q, (const float*)kc, (const float*)vc, bt, ctx, (float*)out,
                                    num_seqs, num_heads, head_dim, max_blocks, scale, st);
  else if (dtype == 1)
    dispatch_paged_attention<__half>((const __half*)q, (const __half*)kc, (const __half*)vc, bt, ctx, (__half*)out,
                                     num_seqs, num_heads, head_dim, max_blocks, scale, st);
  else
    dispatch_paged_attention<__nv_bfloat16>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                            (const __nv_bfloat16*)vc, bt, ctx, (__nv_bfloat16*)out, num_seqs,
                                            num_heads, head_dim, max_blocks, scale, st);
  return (int)cudaGetLastError();
}

// the reference's 8-bit kernel (bytes read as int8, fp8_paged_attention_kernel.cuh:102,135); fp16 query/out
int ref_int8_paged_attention(const void* q, const void* kc, const void* vc, const float* ks, const float* vs,
                             const int32_t* bt, const int32_t* ctx, void* out, int num_seqs, int num_heads,
                             int head_dim, int max_blocks, float scale, int per_block, void* stream) {
  dispatch_fp8_paged_attention<__half, __half>((const __half*)q, (const int8_t*)kc, (const int8_t*)vc, ks, vs, bt,
                                               ctx, (__half*)out, num_seqs, num_heads, head_dim, max_blocks, 16,
                                               scale, per_block != 0, reinterpret_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}
}
