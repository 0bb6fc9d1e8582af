// Whole-page dequantisation to fp32 with the same conversion instructions the decode kernel
// uses; lets the tests check E4M3 / E2M1 / E8M0 decoding and block-table gathering bit for bit.
#include "paged_decode_kernel.cuh"

namespace b200 {

__global__ void dequant_pages_kernel(const uint8_t* __restrict__ cache, const uint8_t* __restrict__ scale,
                                     const int32_t* __restrict__ pages, int n_pages, int Hkv, int D,
                                     int page, int format, int scale_mode, float* __restrict__ out) {
  const long long total = (long long)n_pages * Hkv * D * page;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int tok = (int)(idx % page);
    const int d = (int)((idx / page) % D);
    const int h = (int)((idx / ((long long)page * D)) % Hkv);
    const int n = (int)(idx / ((long long)page * D * Hkv));
    const long long b = pages[n];
    float v;
    if (format == CUDA_LLM_KV_FP4_E2M1) {
      const uint8_t byte = cache[((b * Hkv + h) * (D / 2) + d / 2) * page + tok];
      // same bit placement as the decode kernel: s.ee.m at f16 bits 15, 11..9 is value * 2^-14
      const uint32_t nib = (d & 1) ? (byte >> 4) : (byte & 0xF);
      const unsigned short hb = (unsigned short)(((nib & 8u) << 12) | ((nib & 7u) << 9));
      v = __half2float(__ushort_as_half(hb)) * 16384.f;
    } else {
      const uint8_t byte = cache[((b * Hkv + h) * D + d) * page + tok];
      const uint32_t h2 = e4m3x2_to_f16x2_lo(byte);
      const __half2 hh = *reinterpret_cast<const __half2*>(&h2);
      v = __low2float(hh);
    }
    float s = 1.f;
    if (scale_mode == CUDA_LLM_SCALE_PER_HEAD) s = reinterpret_cast<const float*>(scale)[h];
    else if (scale_mode == CUDA_LLM_SCALE_PER_BLOCK) s = reinterpret_cast<const float*>(scale)[b * Hkv + h];
    else if (scale_mode == CUDA_LLM_SCALE_PER_TOKEN) s = reinterpret_cast<const float*>(scale)[(b * Hkv + h) * page + tok];
    else if (scale_mode == CUDA_LLM_SCALE_MX_E8M0) s = e8m0_to_f32(scale[((b * Hkv + h) * (D / 32) + d / 32) * page + tok]);
    out[idx] = __fmul_rn(v, s);
  }
}

cudaError_t launch_dequant_pages(const void* cache, const void* scale, const int32_t* pages, int n_pages,
                                 int Hkv, int D, int page, int format, int scale_mode, float* out,
                                 cudaStream_t st) {
  const long long total = (long long)n_pages * Hkv * D * page;
  if (total == 0) return cudaSuccess;
  const int grid = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  dequant_pages_kernel<<<grid, 256, 0, st>>>((const uint8_t*)cache, (const uint8_t*)scale, pages, n_pages,
                                             Hkv, D, page, format, scale_mode, out);
  return cudaGetLastError();
}

}  // namespace b200
