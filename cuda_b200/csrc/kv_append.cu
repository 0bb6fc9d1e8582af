// Writes new K/V tokens into the paged, quantised cache: the step that precedes the decode path.
// The reference has no such kernel (its tests quantise with torch on the host,
// tests/test_kernels_misc.py:51-55, and page with make_paged_cache, tests/_utils.py:107-133); this
// one reproduces that recipe bit for bit on the device:
//   per-token fp32 scale : scale = max(amax / 448, 1e-8); code = E4M3(x / scale), round to nearest even
//   E8M0 block scale     : e = floor(log2(amax_block)) - emax (8 for E4M3, 2 for E2M1), code = x / 2^e
//   per-head fp32 scale  : the given scale is used, code = E4M3(x / scale)
// One warp per (token, KV head); lanes split head_dim; codes go to cache[block][head][d][offset].
#include "paged_decode_kernel.cuh"

namespace b200 {

struct AppendArgs {
  const void* k_new;  // [n, Hkv, D]
  const void* v_new;
  const int32_t* slot_block;
  const int32_t* slot_offset;
  uint8_t* kc;
  uint8_t* vc;
  void* ks;
  void* vs;
  uint32_t* status;  // may be null
  int n, Hkv, page, num_blocks, in_dtype, v_format, scale_mode;
  int seq_len;  // 0: source rows are [n, Hkv, D]; > 0: source is [n / seq_len, Hkv, seq_len, D] (prefill layout)
};

__device__ __forceinline__ uint32_t quant_e4m3_byte(float y) { return f32x2_to_e4m3x2(y, 0.f) & 0xffu; }

// round to nearest E2M1 code, ties to the even code, saturating at 6
__device__ __forceinline__ uint32_t quant_e2m1_nibble(float y) {
  const float m = fabsf(y);
  uint32_t c = 0;
  c = m > 0.25f ? 1u : c;
  c = m >= 0.75f ? 2u : c;
  c = m > 1.25f ? 3u : c;
  c = m >= 1.75f ? 4u : c;
  c = m > 2.5f ? 5u : c;
  c = m >= 3.5f ? 6u : c;
  c = m > 5.0f ? 7u : c;
  return c | ((__float_as_uint(y) >> 31) << 3);
}

template <int D>
__global__ void __launch_bounds__(128) kv_append_kernel(const AppendArgs a) {
  constexpr int E = D / 32;  // elements per lane: lane owns d = lane*E .. lane*E+E-1 (E = 2 or 4)
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= 2LL * a.n * a.Hkv) return;
  const int is_v = (int)(item & 1);
  const int h = (int)((item >> 1) % a.Hkv);
  const int tok = (int)((item >> 1) / a.Hkv);
  const int blk = a.slot_block[tok], off = a.slot_offset[tok];
  if (blk < 0 || blk >= a.num_blocks || off < 0 || off >= a.page) {
    if (a.status && lane == 0) atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
    return;
  }
  const void* src = is_v ? a.v_new : a.k_new;
  float x[E];
  const size_t src_row = a.seq_len > 0 ? ((size_t)(tok / a.seq_len) * a.Hkv + h) * a.seq_len + (tok % a.seq_len)
                                       : (size_t)tok * a.Hkv + h;
#pragma unroll
  for (int e = 0; e < E; ++e) x[e] = load_q_elem(src, a.in_dtype, src_row * D + lane * E + e);
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) amax = fmaxf(amax, fabsf(x[e]));
  const bool fp4 = is_v && a.v_format == CUDA_LLM_KV_FP4_E2M1;
  uint8_t* cache = is_v ? a.vc : a.kc;
  void* scale = is_v ? a.vs : a.ks;
  if (a.scale_mode == CUDA_LLM_SCALE_MX_E8M0) {
    // a 32-element block = 32/E consecutive lanes
#pragma unroll
    for (int o = 1; o < 32 / E; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 7.888609052210118e-31f);  // 2^-100, as the host recipe clamps
    const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2(amax))
    const int eb = min(254, max(0, ef - (fp4 ? 2 : 8) + 127));
    const float inv = __uint_as_float((uint32_t)(254 - eb) << 23);      // 2^-(eb-127); eb in [0,254] -> exact except eb=254
    const int b = (lane * E) / 32;
    if ((lane * E) % 32 == 0)
      reinterpret_cast<uint8_t*>(scale)[(((size_t)blk * a.Hkv + h) * (D / 32) + b) * a.page + off] = (uint8_t)eb;
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = (eb == 0) ? x[e] * 1.7014118346046923e38f : x[e] * inv;
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc;
    if (a.scale_mode == CUDA_LLM_SCALE_PER_TOKEN) {
      sc = fmaxf(__fdiv_rn(amax, 448.f), 1e-8f);
      if (lane == 0) reinterpret_cast<float*>(scale)[((size_t)blk * a.Hkv + h) * a.page + off] = sc;
    } else if (a.scale_mode == CUDA_LLM_SCALE_PER_BLOCK) {
      sc = reinterpret_cast<const float*>(scale)[(size_t)blk * a.Hkv + h];
    } else {
      sc = reinterpret_cast<const float*>(scale)[h];
    }
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = __fdiv_rn(x[e], sc);
  }
  if (!fp4) {
    uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * D + lane * E) * a.page + off;
#pragma unroll
    for (int e = 0; e < E; ++e) dst[(size_t)e * a.page] = (uint8_t)quant_e4m3_byte(x[e]);
  } else {
    uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * (D / 2) + lane * (E / 2)) * a.page + off;
#pragma unroll
    for (int e = 0; e < E; e += 2)
      dst[(size_t)(e / 2) * a.page] = (uint8_t)(quant_e2m1_nibble(x[e]) | (quant_e2m1_nibble(x[e + 1]) << 4));
  }
}

cudaError_t launch_kv_append(const AppendArgs& a, int D, cudaStream_t st) {
  const long long items = 2LL * a.n * a.Hkv;
  if (items == 0) return cudaSuccess;
  const int grid = (int)((items + 3) / 4);
  if (D == 64) kv_append_kernel<64><<<grid, 128, 0, st>>>(a);
  else kv_append_kernel<128><<<grid, 128, 0, st>>>(a);
  return cudaGetLastError();
}

cudaError_t run_kv_append_prefill(const void* k, const void* v, const CudaLlmKvCacheTarget& c, int B, int Hkv, int S,
                                  int D, int in_dtype, cudaStream_t st) {
  AppendArgs a;
  a.k_new = k; a.v_new = v; a.slot_block = c.slot_block; a.slot_offset = c.slot_offset;
  a.kc = (uint8_t*)c.key_cache; a.vc = (uint8_t*)c.value_cache; a.ks = c.k_scale; a.vs = c.v_scale; a.status = c.status;
  a.n = B * S; a.Hkv = Hkv; a.page = c.page_size; a.num_blocks = c.num_blocks; a.in_dtype = in_dtype;
  a.v_format = c.v_format; a.scale_mode = c.scale_mode;
  a.seq_len = S;
  return launch_kv_append(a, D, st);
}

}  // namespace b200

using namespace b200;
extern "C" int cuda_llm_kv_append(const void* k_new, const void* v_new, const int32_t* slot_block,
                                  const int32_t* slot_offset, void* key_cache, void* value_cache, void* k_scale,
                                  void* v_scale, int32_t n_tokens, int32_t num_kv_heads, int32_t head_dim,
                                  int32_t page_size, int32_t num_blocks, int32_t in_dtype, int32_t v_format,
                                  int32_t scale_mode, uint32_t* status, void* stream) {
  if (n_tokens == 0) return CUDA_LLM_OK;
  if (!k_new || !v_new || !slot_block || !slot_offset || !key_cache || !value_cache || !k_scale || !v_scale)
    return CUDA_LLM_EINVAL;
  if ((head_dim != 64 && head_dim != 128) || num_kv_heads <= 0 || page_size <= 0 || num_blocks <= 0 ||
      in_dtype < 0 || in_dtype > CUDA_LLM_BF16 || scale_mode < 0 || scale_mode > CUDA_LLM_SCALE_MX_E8M0 ||
      (v_format != CUDA_LLM_KV_FP8_E4M3 && v_format != CUDA_LLM_KV_FP4_E2M1) ||
      (v_format == CUDA_LLM_KV_FP4_E2M1 && scale_mode != CUDA_LLM_SCALE_MX_E8M0))
    return CUDA_LLM_EINVAL;
  AppendArgs a;
  a.k_new = k_new; a.v_new = v_new; a.slot_block = slot_block; a.slot_offset = slot_offset;
  a.kc = (uint8_t*)key_cache; a.vc = (uint8_t*)value_cache; a.ks = k_scale; a.vs = v_scale; a.status = status;
  a.n = n_tokens; a.Hkv = num_kv_heads; a.page = page_size; a.num_blocks = num_blocks; a.in_dtype = in_dtype;
  a.v_format = v_format; a.scale_mode = scale_mode;
  a.seq_len = 0;
  return launch_kv_append(a, head_dim, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? CUDA_LLM_OK
                                                                                              : CUDA_LLM_ECUDA;
}
