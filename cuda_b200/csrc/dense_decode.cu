// Decode attention over unquantised KV: the paged fp32/fp16/bf16 cache of the reference's
// paged_attention_kernel (paged_attention_kernel.cuh:20-145 in the reference project, layout
// cache[num_blocks, heads, head_dim, page], token innermost) and the contiguous [B, H, S, D]
// tensors of its async_flash_decode_kernel (async_flash_decode_kernel.cuh:29-220).
//
// These two entry points are not the bandwidth-shaped path of this library (that is
// paged_decode_kernel); they are plain split-KV SIMT kernels: one warp per (sequence, KV head,
// KV split) walks its token range 32 tokens at a time, lane = token for Q.K (no shuffles in the
// dot product, the GQA group shares every K element), one warp-wide online-softmax update per
// query row, lane = head_dim slice for P.V.  In the paged layout a V row of 16 tokens is 64 contiguous
// bytes and consecutive head_dim rows are a page apart, so the warp first copies the [head_dim][16 tokens]
// tile of a page into shared memory as [token][head_dim + 1] with coalesced loads and reads it back
// conflict-free (reading V straight from global memory touched 32 sectors per load for 128 useful bytes).
// Partials are merged by merge_partials_kernel.
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "paged_decode_kernel.cuh"

namespace b200 {

cudaError_t launch_merge_partials(const float*, const float*, int, long long, int, void*, int, float*,
                                  cudaStream_t);

struct DenseArgs {
  const void* q;    // paged: [S, Hq, D]; contiguous: [B, Hq, 1, D]
  const void* k;    // paged: [NB, Hkv, D, page]; contiguous: [B, Hkv, S, D]
  const void* v;
  const int32_t* bt;
  const int32_t* ctx;
  float* part_o;    // [n_splits, S*Hq, D]
  float* part_lse;  // [n_splits, S*Hq]   natural log
  int S, Hq, Hkv, group, page, max_blocks, num_blocks, seq_len, n_splits, chunk;
  float scale_log2;
};

template <typename T> __device__ __forceinline__ float elem_to_float(T x);
template <> __device__ __forceinline__ float elem_to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float elem_to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T, int D, int G, bool PAGED>
__global__ void __launch_bounds__(128) dense_decode_kernel(const DenseArgs a) {
  constexpr int C = D / 32;  // head_dim values per lane in P.V
  constexpr float NEG_INF = -__builtin_huge_valf();
  __shared__ float q_s[4][G][D];
  __shared__ float p_s[4][G][32];
  extern __shared__ float v_tile[];  // paged: [4 warps][16 tokens][D + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  const long long n_items = (long long)a.S * a.Hkv * a.n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % a.n_splits);
  const int kvh = (int)((item / a.n_splits) % a.Hkv);
  const int s = (int)(item / ((long long)a.n_splits * a.Hkv));
  int ctx = PAGED ? a.ctx[s] : a.seq_len;
  if (PAGED) ctx = max(0, min(ctx, a.max_blocks * a.page));
  const int t0 = min(ctx, split * a.chunk), t1 = min(ctx, t0 + a.chunk);
  const T* Q = reinterpret_cast<const T*>(a.q);
  const T* K = reinterpret_cast<const T*>(a.k);
  const T* V = reinterpret_cast<const T*>(a.v);

  for (int r = 0; r < G; ++r) {
    const int rr = min(r, a.group - 1);
    const size_t base = ((size_t)s * a.Hq + (size_t)kvh * a.group + rr) * D;
    for (int d = lane; d < D; d += 32) q_s[warp][r][d] = elem_to_float(Q[base + d]);
  }
  __syncwarp();

  float m[G], l[G], acc[G][C];
#pragma unroll
  for (int r = 0; r < G; ++r) {
    m[r] = NEG_INF;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) acc[r][c] = 0.f;
  }

  for (int tb = t0; tb < t1; tb += 32) {
    const int tok = tb + lane;
    const bool valid = tok < t1;
    const int tk = valid ? tok : t1 - 1;  // clamp: dead lanes read a live token and are masked
    long long blk = 0;
    size_t kbase;
    if (PAGED) {
      blk = a.bt[(size_t)s * a.max_blocks + tk / a.page];
      if (blk < 0 || blk >= a.num_blocks) blk = 0;
      kbase = ((size_t)blk * a.Hkv + kvh) * D * a.page + tk % a.page;
    } else {
      kbase = (((size_t)s * a.Hkv + kvh) * a.seq_len + tk) * D;
    }
    float sc[G];
#pragma unroll
    for (int r = 0; r < G; ++r) sc[r] = 0.f;
    if (PAGED) {
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        const float kv = elem_to_float(K[kbase + (size_t)d * a.page]);
#pragma unroll
        for (int r = 0; r < G; ++r) sc[r] = fmaf(q_s[warp][r][d], kv, sc[r]);
      }
    } else {
#pragma unroll 8
      for (int d = 0; d < D; ++d) {
        const float kv = elem_to_float(K[kbase + d]);
#pragma unroll
        for (int r = 0; r < G; ++r) sc[r] = fmaf(q_s[warp][r][d], kv, sc[r]);
      }
    }
    float alpha[G];
#pragma unroll
    for (int r = 0; r < G; ++r) {
      const float x = valid ? sc[r] * a.scale_log2 : NEG_INF;
      float mx = x;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m[r], mx);
      const float mu = (mn == NEG_INF) ? 0.f : mn;
      alpha[r] = fast_exp2(m[r] - mu);
      const float p = fast_exp2(x - mu);
      float ps = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l[r] = l[r] * alpha[r] + ps;
      m[r] = mn;
      p_s[warp][r][lane] = p;
#pragma unroll
      for (int c = 0; c < C; ++c) acc[r][c] *= alpha[r];
    }
    __syncwarp();
    const int nvalid = min(32, t1 - tb);
    if (PAGED) {
      // 16 tokens at a time (they lie in one page: tb is a multiple of 32, pages hold 16, 32 or 64 tokens)
      float* vt = v_tile + warp * 16 * (D + 1);
      for (int half = 0; half < 2 && half * 16 < nvalid; ++half) {
        const long long bj = __shfl_sync(0xffffffffu, blk, half * 16);
        const size_t vbase = ((size_t)bj * a.Hkv + kvh) * D * a.page + (tb + half * 16) % a.page;
        const int t = lane & 15, dd = lane >> 4;
#pragma unroll 8
        for (int i = 0; i < D / 2; ++i) {
          const int d = 2 * i + dd;
          vt[t * (D + 1) + d] = elem_to_float(V[vbase + (size_t)d * a.page + t]);
        }
        __syncwarp();
        const int nt = min(16, nvalid - half * 16);
        for (int j = 0; j < nt; ++j) {
          float vv[C];
#pragma unroll
          for (int c = 0; c < C; ++c) vv[c] = vt[j * (D + 1) + lane + 32 * c];
#pragma unroll
          for (int r = 0; r < G; ++r) {
            const float p = p_s[warp][r][half * 16 + j];
#pragma unroll
            for (int c = 0; c < C; ++c) acc[r][c] = fmaf(p, vv[c], acc[r][c]);
          }
        }
        __syncwarp();
      }
    } else {
      for (int j = 0; j < nvalid; ++j) {
        float vv[C];
        const size_t vbase = (((size_t)s * a.Hkv + kvh) * a.seq_len + tb + j) * D;
#pragma unroll
        for (int c = 0; c < C; ++c) vv[c] = elem_to_float(V[vbase + lane + 32 * c]);
#pragma unroll
        for (int r = 0; r < G; ++r) {
          const float p = p_s[warp][r][j];
#pragma unroll
          for (int c = 0; c < C; ++c) acc[r][c] = fmaf(p, vv[c], acc[r][c]);
        }
      }
    }
    __syncwarp();
  }

  const size_t rows = (size_t)a.S * a.Hq;
#pragma unroll
  for (int r = 0; r < G; ++r) {
    if (r >= a.group) break;
    const size_t row = (size_t)split * rows + (size_t)s * a.Hq + (size_t)kvh * a.group + r;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) a.part_o[row * D + lane + 32 * c] = acc[r][c] * inv;
    if (lane == 0) a.part_lse[row] = l[r] > 0.f ? (m[r] + log2f(l[r])) * 0.69314718055994531f : NEG_INF;
  }
}

template <typename T, int D, bool PAGED>
static cudaError_t launch_dense_g(const DenseArgs& a, cudaStream_t st) {
  const long long n_items = (long long)a.S * a.Hkv * a.n_splits;
  if (n_items == 0) return cudaSuccess;
  const int grid = (int)((n_items + 3) / 4);
  const size_t dyn = PAGED ? (size_t)4 * 16 * (D + 1) * sizeof(float) : 0;  // the V tile of every warp
  auto go = [&](auto kern) -> cudaError_t {
    if (dyn + 4 * 8 * D * sizeof(float) + 4096 > 48 * 1024) {  // static + dynamic beyond the default limit
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
      if (e != cudaSuccess) return e;
    }
    kern<<<grid, 128, dyn, st>>>(a);
    return cudaGetLastError();
  };
  if (a.group <= 1) return go(dense_decode_kernel<T, D, 1, PAGED>);
  if (a.group <= 2) return go(dense_decode_kernel<T, D, 2, PAGED>);
  if (a.group <= 4) return go(dense_decode_kernel<T, D, 4, PAGED>);
  return go(dense_decode_kernel<T, D, 8, PAGED>);
}
template <int D, bool PAGED>
static cudaError_t launch_dense_t(const DenseArgs& a, int dtype, cudaStream_t st) {
  if (dtype == CUDA_LLM_F32) return launch_dense_g<float, D, PAGED>(a, st);
  if (dtype == CUDA_LLM_F16) return launch_dense_g<__half, D, PAGED>(a, st);
  return launch_dense_g<__nv_bfloat16, D, PAGED>(a, st);
}

// Split count: enough warps to fill the GPU, no split shorter than 128 tokens.
static int choose_splits(int S, int Hkv, int max_tokens) {
  const long long base = (long long)S * Hkv;
  int n = (int)((148LL * 16 + base - 1) / (base > 0 ? base : 1));
  const int cap = max_tokens / 128 > 0 ? max_tokens / 128 : 1;
  if (n > cap) n = cap;
  if (n < 1) n = 1;
  if (n > 64) n = 64;
  return n;
}

size_t dense_decode_workspace_bytes(int S, int Hq, int Hkv, int D, int max_tokens) {
  const int n = choose_splits(S, Hkv, max_tokens);
  const size_t rows = (size_t)S * Hq;
  // the first 256 bytes stay free: a workspace shared with the paged decode keeps its status word there
  return 256 + ((size_t)n * rows * sizeof(float) + 255) / 256 * 256 + (size_t)n * rows * D * sizeof(float);
}

cudaError_t run_dense_decode(bool paged, const void* q, const void* k, const void* v, const int32_t* bt,
                             const int32_t* ctx, void* out, int S, int Hq, int Hkv, int D, int page,
                             int max_blocks, int num_blocks, int seq_len, float softmax_scale, int dtype,
                             void* workspace, cudaStream_t st) {
  DenseArgs a;
  a.q = q; a.k = k; a.v = v; a.bt = bt; a.ctx = ctx;
  a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.group = Hq / Hkv; a.page = page; a.max_blocks = max_blocks;
  a.num_blocks = num_blocks; a.seq_len = seq_len;
  const int max_tokens = paged ? max_blocks * page : seq_len;
  a.n_splits = choose_splits(S, Hkv, max_tokens);
  a.chunk = ((max_tokens + a.n_splits - 1) / a.n_splits + 31) / 32 * 32;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  const size_t rows = (size_t)S * Hq;
  a.part_lse = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);  // behind the status header
  a.part_o = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256 +
                                      ((size_t)a.n_splits * rows * sizeof(float) + 255) / 256 * 256);
  cudaError_t e;
  if (paged) e = (D == 64) ? launch_dense_t<64, true>(a, dtype, st) : launch_dense_t<128, true>(a, dtype, st);
  else e = (D == 64) ? launch_dense_t<64, false>(a, dtype, st) : launch_dense_t<128, false>(a, dtype, st);
  if (e != cudaSuccess) return e;
  return launch_merge_partials(a.part_o, a.part_lse, a.n_splits, (long long)rows, D, out, dtype, nullptr, st);
}

}  // namespace b200
