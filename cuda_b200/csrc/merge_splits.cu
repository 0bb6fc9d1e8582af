// Split merge kernel launches and the stand-alone partial merge used after the all-gather of
// the split-context mode.
#include "decode_launch.cuh"

namespace b200 {

template <int D>
cudaError_t launch_merge_splits(const DecodeArgs& a, int page, int decode_grid, cudaStream_t st) {
  const long long blocks = (long long)a.S * a.Hq;
  if (blocks == 0) return cudaSuccess;
  // few sequences cut across many CTAs leave many results per row: more warps per block then.  (Blocks of 16
  // warps fit four to an SM and the kernel is a chain of dependent loads, so they are taken only where a row
  // really has that many parts: about grid / (S n_hg) + 2 CTAs per row, SUBS results each, two for helper pairs;
  // measured: 48 parts per row take 16 us with 4 warps and 29 us with 16.)
  const long long est_parts = ((long long)decode_grid / ((long long)a.S * a.n_hg) + 2) * a.SUBS *
                              ((a.helper_pairs && a.rows_max == 16) ? 2 : 1);
  const bool many_parts = est_parts > 128;
  cudaLaunchConfig_t cfg = {};
  // y: the query tokens of a sequence (blocks beyond its q_len return at once), so that the rows of a
  // multi-token query are merged side by side instead of one after the other
  // (as long as that keeps the grid to about 8192 blocks: with many sequences the blocks that find no token
  // of their own cost more than the serial loop)
  const int q_max = a.cuq ? (a.rows_max / a.group > 1 ? a.rows_max / a.group : 1) : 1;
  long long q_par = 8192 / blocks;
  q_par = q_par < 1 ? 1 : q_par > q_max ? q_max : q_par;
  cfg.gridDim = dim3((unsigned)blocks, (unsigned)q_par);
  const bool some_parts = !many_parts && est_parts > 32;  // 8 warps: eight such blocks still fit an SM
  cfg.blockDim = dim3(many_parts ? 512 : some_parts ? 256 : 128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the decode kernel drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (many_parts) return cudaLaunchKernelEx(&cfg, merge_splits_kernel<D, 16>, a, page);
  if (some_parts) return cudaLaunchKernelEx(&cfg, merge_splits_kernel<D, 8>, a, page);
  return cudaLaunchKernelEx(&cfg, merge_splits_kernel<D, 4>, a, page);
}
template cudaError_t launch_merge_splits<64>(const DecodeArgs&, int, int, cudaStream_t);
template cudaError_t launch_merge_splits<128>(const DecodeArgs&, int, int, cudaStream_t);

// Part p holds out [rows, D] fp32 at parts_out + p * part_stride and lse [rows] (natural log) at
// parts_lse + p * part_stride (strides in floats).  One warp per row.
template <int D>
__global__ void __launch_bounds__(128)
merge_partials_kernel(const float* __restrict__ parts_out, const float* __restrict__ parts_lse,
                      size_t out_stride, size_t lse_stride, int num_parts, long long rows, void* out,
                      int out_dtype, float* lse) {
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  // may be launched as a programmatic dependent of the kernel that writes the parts: nothing of theirs
  // is read before this wait (a no-op after an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (row >= rows) return;
  constexpr int VPL = D / 32;
  constexpr float LOG2E = 1.4426950408889634f;
  float mx = -__builtin_huge_valf();
  for (int p = lane; p < num_parts; p += 32) mx = fmaxf(mx, parts_lse[(size_t)p * lse_stride + row]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float mu = (mx == -__builtin_huge_valf()) ? 0.f : mx;
  float acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) acc[v] = 0.f;
  float wsum = 0.f;
  // weights 32 parts at a time (one per lane), then independent row loads
  for (int base = 0; base < num_parts; base += 32) {
    const int mine = base + lane;
    const float wl = mine < num_parts ? fast_exp2((parts_lse[(size_t)mine * lse_stride + row] - mu) * LOG2E) : 0.f;
    const int cnt = min(32, num_parts - base);
#pragma unroll 4
    for (int j = 0; j < cnt; ++j) {
      const float w = __shfl_sync(0xffffffffu, wl, j);
      wsum += w;
      const float* po = parts_out + (size_t)(base + j) * out_stride + (size_t)row * D + lane * VPL;
#pragma unroll
      for (int v = 0; v < VPL; ++v) acc[v] = fmaf(w, po[v], acc[v]);
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
  for (int v = 0; v < VPL; ++v)
    store_out_elem(out, out_dtype, (size_t)row * D + lane * VPL + v, acc[v] * inv);
  if (lse && lane == 0) lse[row] = wsum > 0.f ? mu + logf(wsum) : -__builtin_huge_valf();
}

// The same merge for rows with many parts (a few long sequences cut into hundreds of chunks): one block of W
// warps per row, warp w takes parts w, w + W, ...
template <int D, int W>
__global__ void __launch_bounds__(32 * W)
merge_partials_wide_kernel(const float* __restrict__ parts_out, const float* __restrict__ parts_lse, size_t out_stride,
                           size_t lse_stride, int num_parts, long long rows, void* out, int out_dtype, float* lse) {
  constexpr int VPL = D / 32;
  constexpr float LOG2E = 1.4426950408889634f;
  constexpr float NEG_INF = -__builtin_huge_valf();
  __shared__ float s_max[W];
  __shared__ float s_sum[W];
  __shared__ float s_acc[W][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = blockIdx.x;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float mx = NEG_INF;
  for (int p = threadIdx.x; p < num_parts; p += 32 * W) mx = fmaxf(mx, parts_lse[(size_t)p * lse_stride + row]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[warp] = mx;
  __syncthreads();
  mx = s_max[0];
#pragma unroll
  for (int w = 1; w < W; ++w) mx = fmaxf(mx, s_max[w]);
  const float mu = (mx == NEG_INF) ? 0.f : mx;
  float acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) acc[v] = 0.f;
  float wsum = 0.f;
  // 32 of the warp's parts at a time: one weight per lane, then every lane walks their rows
  for (int base = warp; base < num_parts; base += 32 * W) {
    const int mine = base + W * lane;
    const float wl = mine < num_parts ? fast_exp2((parts_lse[(size_t)mine * lse_stride + row] - mu) * LOG2E) : 0.f;
    const int cnt = min(32, (num_parts - base + W - 1) / W);
#pragma unroll 8
    for (int j = 0; j < cnt; ++j) {
      const float w = __shfl_sync(0xffffffffu, wl, j);
      wsum += w;
      const float* po = parts_out + (size_t)(base + W * j) * out_stride + (size_t)row * D + lane * VPL;
#pragma unroll
      for (int v = 0; v < VPL; ++v) acc[v] = fmaf(w, po[v], acc[v]);
    }
  }
#pragma unroll
  for (int v = 0; v < VPL; ++v) s_acc[warp][lane * VPL + v] = acc[v];
  if (lane == 0) s_sum[warp] = wsum;
  __syncthreads();
  if (warp == 0) {
    wsum = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) wsum += s_sum[w];
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int d = lane * VPL + v;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) sum += s_acc[w][d];
      store_out_elem(out, out_dtype, (size_t)row * D + d, sum * inv);
    }
    if (lse && lane == 0) lse[row] = wsum > 0.f ? mu + logf(wsum) : NEG_INF;
  }
}

cudaError_t launch_merge_partials_strided(const float* parts_out, const float* parts_lse, size_t part_stride,
                                          int num_parts, long long rows, int head_dim, void* out, int out_dtype,
                                          float* lse, cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  const int grid = (int)((rows + 3) / 4);
  if (head_dim == 64)
    merge_partials_kernel<64><<<grid, 128, 0, st>>>(parts_out, parts_lse, part_stride, part_stride, num_parts,
                                                    rows, out, out_dtype, lse);
  else
    merge_partials_kernel<128><<<grid, 128, 0, st>>>(parts_out, parts_lse, part_stride, part_stride, num_parts,
                                                     rows, out, out_dtype, lse);
  return cudaGetLastError();
}

cudaError_t launch_merge_partials(const float* parts_out, const float* parts_lse, int num_parts,
                                  long long rows, int head_dim, void* out, int out_dtype,
                                  float* lse, cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  const size_t os = (size_t)rows * head_dim, ls = (size_t)rows;  // dense [P, rows, D] and [P, rows]
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((rows + 3) / 4));
  cfg.blockDim = dim3(128);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the kernel in front drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (num_parts > 64) {  // many parts per row: a block of 16 warps per row
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(512);
    if (head_dim == 64)
      return cudaLaunchKernelEx(&cfg, merge_partials_wide_kernel<64, 16>, parts_out, parts_lse, os, ls, num_parts, rows, out,
                                out_dtype, lse);
    return cudaLaunchKernelEx(&cfg, merge_partials_wide_kernel<128, 16>, parts_out, parts_lse, os, ls, num_parts, rows, out,
                              out_dtype, lse);
  }
  if (head_dim == 64)
    return cudaLaunchKernelEx(&cfg, merge_partials_kernel<64>, parts_out, parts_lse, os, ls, num_parts, rows, out,
                              out_dtype, lse);
  return cudaLaunchKernelEx(&cfg, merge_partials_kernel<128>, parts_out, parts_lse, os, ls, num_parts, rows, out,
                            out_dtype, lse);
}

}  // namespace b200
