// Launch shims shared by the instantiation units and the C ABI.
#pragma once
#include "paged_decode_kernel.cuh"

namespace b200 {

// One explicit instantiation per (D, PAGE, MODE, NT, PRECISE) lives in a paged_decode_inst_*.cu
// unit; the C ABI only sees these declarations.
template <int D, int PAGE, int MODE, int NT, bool PRECISE>
cudaError_t launch_paged_decode(const DecodeArgs& a, const KvTensorMaps& tm, int grid, size_t smem, cudaStream_t st);

template <int D>
cudaError_t launch_merge_splits(const DecodeArgs& a, int page, int decode_grid, cudaStream_t st);

#define B200_DEFINE_DECODE_LAUNCH(D, PAGE, MODE, NT, PRECISE)                                   \
  template <>                                                                                   \
  cudaError_t launch_paged_decode<D, PAGE, MODE, NT, PRECISE>(const DecodeArgs& a,              \
                                                              const KvTensorMaps& tm, int grid, \
                                                              size_t smem, cudaStream_t st) {   \
    auto kern = paged_decode_kernel<D, PAGE, MODE, NT, PRECISE>;                                \
    static int configured[64] = {0};                                                            \
    int dev = 0;                                                                                \
    cudaError_t e = cudaGetDevice(&dev);                                                        \
    if (e != cudaSuccess) return e;                                                             \
    if (dev < 64 && !configured[dev]) {                                                         \
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,               \
                               (int)kSmemBudget);                                               \
      if (e != cudaSuccess) return e;                                                           \
      configured[dev] = 1;                                                                      \
    }                                                                                           \
    cudaLaunchConfig_t cfg = {};                                                                \
    cfg.gridDim = dim3((unsigned)grid);                                                         \
    cfg.blockDim = dim3(kDecodeThreads);                                                        \
    cfg.dynamicSmemBytes = smem;                                                                \
    cfg.stream = st;                                                                            \
    cudaLaunchAttribute attr[1];                                                                \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                            \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                     \
    cfg.attrs = attr;                                                                           \
    cfg.numAttrs = 1;                                                                           \
    return cudaLaunchKernelEx(&cfg, kern, a, tm);                                               \
  }

// every page size and row-tile variant of one (MODE, D)
#define B200_DEFINE_DECODE_FAMILY(D, MODE)            \
  B200_DEFINE_DECODE_LAUNCH(D, 16, MODE, 1, false)    \
  B200_DEFINE_DECODE_LAUNCH(D, 16, MODE, 1, true)     \
  B200_DEFINE_DECODE_LAUNCH(D, 16, MODE, 2, false)    \
  B200_DEFINE_DECODE_LAUNCH(D, 32, MODE, 1, false)    \
  B200_DEFINE_DECODE_LAUNCH(D, 32, MODE, 1, true)     \
  B200_DEFINE_DECODE_LAUNCH(D, 32, MODE, 2, false)    \
  B200_DEFINE_DECODE_LAUNCH(D, 64, MODE, 1, false)    \
  B200_DEFINE_DECODE_LAUNCH(D, 64, MODE, 1, true)     \
  B200_DEFINE_DECODE_LAUNCH(D, 64, MODE, 2, false)

}  // namespace b200
