// Device primitives for sm_100a used by the paged decode kernels: mbarrier with bounded
// waits, 1-D bulk (TMA) global->shared copies, warp-level f16 MMA, E4M3 -> f16
// conversion and byte shuffles.
//
// Every wait in this file gives up after a bounded number of polls and reports failure to
// its caller instead of spinning forever; callers turn that into a status word the host
// reads (the reference's only wait primitive spins without bound,
// cuda_compat.h:174-193 in the reference project).
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cuda.h>  // CUtensorMap (type only; no driver-API call is linked)

namespace b200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// upper bound (ns) a single try_wait may sleep in hardware before it reports "not yet"
constexpr uint32_t kSuspendHintNs = 2000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait: false after kMaxPolls unsuccessful polls (each poll may itself suspend for up to
// kSuspendHintNs, so the bound is of the order of a few seconds at most), or after kShortPolls of
// them when `short_limit` is set (a run-time switch, so that a test can make a wait run out in
// milliseconds; written as a second comparison against a constant because a run-time loop bound
// costs the decode kernel a register it does not have).
constexpr uint32_t kMaxPolls = 1u << 21;
constexpr uint32_t kShortPolls = 1u << 12;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int short_limit) {
  for (uint32_t i = 0; i < kMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (short_limit && i >= kShortPolls) break;
  }
  return false;
}

// ----------------------------------------------------------------------------------------
// 1-D bulk copy global -> shared, completion counted on an mbarrier (bytes).
// Both addresses 16-byte aligned, size a multiple of 16.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// The same copy with an L2 eviction policy (createpolicy): data that is read once should not push
// the small, re-read tensors (tables, lengths, partial results) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

// 3-D tiled TMA copy global -> shared through a tensor map (cuTensorMapEncodeTiled), completion counted
// on an mbarrier, with an L2 eviction policy.  The box lands in this CTA's own
// shared memory.  The innermost coordinate times the element size must be a multiple of 16 bytes
// (callers pass 0), the destination aligned to the swizzle pattern of the map.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst_smem, const void* tensor_map, int c0, int c1, int c2,
                                                 uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy)
      : "memory");
}

// 4-byte asynchronous copy global -> shared (no register in between), grouped and waited on
// with commit / wait_group.
__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------
// Shared-memory loads and stores
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {  // zero-extended
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, int v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, int x, int y, int z, int w) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// ----------------------------------------------------------------------------------------
// Byte permute and conversions
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// two E4M3 bytes (low 16 bits of x) -> f16x2; low byte -> low half.  Exact for every code.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_lo(uint32_t x) {
  uint32_t d;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}"
      : "=r"(d) : "r"(x));
  return d;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_hi(uint32_t x) {
  uint32_t d;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, hi;\n\t}"
      : "=r"(d) : "r"(x));
  return d;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// E8M0 byte -> fp32 2^(e-127).  0 -> 2^-127 (fp32 subnormal), 255 -> NaN.
__device__ __forceinline__ float e8m0_to_f32(uint32_t e) {
  uint32_t bits = (e == 0u) ? 0x00400000u : (e == 255u ? 0x7fc00000u : (e << 23));
  return __uint_as_float(bits);
}

// two fp32 -> two E4M3 bytes (round to nearest even, saturating): lo -> bits 7..0, hi -> 15..8
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
// low / high half of an f16x2 as fp32
__device__ __forceinline__ float f16x2_lo(uint32_t v) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xffffu)));
}
__device__ __forceinline__ float f16x2_hi(uint32_t v) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16)));
}

// ----------------------------------------------------------------------------------------
// ldmatrix: four 8x8 matrices of 16-bit elements; lane l supplies the address of row (l % 8)
// of matrix (l / 8), rows are 16 bytes.  Plain: thread (g,t) gets, per matrix, the 4 bytes
// 4t..4t+3 of row g.  Transposed: thread (g,t) gets {M[2t][g], M[2t+1][g]} as 16-bit elements,
// i.e. bytes (2g, 2g+1) of row 2t in the low half and of row 2t+1 in the high half.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// ----------------------------------------------------------------------------------------
// Warp MMA m16n8k16, f16 inputs, fp32 accumulate:  D(16x8) += A(16x16) * B(16x8)
// Fragment ownership (g = lane/4, t = lane%4):
//   a0:(row g,   k 2t..2t+1)  a1:(row g+8, k 2t..2t+1)  a2:(row g, k 2t+8..9)  a3:(row g+8, k 2t+8..9)
//   b0:(k 2t..2t+1, col g)    b1:(k 2t+8..9, col g)
//   c0:(row g, col 2t) c1:(row g, col 2t+1) c2:(row g+8, col 2t) c3:(row g+8, col 2t+1)
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 8x8 b16 transpose across the warp: thread (g,t) gives row g cols 2t..2t+1 and receives
// {M[2t][g], M[2t+1][g]}.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

}  // namespace b200
