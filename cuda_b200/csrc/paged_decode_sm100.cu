// Paged decode attention over an 8-bit KV cache on the 5th-generation tensor cores (tcgen05.mma
// kind::f8f6f4, accumulators in tensor memory), sm_100a.  Same contract, work plan, workspace format
// and split merge as paged_decode_kernel (paged_decode_kernel.cuh); what changes is where the E4M3
// bytes are widened: nowhere.  The page slabs of the reference layout cache[num_blocks, heads,
// head_dim, page] are valid tensor-core operands as they land in shared memory:
//
//   S^T[token, row] = K^T Q^T   A = K tile, MN-major (tokens contiguous): a page [head_dim][16 tokens] is
//                               sixteen 8 x 16-byte core matrices; eight pages make the 128 accumulator
//                               lanes.  B = the query rows of the KV head, quantised once per (sequence,
//                               KV head) to E4M3 as a high part and a residual (two terms keep 16-bit
//                               accuracy), K-major.
//   O^T[d, row] += V^T P^T      A = V tile, K-major (the same slabs read the other way), B = P^T written
//                               by the softmax threads as E4M3 high + residual, MN-major (one 16-byte
//                               store per token).
//
// Tokens sit on the TMEM lanes, so a softmax thread owns one token of the tile and all query rows of
// the KV head; per-token scales are scalars of the thread.  E8M0 block scales along head_dim: K is
// multiplied block by block (four S accumulators, one per 32 head_dim values, combined in fp32 by the
// thread); V needs P * 2^e_b(token), which differs per block, so there are four P variants and four O
// accumulators, each with its own running maximum (w_b = s + e_b), and a thread reads the lane quarter
// of "its" block at the end.  The running maxima are only raised when a tile exceeds them by 2^2
// (P = 2^(w - m + 6) then stays below 2^8, inside E4M3), so the cross-lane maximum and the rescale of
// O in TMEM run on the first tile of a segment and rarely afterwards.  Both E4M3 B operands carry a
// second term, 16 x the rounding residual, in accumulator columns of their own.
//
// A work unit is a 128-token tile of TWO adjacent KV heads (their slabs are contiguous in a page, so one
// 4 KB bulk copy per page and tensor brings both: the copy engine takes a request every ~80 cycles
// whatever its size, and 2 KB requests could not keep up with HBM).  Roles (352 threads): warps 0-3 and
// 4-7 are two softmax groups, one per head of the pair, each with its own S / P / O buffers; warp 8
// walks the CTA's range and issues the copies; warp 9 issues the MMAs; warp 10 quantises the query
// rows of the coming (sequence, head pair) segments.
#include "paged_decode_kernel.cuh"
#include "tcgen05_primitives.cuh"

namespace b200 {

constexpr int kD100Threads = 352;  // 8 softmax warps, producer, MMA issue, query preparation
constexpr int kD100Tile = 128;        // tokens per tile = TMEM lanes
// P is written as E4M3: P = 2^(w - m + kPShift), so that weights down to 2^-(9 + kPShift) of the running
// maximum are still represented; a running maximum is raised when a tile exceeds it by 2^kLazyMax, so P
// stays below 2^(kPShift + kLazyMax) = 256 (E4M3 reaches 448).  The residual terms of Q and P are stored
// times 2^kResShift in accumulator columns of their own, which extends the small end by another 2^4.
constexpr float kLazyMax = 2.f;
constexpr float kPShift = 6.f;
constexpr float kResScale = 16.f, kResInv = 0.0625f;

__device__ unsigned int g_decode100_wait_timeouts = 0;

template <int MODE, int RP>
struct D100Cfg {
  static constexpr bool MX = (MODE == MODE_MX8 || MODE == MODE_MX8K_MX4V);
  static constexpr bool V4 = (MODE == MODE_MX8K_MX4V);
  static constexpr int NV = MX ? 4 : 1;        // P variants = O accumulators
  static constexpr int NVW = MX ? 5 : 1;       // running-maximum sets (the last one, MX only, is the denominator's)
  static constexpr int NH = (RP == 16) ? 2 : 1;  // B operands per product: [high | residual] in one (8 rows) or two (16 rows)
  // accumulator columns per S block / O variant: [high rows | residual rows], padded to the 16 columns an MMA has at least
  static constexpr int CS = (RP <= 8) ? 16 : 32;
  // tensor memory, per group (= head of the pair) 256 columns: S blocks from 0 (a second S buffer from 64
  // where the blocks of one fit in 64 columns), O variants from 128
  static constexpr int SCOLS = (MX ? 4 : 1) * CS;    // columns of one S buffer
  static constexpr int NSB = (SCOLS <= 64) ? 2 : 1;  // S buffers per group
  // shared memory (bytes from the 1024-aligned base): mbarriers in the first 256 bytes
  static constexpr uint32_t kBarFull = 0, kBarEmpty = 64, kBarSFull = 128, kBarSFree = 160, kBarPFull = 192,
                            kBarPvDone = 208, kBarQReady = 224, kBarQFree = 240;
  static constexpr uint32_t kGrp = kBtRingOff + kBtRing * kMaxPagesPerStage * 4;  // per-group scratch
  static constexpr uint32_t kGrpBytes = 2304;
  // group scratch: maxima [5][16] f32 @0, factors [5][16] @320, reduction [4][5][16] @640, sums [4][16] @1920,
  // flags [4] @2176, "a wait of this group ran out" @2192; behind that in group 0's: TMEM address, end flag, plan
  static constexpr uint32_t kTmemSlot = kGrp + 2208, kDone = kGrp + 2212, kPlan = kGrp + 2216;
  static constexpr uint32_t kQs = kGrp + 2 * kGrpBytes;      // per query buffer and head: 16 row factors
  static constexpr uint32_t kQbuf = (kQs + 2 * 2 * 64 + 127) / 128 * 128;
  static constexpr uint32_t kQHead = NH * 2048;              // one head's operand
  static constexpr uint32_t kQbufBytes = 2 * kQHead;         // one buffer: both heads
  static constexpr uint32_t kP = kQbuf + 2 * kQbufBytes;
  static constexpr uint32_t kPBytes = NV * NH * 2048;        // per group
  static constexpr uint32_t kStages = (kP + 2 * kPBytes + 1023) / 1024 * 1024;
  // stage: 8 pages x 2 heads of K slabs, the same of V, 8 x 128 bytes of K scales, 8 x 128 bytes of V scales
  static constexpr uint32_t kPageK = 4096, kOffV = 8 * kPageK, kOffKs = 2 * kOffV, kOffVs = kOffKs + 8 * 128;
  static constexpr uint32_t kStageBytes = kOffVs + 8 * 128;
  static constexpr int kStagesMax = (int)((kSmemBudget - kStages) / kStageBytes) < kMaxStages
                                        ? (int)((kSmemBudget - kStages) / kStageBytes) : kMaxStages;
};

// The same bounded wait for events that are a tile time away: a short sleep between polls, so that the
// waiting warp leaves the issue slots of its scheduler to the warps that are working.
__device__ __forceinline__ bool tc_wait_relaxed(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 21); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    __nanosleep(32);
  }
  return false;
}
// waits whose outcome is the same for every lane of the (converged) warp
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, tc_wait(bar, parity));
}
__device__ __forceinline__ bool warp_wait_relaxed(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, tc_wait_relaxed(bar, parity));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
// one arrival on the mbarrier once every cp.async this thread has issued so far has landed (the arrival
// is part of the barrier's expected count)
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128u(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// order-preserving map float <-> int32, for redux.sync.max
__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }
__device__ __forceinline__ float warp_max(float v) {
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(f2ord(v)));
  return ord2f(r);
}
// two values -> E4M3 high bytes and E4M3 bytes of 16 x the residual, through f16 (values up to 448)
__device__ __forceinline__ void split_e4m3x2(float lo, float hi, uint32_t& top, uint32_t& rest) {
  const uint32_t h2 = pack_f16x2(lo, hi);
  uint16_t t;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(t) : "r"(h2));
  uint32_t back, res;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(back) : "h"(t));
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(res) : "r"(h2), "r"(back));
  asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(res) : "r"(0x4C004C00u));  // x 16
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(res));
  top = t;
  rest = r;
}

template <int MODE, int RP>
__global__ void __launch_bounds__(kD100Threads, 1)
paged_decode_sm100_kernel(const __grid_constant__ DecodeArgs a) {
  using C = D100Cfg<MODE, RP>;
  constexpr bool MX = C::MX;
  constexpr int NV = C::NV, NVW = C::NVW, NH = C::NH;
  constexpr int D = 128, PAGE = 16, PPS = 8, NB = 4;
  constexpr float NEG_INF = -__builtin_huge_valf();
  constexpr float kMaxFloor = -1.0e30f;

  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb0 = smem_u32(smem);
  const uint32_t full_bar = sb0 + C::kBarFull, empty_bar = sb0 + C::kBarEmpty;
  volatile long long* plan = reinterpret_cast<volatile long long*>(smem + C::kPlan);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kTmemSlot);
  volatile uint32_t* done_flag = reinterpret_cast<volatile uint32_t*>(smem + C::kDone);
  long long* scan = reinterpret_cast<long long*>(smem + C::kStages);  // prologue scratch (stage memory)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NS = a.n_stages;

  if (!a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(full_bar + 8 * i, 9);   // the byte count's arrival + one per page lane of the producer (scale copies)
      mbar_init(empty_bar + 8 * i, 1);
    }
    for (int g = 0; g < 2; ++g) {
      for (int b = 0; b < 2; ++b) {  // per S buffer
        mbar_init(sb0 + C::kBarSFull + 8 * (2 * g + b), 1);
        mbar_init(sb0 + C::kBarSFree + 8 * (2 * g + b), 4);
      }
      mbar_init(sb0 + C::kBarPFull + 8 * g, 4);
      mbar_init(sb0 + C::kBarPvDone + 8 * g, 1);
      mbar_init(sb0 + C::kBarQReady + 8 * g, 1);
      // freed by the MMA warp (its products with the operand are done) and by every softmax thread (it has read
      // the segment's row factors, which live in the same buffer)
      mbar_init(sb0 + C::kBarQFree + 8 * g, 1 + 256);
      *reinterpret_cast<volatile uint32_t*>(smem + C::kGrp + g * C::kGrpBytes + 2192) = 0;
    }
    *done_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(sb0 + C::kTmemSlot, 512);
    tmem_relinquish();
  }

  // ---------------------------------------------------------------- plan: equal unit ranges
  // (the arithmetic of paged_decode_kernel with two KV heads per unit and tiles of 128 tokens)
  const int per = (a.S + kD100Threads - 1) / kD100Threads;
  const int s_lo = min(a.S, tid * per), s_hi = min(a.S, s_lo + per);
  auto seq_cost = [&](int s) -> long long {
    int qb, ql;
    seq_q(a, s, qb, ql);
    const int c = eff_ctx(a, s, PAGE);
    if (ql <= 0 || c <= 0) return 0;
    return ((long long)((c + kD100Tile - 1) / kD100Tile) + kSegGap) * a.n_hg;
  };
  long long my_units = 0;
  for (int s = s_lo; s < s_hi; ++s) my_units += seq_cost(s);
  long long incl = my_units;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) scan[warp] = incl;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  long long warp_base = 0, total_units = 0;
#pragma unroll
  for (int w = 0; w < kD100Threads / 32; ++w) {
    const long long v = scan[w];
    if (w < warp) warp_base += v;
    total_units += v;
  }
  const long long my_prefix = warp_base + incl - my_units;
  const long long per_cta = max((total_units + gridDim.x - 1) / gridDim.x, 1ll);
  const int vb = (int)blockIdx.x;
  const long long u_begin = min(total_units, (long long)vb * per_cta);
  const long long u_end = min(total_units, u_begin + per_cta);
  if (u_begin < u_end && my_units > 0 && u_begin >= my_prefix && u_begin < my_prefix + my_units) {
    long long U = my_prefix;
    for (int s = s_lo; s < s_hi; ++s) {
      const long long n = seq_cost(s);
      if (u_begin < U + n) {
        plan[1] = s;
        plan[2] = U;
        break;
      }
      U += n;
    }
  }
  __syncthreads();
  const bool has_work = u_begin < u_end;

  // the (sequence, head pair, tile) units of this CTA's range, walked by the producer, by the table
  // prefetch and by the query warp (each with its own cursor)
  auto load_seq = [&](UnitCursor& c) {
    c.ctx = eff_ctx(a, c.s, PAGE);
    seq_q(a, c.s, c.qbase, c.qlen);
    c.tiles = (c.qlen > 0) ? (c.ctx + kD100Tile - 1) / kD100Tile : 0;
    c.w = 1;
  };
  auto advance = [&](UnitCursor& c) {
    c.pos += 1;
    if (c.pos >= u_end) return;
    if (++c.tile < c.tiles) return;
    c.tile = 0;
    c.pos += kSegGap;
    if (c.pos >= u_end) return;
    c.seg_first = c.pos;
    if (++c.hg < a.n_hg) return;
    c.hg = 0;
    for (;;) {
      ++c.s;
      if (c.s >= a.S) {
        c.s = a.S - 1;
        c.tiles = 0;
        return;
      }
      load_seq(c);
      if (c.tiles > 0) return;
    }
  };
  auto seat = [&](UnitCursor& c) {  // first unit at or behind u_begin
    c.s = (int)plan[1];
    load_seq(c);
    const long long base = plan[2];
    const int stride = kSegGap + c.tiles;
    const int o = (int)(u_begin - base);
    c.hg = o / stride;
    const int rem = o - c.hg * stride - kSegGap;  // offset behind the gap (negative: inside it)
    c.tile = rem <= 0 ? 0 : rem;
    c.seg_first = base + (long long)c.hg * stride + kSegGap;
    c.pos = c.seg_first + c.tile;
  };

  if (has_work && warp == 8) {
    // =============================================================== producer warp
    const uint64_t stream_policy = l2_policy_evict_first();
    UnitCursor ic;
    seat(ic);
    UnitCursor pc = ic;
    const uint32_t ring = sb0 + kBtRingOff;
    int pf_done = 0;
    auto prefetch = [&]() {
      if (pc.pos < u_end) {
        const int tok0 = pc.tile * kD100Tile;
        const int np = min(PPS, (pc.ctx - tok0 + PAGE - 1) / PAGE);
        if (lane < np) {
          const int32_t* src = a.bt + (size_t)pc.s * a.max_blocks + min(tok0 / PAGE + lane, a.max_blocks - 1);
          cp_async_4(ring + ((pf_done % kBtRing) * kMaxPagesPerStage + lane) * 4, src);
        }
        ++pf_done;
        advance(pc);
      }
      cp_async_commit();
    };
    for (int j = 0; j < kBtAhead; ++j) prefetch();
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");

    int seg_cta_first = 0, seg_n_cta = 1, seg_idx = 0, seg_n = 1, seg_count = -1;
    bool seg_fresh = true, seg_direct = false, ok = true;
    int issued = 0, slot = 0;
    uint32_t phase = 0;
    for (int it = 0;; ++it, slot = (slot + 1 == NS) ? 0 : slot + 1, phase ^= (slot == 0) ? 1u : 0u) {
      if (it >= NS && !warp_wait_relaxed(empty_bar + 8 * slot, phase ^ 1)) {
        ok = false;
        break;
      }
      const uint32_t fb = full_bar + 8 * slot;
      if (ic.pos >= u_end) {
        // terminal stage: no bytes, tells warp 9 that this CTA's range is done
        if (lane == 0) {
          sts128(sb0 + kMetaOff + slot * (uint32_t)sizeof(StageMeta) + 16, FLAG_END, 0, 0, 0);
          mbar_arrive_expect_tx(fb, 0u);
        }
        if (lane < 8) mbar_arrive(fb);
        break;
      }
      cp_async_wait<kBtAhead - 1>();
      __syncwarp();
      const bool is_new = seg_fresh || (ic.tile == 0);
      if (is_new) {
        const long long seg_last = ic.seg_first + (long long)(ic.tiles - 1);
        seg_cta_first = (int)(ic.seg_first / per_cta);
        seg_n_cta = (int)(seg_last / per_cta) - seg_cta_first + 1;
        seg_direct = seg_n_cta == 1;   // the whole (sequence, head pair) lies in this CTA's range: no merge needed
        seg_idx = 0;
        ++seg_count;
        seg_n = (int)min((long long)(ic.tiles - ic.tile), u_end - ic.pos);  // tiles of this segment in this CTA's range
      }
      const int tok0 = ic.tile * kD100Tile;
      const int np = min(PPS, (ic.ctx - tok0 + PAGE - 1) / PAGE);
      int c_blk = 0;
      if (lane < np) {
        c_blk = (int)lds32(ring + ((it % kBtRing) * kMaxPagesPerStage + lane) * 4);
        if (c_blk < 0 || c_blk >= a.num_blocks) {
          atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
          c_blk = 0;
        }
      }
      const bool is_last = (seg_idx == seg_n - 1);
      const uint32_t meta = sb0 + kMetaOff + slot * (uint32_t)sizeof(StageMeta);
      if (lane == 0) {
        const int flags = (is_new ? FLAG_NEW : 0) | (is_last ? FLAG_LAST : 0) | (seg_direct ? FLAG_DIRECT : 0);
        sts128(meta, ic.s, ic.hg, tok0, ic.ctx);
        sts128(meta + 16, flags, ic.s * a.n_hg + ic.hg + vb, ic.qbase, ic.qlen);
        sts128(meta + 32, seg_idx, seg_n, seg_count, 0);
        if (ic.tile == 0) {
          int32_t* t = a.table + 4 * (size_t)(ic.s * a.n_hg + ic.hg);
          t[0] = seg_cta_first;
          t[1] = seg_n_cta;
          t[2] = seg_direct ? 1 : 0;
        }
        mbar_arrive_expect_tx(fb, (uint32_t)np * (a.k_chunk + a.v_chunk));
      }
      seg_fresh = false;
      __syncwarp();
      // failure-path test: the bytes of the first unit of the launch are announced but never sent
      const bool stalled = a.stall_test && ic.pos == kSegGap;
      const uint32_t sb = sb0 + C::kStages + slot * C::kStageBytes;
      if (lane < np && !stalled) {
        // both heads of the pair are contiguous in the page: one 4 KB copy per tensor
        const uint64_t b = (uint64_t)c_blk;
        bulk_g2s_hint(sb + lane * C::kPageK, a.kc + b * a.k_blk_stride + (uint64_t)ic.hg * a.k_chunk, a.k_chunk, fb, stream_policy);
        bulk_g2s_hint(sb + C::kOffV + lane * C::kPageK, a.vc + b * a.v_blk_stride + (uint64_t)ic.hg * a.v_chunk, a.v_chunk, fb,
                      stream_policy);
      }
      if (lane < 8) {
        // the 128 scale bytes of a (page, head pair) go as 16-byte cp.async from the lane of the page (the
        // bulk-copy engine takes as long for them as for 4 KB), then one arrival per lane that fires when
        // they have landed
        if (lane < np) {
          const uint64_t off = (uint64_t)c_blk * a.ks_blk_stride + (uint64_t)ic.hg * a.ks_chunk;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            cp_async_16(sb + C::kOffKs + lane * 128 + ch * 16, a.ks + off + ch * 16);
            cp_async_16(sb + C::kOffVs + lane * 128 + ch * 16, a.vs + off + ch * 16);
          }
        }
        cp_async_arrive_noinc(fb);
      }
      issued = it + 1;
      ++seg_idx;
      prefetch();
      advance(ic);
    }
    cp_async_wait<0>();
    if (!ok) {
      if (lane == 0) {
        atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
        atomicAdd(&g_decode100_wait_timeouts, 1u);
      }
      // wait (bounded) for this warp's own copies still in flight before leaving
      for (int it = max(0, issued - NS); it < issued; ++it) (void)warp_wait(full_bar + 8 * (it % NS), (it / NS) & 1);
    }
  } else if (has_work && warp == 10) {
    // =============================================================== query warp
    // The query rows of every (sequence, head pair) of the range, up to two segments ahead of the MMAs:
    // per head, E4M3 high part and 16 x residual as a K-major operand, byte (row n, d) at
    // (d / 16) * 256 + n * 16 + d % 16.  Every row is scaled by a power of two that brings its largest
    // magnitude into [128, 256); the factor goes back in with the softmax scale.
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
    UnitCursor c;
    seat(c);
    int segc = -1;
    bool fresh = true, ok = true;
    while (c.pos < u_end) {
      if (fresh || c.tile == 0) {
        ++segc;
        const int qb = segc & 1;
        if (segc >= 2 && !warp_wait_relaxed(sb0 + C::kBarQFree + 8 * qb, (uint32_t)((segc >> 1) - 1) & 1)) {
          ok = false;
          break;
        }
        const int R = a.group * c.qlen;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          const int kvh = c.hg * 2 + h;
          const uint32_t qbuf = sb0 + C::kQbuf + qb * C::kQbufBytes + h * C::kQHead;
          float* qs = reinterpret_cast<float*>(smem + C::kQs + (qb * 2 + h) * 64);
          uint2 raw[RP];
#pragma unroll
          for (int r = 0; r < RP; ++r) {
            raw[r] = make_uint2(0u, 0u);
            if (r < R) {
              const int jq = r / a.group, iq = r - jq * a.group;
              const size_t base = ((size_t)(c.qbase + jq) * a.Hq + (size_t)kvh * a.group + iq) * D + 4 * lane;
              raw[r] = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(a.q) + base);
            }
          }
#pragma unroll
          for (int r = 0; r < RP; ++r) {
            float x[4];
            if (a.q_dtype == CUDA_LLM_F16) {
              x[0] = f16x2_lo(raw[r].x); x[1] = f16x2_hi(raw[r].x); x[2] = f16x2_lo(raw[r].y); x[3] = f16x2_hi(raw[r].y);
            } else {
              x[0] = __uint_as_float(raw[r].x << 16); x[1] = __uint_as_float(raw[r].x & 0xffff0000u);
              x[2] = __uint_as_float(raw[r].y << 16); x[3] = __uint_as_float(raw[r].y & 0xffff0000u);
            }
            float am = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            // 2^k with amax * 2^k in [128, 256): exponent field 127 + 7 - (field(amax) - 127)
            int ef = (int)((__float_as_uint(am) >> 23) & 0xffu);
            ef = min(max(ef, 16), 250);  // zero / tiny rows: a finite factor, the bytes come out as zeros anyway
            const float up = __uint_as_float((uint32_t)(261 - ef) << 23);
            const float dn = __uint_as_float((uint32_t)(ef - 7) << 23);
            uint32_t top = 0, rest = 0;
#pragma unroll
            for (int pp = 0; pp < 2; ++pp) {
              const float y0 = x[2 * pp] * up, y1 = x[2 * pp + 1] * up;
              const uint32_t t = f32x2_to_e4m3x2(y0, y1);
              const uint32_t t16 = e4m3x2_to_f16x2_lo(t);
              const uint32_t rr = f32x2_to_e4m3x2((y0 - f16x2_lo(t16)) * kResScale, (y1 - f16x2_hi(t16)) * kResScale);
              top |= t << (16 * pp);
              rest |= rr << (16 * pp);
            }
            const uint32_t off = (uint32_t)(lane >> 2) * 256 + (lane & 3) * 4;
            sts32(qbuf + off + r * 16, (int)top);
            sts32(qbuf + (NH == 1 ? (RP + r) * 16 : 2048 + r * 16) + off, (int)rest);
            if (lane == 0) qs[r] = a.scale_log2 * dn;
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(sb0 + C::kBarQReady + 8 * qb);
      }
      fresh = false;
      advance(c);
    }
    if (!ok && lane == 0) {
      atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      atomicAdd(&g_decode100_wait_timeouts, 1u);
    }
  } else if (has_work && warp == 9) {
    // =============================================================== MMA issue
    // Descriptors as 32-bit halves: the high word is a constant of the layout, the low word is
    // (address >> 4) | (leading offset >> 4) << 16 and steps by an addition.
    const uint32_t idesc_s = instr_desc_e4m3(1, 0, 128, 16);   // A = K (MN-major), B = Q (K-major)
    const uint32_t idesc_pv = instr_desc_e4m3(0, 1, 128, 16);  // A = V (K-major), B = P^T (MN-major)
    const uint32_t hi_k = ((C::kPageK >> 4) & 0x3FFFu) | (1u << 14);  // K: next 16 tokens = next page
    const uint32_t hi_q = ((128u >> 4) & 0x3FFFu) | (1u << 14);       // Q: next 8 rows
    const uint32_t hi_v = ((128u >> 4) & 0x3FFFu) | (1u << 14);       // V: next 8 head_dim rows
    const uint32_t hi_p = ((2048u >> 4) & 0x3FFFu) | (1u << 14);      // P: next 16 columns (unused at N = 16)
    uint32_t n_it = 0;
    int qb = 0;  // query buffer of the current segment (segments alternate)
    bool ok = true;
    int pv_slot = 0, pv_nv = 0, pv_fresh = 0;
    // P V of the previous stage, both heads: k-steps of 32 tokens, every variant into its accumulator
    auto issue_pv = [&](uint32_t n) -> bool {
      for (int g = 0; g < 2; ++g) {
        if (!warp_wait_relaxed(sb0 + C::kBarPFull + 8 * g, n & 1)) return false;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t vt_lo = smem_desc_lo(sb0 + C::kStages + pv_slot * C::kStageBytes + C::kOffV + g * 2048, C::kPageK);
          const uint32_t pb_lo = smem_desc_lo(sb0 + C::kP + g * C::kPBytes, 128);
          const int nk = (pv_nv + 31) >> 5;
          for (int ks = 0; ks < nk; ++ks) {
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int hh = 0; hh < NH; ++hh)
                umma_f8_parts(tmem + g * 256 + 128 + v * C::CS + hh * 16, vt_lo + ks * ((2 * C::kPageK) >> 4), hi_v,
                              pb_lo + (((v * NH + hh) * 2048 + ks * 512) >> 4), hi_p, idesc_pv, (pv_fresh && ks == 0) ? 0u : 1u);
          }
          umma_commit(sb0 + C::kBarPvDone + 8 * g);
          if (g == 1) umma_commit(empty_bar + 8 * pv_slot);
        }
        __syncwarp();
      }
      return true;
    };
    int slot = 0;
    uint32_t phase = 0;
    for (;; ++n_it, slot = (slot + 1 == NS) ? 0 : slot + 1, phase ^= (slot == 0) ? 1u : 0u) {
      if (!warp_wait(full_bar + 8 * slot, phase)) { ok = false; break; }
      const uint32_t meta = sb0 + kMetaOff + slot * (uint32_t)sizeof(StageMeta);
      const uint4 m0 = lds128(meta), m1 = lds128(meta + 16), m2 = lds128(meta + 32);
      const int flags = (int)m1.x;
      if (flags & FLAG_END) break;
      if (flags & FLAG_NEW) {
        const int segc = (int)m2.z;
        // every product issued so far, among them all with the previous segment's query operand, frees that buffer
        if (segc >= 1 && lane == 0) umma_commit(sb0 + C::kBarQFree + 8 * ((segc - 1) & 1));
        qb = segc & 1;
        if (!warp_wait(sb0 + C::kBarQReady + 8 * qb, (uint32_t)(segc >> 1) & 1)) { ok = false; break; }
      }
      // S buffer of this stage (two per group where they fit: the S of stage n is then issued as soon as its
      // data is there, not only once the group has started on stage n - 1) and the use count of that buffer
      const uint32_t sbuf = n_it % C::NSB, suse = n_it / C::NSB;
      for (int g = 0; g < 2 && ok; ++g) {
        // the previous S in this buffer has been read
        if (suse > 0 && !warp_wait(sb0 + C::kBarSFree + 8 * (2 * g + sbuf), (suse - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t kt_lo = smem_desc_lo(sb0 + C::kStages + slot * C::kStageBytes + g * 2048, 128);
          const uint32_t q_lo = smem_desc_lo(sb0 + C::kQbuf + qb * C::kQbufBytes + g * C::kQHead, 256);
#pragma unroll
          for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int hh = 0; hh < NH; ++hh)
              umma_f8_parts(tmem + g * 256 + sbuf * 64 + (MX ? b * C::CS : 0) + hh * 16, kt_lo + ((b * 512) >> 4), hi_k,
                            q_lo + ((hh * 2048 + b * 512) >> 4), hi_q, idesc_s, (MX || b == 0) ? 0u : 1u);
          umma_commit(sb0 + C::kBarSFull + 8 * (2 * g + sbuf));
        }
        __syncwarp();
      }
      if (!ok) break;
      if (n_it > 0 && !issue_pv(n_it - 1)) { ok = false; break; }
      pv_slot = slot;
      pv_nv = min(kD100Tile, (int)m0.w - (int)m0.z);
      pv_fresh = (flags & FLAG_NEW) ? 1 : 0;
    }
    if (ok && n_it > 0 && !issue_pv(n_it - 1)) ok = false;
    if (!ok && lane == 0) {
      atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      atomicAdd(&g_decode100_wait_timeouts, 1u);
    }
    // wake both groups: nothing more is coming
    if (lane == 0) {
      *done_flag = 1;
      __threadfence_block();
      for (int i = 0; i < 4; ++i) mbar_arrive(sb0 + C::kBarSFull + 8 * i);
    }
  } else if (has_work && warp < 8) {
    // =============================================================== softmax groups (one per head of the pair)
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int g = warp >> 2, gw = warp & 3;
    const int tk = gw * 32 + lane;  // token of the tile / head_dim index of the output this thread owns
    const uint32_t grp = C::kGrp + g * C::kGrpBytes;
    float* mtab = reinterpret_cast<float*>(smem + grp);            // [NVW][16] running maxima
    float* ftab = reinterpret_cast<float*>(smem + grp + 320);      // [NVW][16] rescale factors
    float* red = reinterpret_cast<float*>(smem + grp + 640);       // [4][NVW][16]
    float* sums = reinterpret_cast<float*>(smem + grp + 1920);     // [4][16]
    volatile uint32_t* flg = reinterpret_cast<volatile uint32_t*>(smem + grp + 2176);  // [4], then [4] = a wait ran out
    const uint32_t p_full = sb0 + C::kBarPFull + 8 * g, pv_done = sb0 + C::kBarPvDone + 8 * g;
    const uint32_t t_g = tmem + ((uint32_t)(gw * 32) << 16) + g * 256;
    const uint32_t t_o = t_g + 128;
    const uint32_t pbuf = sb0 + C::kP + g * C::kPBytes;
    uint32_t n_g = 0;
    float l_t[RP];
    float qsr[RP];
    uint32_t scale_range_bad = 0;
    // A wait that runs out must not make one thread leave while the others go on to a named barrier:
    // the thread records it in the group's flag and carries on (every access stays inside the CTA's
    // shared and tensor memory whatever the data is); the flag is looked at behind every named barrier,
    // where all 128 threads see the same value, and global memory is only written behind such a look.
#pragma unroll
    for (int r = 0; r < RP; ++r) l_t[r] = 0.f, qsr[r] = 0.f;
    // query token of row r (r / group), four bits per row
    unsigned long long jq_of = 0;
    for (int r = 0; r < RP; ++r) jq_of |= (unsigned long long)((r / a.group) & 15) << (4 * r);
    int slot = 0;
    uint32_t sphase = 0;
    for (;;) {
      const uint32_t sbuf = n_g % C::NSB, suse = n_g / C::NSB;
      const uint32_t s_full = sb0 + C::kBarSFull + 8 * (2 * g + sbuf), s_free = sb0 + C::kBarSFree + 8 * (2 * g + sbuf);
      const uint32_t t_s = t_g + sbuf * 64;
      if (!tc_wait_relaxed(s_full, suse & 1)) flg[4] = 1;
      const bool finished = *done_flag != 0;  // set before the arrival that ended the wait above
      if (!finished) (void)tc_wait(full_bar + 8 * slot, sphase);  // complete already: orders the reads of the stage
      tc_fence_after();
      const uint32_t meta = sb0 + kMetaOff + slot * (uint32_t)sizeof(StageMeta);
      const uint4 m0 = lds128(meta), m1 = lds128(meta + 16), m2 = lds128(meta + 32);
      const int tok0 = (int)m0.z, ctx = (int)m0.w, flags = (int)m1.x, mslot = (int)m1.y, qbase = (int)m1.z, qlen = (int)m1.w;
      const int kvh = (int)m0.y * 2 + g;
      const int R = a.group * qlen;
      const int nv = max(0, min(kD100Tile, ctx - tok0));
      const uint32_t sb = sb0 + C::kStages + slot * C::kStageBytes;
      const bool grp_new = (flags & FLAG_NEW) != 0, grp_last = (flags & FLAG_LAST) != 0;
      if (grp_new) {
        // row factors of the segment's query operand (written by the query warp before it arrived on q_ready)
        const int qbi = (int)m2.z & 1;
        if (!finished && !tc_wait(sb0 + C::kBarQReady + 8 * qbi, ((uint32_t)m2.z >> 1) & 1)) flg[4] = 1;
        const float* qs = reinterpret_cast<const float*>(smem + C::kQs + (qbi * 2 + g) * 64);
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          qsr[r] = qs[r];
          l_t[r] = 0.f;
        }
        // this thread is done with the buffer: without this arrival the query warp, released by the MMA warp
        // alone, could refill it (and complete q_ready a second time) while a group that lags two one-stage
        // segments behind had not yet waited for the first completion, which it would then never see
        if (!finished) mbar_arrive(sb0 + C::kBarQFree + 8 * qbi);
      }
      // ---- raw logits of this token: S accumulators -> x[r] (log2 domain, softmax scale applied)
      float x[RP];
      const uint32_t sc_off = (uint32_t)(tk >> 4) * 128 + g * 64;  // this token's page and head in the scale areas
      {
        float kscl[MX ? 4 : 1];
        if (MX) {
#pragma unroll
          for (int b = 0; b < 4; ++b) kscl[MX ? b : 0] = __uint_as_float(lds8(sb + C::kOffKs + sc_off + b * 16 + (tk & 15)) << 23);
        } else {
          kscl[0] = __uint_as_float(lds32(sb + C::kOffKs + sc_off + (tk & 15) * 4));
        }
#pragma unroll
        for (int r = 0; r < RP; ++r) x[r] = 0.f;
#pragma unroll
        for (int b = 0; b < (MX ? 4 : 1); ++b) {
          uint32_t sr[C::CS];
          if constexpr (C::CS == 16) tmem_ld16(t_s + b * C::CS, sr);
          else tmem_ld32(t_s + b * C::CS, sr);
          tc_wait_ld();
#pragma unroll
          for (int r = 0; r < RP; ++r)
            x[r] = fmaf(fmaf(__uint_as_float(sr[RP + r]), kResInv, __uint_as_float(sr[r])), kscl[b], x[r]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
#pragma unroll
        for (int r = 0; r < RP; ++r) x[r] *= qsr[r];
      }
      // mask: dead tokens of the tile, causal limit of a multi-token query (row r = j * group + i sees
      // positions < ctx - qlen + 1 + j)
      {
        const bool alive = tk < nv;
        const bool need_causal = (qlen > 1) && (tok0 + kD100Tile > ctx - qlen + 1);
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          bool vis = alive && r < R;
          if (need_causal) vis = vis && (tok0 + tk < ctx - qlen + 1 + (int)((jq_of >> (4 * r)) & 15));
          x[r] = vis ? x[r] : NEG_INF;
        }
      }
      // ---- exponent offsets of the variants: fp32 V scale folded in as log2, or one E8M0 exponent per block
      float woff[NV];
      float vrc = 1.f;
      if (MX) {
        const uint32_t base = sb + C::kOffVs + sc_off + (tk & 15);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          uint32_t e = lds8(base + b * 16);
          if (tk >= nv) e = 127u;
          scale_range_bad |= (e < 32u || e > 223u) ? 1u : 0u;
          woff[MX ? b : 0] = (float)((int)e - 127);
        }
      } else {
        float v = __uint_as_float(lds32(sb + C::kOffVs + sc_off + (tk & 15) * 4));
        if (tk >= nv) v = 1.f;
        v = fmaxf(v, 1e-30f);
        woff[0] = fast_log2(v);
        vrc = fast_rcp(v);
      }
      // ---- does any weight exceed its running maximum by more than 2^kLazyMax?  (The first tile of a
      // segment always takes the update path, which also initialises the maxima.)
      bool exceed = false;
      if (!grp_new) {
#pragma unroll
        for (int v = 0; v < NVW; ++v)
#pragma unroll
          for (int r4 = 0; r4 < RP / 4; ++r4) {
            const float4 m = *reinterpret_cast<const float4*>(mtab + v * 16 + 4 * r4);
            const float o = (v < NV) ? woff[v < NV ? v : 0] : 0.f;
            exceed |= (x[4 * r4] + o > m.x + kLazyMax) | (x[4 * r4 + 1] + o > m.y + kLazyMax) |
                      (x[4 * r4 + 2] + o > m.z + kLazyMax) | (x[4 * r4 + 3] + o > m.w + kLazyMax);
          }
      }
      const bool w_exceed = __any_sync(0xffffffffu, exceed);
      if (lane == 0) flg[gw] = w_exceed ? 1u : 0u;
      named_bar(1 + g, 128);
      if (*done_flag || flg[4]) break;
      const bool update = grp_new || ((flg[0] | flg[1] | flg[2] | flg[3]) != 0);
      bool pv_waited = false;
      if (update) {
        // exact tile maxima (warp reduction, then across the four warps), new running maxima, factors
#pragma unroll
        for (int v = 0; v < NVW; ++v)
#pragma unroll
          for (int r = 0; r < RP; ++r) {
            const float o = (v < NV) ? woff[v < NV ? v : 0] : 0.f;
            const float mx = warp_max(x[r] + o);
            if (lane == 0) red[(gw * NVW + v) * 16 + r] = mx;
          }
        named_bar(1 + g, 128);
        if (tk < NVW * 16 && (tk & 15) < RP) {
          const int v = tk >> 4, r = tk & 15;
          const float mx = fmaxf(fmaxf(red[(0 * NVW + v) * 16 + r], red[(1 * NVW + v) * 16 + r]),
                                 fmaxf(red[(2 * NVW + v) * 16 + r], red[(3 * NVW + v) * 16 + r]));
          const float mo = grp_new ? kMaxFloor : mtab[tk];
          const float mn = fmaxf(mo, mx);
          mtab[tk] = mn;
          ftab[tk] = fast_exp2(mo - mn);
        }
        named_bar(1 + g, 128);
        // the denominator's factor set: the last one (MX) or the only one
#pragma unroll
        for (int r = 0; r < RP; ++r) l_t[r] *= ftab[(NVW - 1) * 16 + r];
        // O of this group in TMEM: wait for its last P V, scale this thread's lane
        if (n_g > 0) {
          if (!tc_wait(pv_done, (n_g - 1) & 1)) flg[4] = 1;
          pv_waited = true;
          tc_fence_after();
          if (!grp_new) {
            const int v = MX ? gw : 0;
            uint32_t o[C::CS];
            if constexpr (C::CS == 16) tmem_ld16(t_o + v * C::CS, o);
            else tmem_ld32(t_o + v * C::CS, o);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < C::CS; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * ftab[v * 16 + (c & (RP - 1))]);  // (unused columns: any factor)
            if constexpr (C::CS == 16) tmem_st16(t_o + v * C::CS, o);
            else tmem_st32(t_o + v * C::CS, o);
            tc_wait_st();
            tc_fence_before();
          }
        }
      }
      // ---- P = 2^(w - m) per variant, denominator, E4M3 high + residual, one 16-byte store per token
      if (!pv_waited && n_g > 0) {
        if (!tc_wait(pv_done, (n_g - 1) & 1)) flg[4] = 1;  // the previous P V has read the P buffer
      }
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float p[RP];
#pragma unroll
        for (int r = 0; r < RP; ++r) p[r] = fast_exp2(x[r] + (woff[v] + kPShift) - mtab[v * 16 + r]);
        if (!MX) {
#pragma unroll
          for (int r = 0; r < RP; ++r) l_t[r] = fmaf(p[r], vrc, l_t[r]);
        }
        uint32_t top[RP / 2], rest[RP / 2];
#pragma unroll
        for (int j = 0; j < RP / 2; ++j) split_e4m3x2(p[2 * j], p[2 * j + 1], top[j], rest[j]);
        if (RP == 4) {
          // columns: high rows 0..3, residual rows 0..3, eight columns of zeros
          sts128u(pbuf + v * 2048 + tk * 16, make_uint4(top[0] | (top[1] << 16), rest[0] | (rest[1] << 16), 0u, 0u));
        } else if (RP == 8) {
          uint4 w;
          w.x = top[0] | (top[1] << 16); w.y = top[2] | (top[RP == 8 ? 3 : 0] << 16);
          w.z = rest[0] | (rest[1] << 16); w.w = rest[RP == 8 ? 2 : 0] | (rest[RP == 8 ? 3 : 0] << 16);
          sts128u(pbuf + v * 2048 + tk * 16, w);
        } else {
          uint4 w, u;
          w.x = top[0] | (top[1] << 16); w.y = top[RP == 16 ? 2 : 0] | (top[RP == 16 ? 3 : 0] << 16);
          w.z = top[RP == 16 ? 4 : 0] | (top[RP == 16 ? 5 : 0] << 16); w.w = top[RP == 16 ? 6 : 0] | (top[RP == 16 ? 7 : 0] << 16);
          u.x = rest[0] | (rest[1] << 16); u.y = rest[RP == 16 ? 2 : 0] | (rest[RP == 16 ? 3 : 0] << 16);
          u.z = rest[RP == 16 ? 4 : 0] | (rest[RP == 16 ? 5 : 0] << 16); u.w = rest[RP == 16 ? 6 : 0] | (rest[RP == 16 ? 7 : 0] << 16);
          sts128u(pbuf + (v * 2) * 2048 + tk * 16, w);
          sts128u(pbuf + (v * 2 + 1) * 2048 + tk * 16, u);
        }
      }
      if (MX) {
#pragma unroll
        for (int r = 0; r < RP; ++r) l_t[r] += fast_exp2(x[r] - mtab[(NVW - 1) * 16 + r]);
      }
      // a tile that ends inside its last 32-token step: the V bytes of the dead tokens of that step may be
      // anything (a NaN code times P = 0 is a NaN): zero them.  This thread takes head_dim row tk of its head.
      if (nv < kD100Tile) {
        const int p_lo = nv >> 4, p_hi = ((nv + 31) >> 5) << 1;  // first page with dead tokens, end of the live steps
        for (int pg = p_lo; pg < p_hi; ++pg) {
          const uint32_t addr = sb + C::kOffV + pg * C::kPageK + g * 2048 + tk * 16;
          const int keep = max(0, nv - pg * 16);  // live tokens of this page (0..15)
          uint4 w = lds128(addr);
          uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int kb = min(4, max(0, keep - 4 * j));
            ww[j] = kb >= 4 ? ww[j] : (kb == 0 ? 0u : (ww[j] & ((1u << (8 * kb)) - 1u)));
          }
          sts128u(addr, make_uint4(ww[0], ww[1], ww[2], ww[3]));
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);

      if (grp_last) {
        // ---- result of this head for the segment: O / l and the base-2 log-sum-exp into the partial slot, or
        // straight into the output when the whole segment lay in this CTA's range
        if (!tc_wait(pv_done, n_g & 1)) flg[4] = 1;
        tc_fence_after();
        const int v = MX ? gw : 0;
        uint32_t o[C::CS];
        if constexpr (C::CS == 16) tmem_ld16(t_o + v * C::CS, o);
        else tmem_ld32(t_o + v * C::CS, o);
        tc_wait_ld();
        tc_fence_before();
        float ls[RP];
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          float s = l_t[r];
#pragma unroll
          for (int of = 16; of > 0; of >>= 1) s += __shfl_xor_sync(0xffffffffu, s, of);
          ls[r] = s;
        }
        if (lane == 0) {
#pragma unroll
          for (int r = 0; r < RP; ++r) sums[gw * 16 + r] = ls[r];
        }
        named_bar(1 + g, 128);
        if (flg[4]) break;
        if (MX && scale_range_bad) {
          atomicOr(a.status, CUDA_LLM_ST_SCALE_RANGE);
          scale_range_bad = 0;
        }
        const bool direct = (flags & FLAG_DIRECT) != 0;
        const size_t prow0 = ((size_t)mslot * 2 + g) * RP;  // [slot][head of the pair][row]
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          if (r >= R) continue;
          const float l = sums[r] + sums[16 + r] + sums[32 + r] + sums[48 + r];
          const float val = fmaf(__uint_as_float(o[RP + r]), kResInv, __uint_as_float(o[r]));
          const float m_l = mtab[(NVW - 1) * 16 + r];
          // an accumulator is relative to its own running maximum (and carries 2^kPShift), the denominator
          // to the last set's (fp32 scales: the same set, and the same 2^kPShift)
          const float rel = MX ? fast_exp2(mtab[v * 16 + r] - m_l - kPShift) : 1.f;
          const float inv = (l > 0.f) ? rel * fast_rcp(l) : 0.f;
          const float lse2 = (l > 0.f) ? m_l + fast_log2(l) - (MX ? 0.f : kPShift) : NEG_INF;
          if (direct) {
            const int jq = (int)((jq_of >> (4 * r)) & 15), iq = r - jq * a.group;
            const size_t row = (size_t)(qbase + jq) * a.Hq + (size_t)kvh * a.group + iq;
            store_out_elem(a.out, a.out_dtype, row * D + tk, val * inv);
            if (a.lse && tk == r) a.lse[row] = lse2 * 0.69314718055994531f;
          } else {
            a.part_o[(prow0 + r) * D + tk] = val * inv;
            if (tk == r) a.part_lse[prow0 + r] = lse2;
          }
        }
        named_bar(1 + g, 128);  // sums[] and the tables are rewritten by the next segment
      }
      ++n_g;
      if (++slot == NS) {
        slot = 0;
        sphase ^= 1u;
      }
    }
    if (flg[4] && tk == 0) {
      atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      atomicAdd(&g_decode100_wait_timeouts, 1u);
    }
  } else if (!has_work) {
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // common exit: every warp arrives here, whatever happened, and the tensor memory goes back
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

unsigned int decode100_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_decode100_wait_timeouts, sizeof(v));
  return v;
}

template <int MODE, int RP>
static cudaError_t launch_d100(const DecodeArgs& a, int grid, cudaStream_t st) {
  using C = D100Cfg<MODE, RP>;
  auto kern = paged_decode_sm100_kernel<MODE, RP>;
  static int configured[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    if (e != cudaSuccess) return e;
    configured[dev] = 1;
  }
  DecodeArgs b = a;
  b.n_stages = C::kStagesMax;
  if (a.n_stages >= 2 && a.n_stages < b.n_stages) b.n_stages = a.n_stages;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kD100Threads);
  cfg.dynamicSmemBytes = C::kStages + (size_t)b.n_stages * C::kStageBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, b);
}

// mode: MODE_TOKEN_SCALE / MODE_MX8; rp: 4, 8 or 16 padded query rows per KV head.  `a.n_stages` > 0 caps the ring.
cudaError_t launch_paged_decode_sm100(const DecodeArgs& a, int mode, int rp, int grid, cudaStream_t st) {
  if (mode == MODE_TOKEN_SCALE)
    return rp == 4 ? launch_d100<MODE_TOKEN_SCALE, 4>(a, grid, st)
                   : rp == 8 ? launch_d100<MODE_TOKEN_SCALE, 8>(a, grid, st) : launch_d100<MODE_TOKEN_SCALE, 16>(a, grid, st);
  if (mode == MODE_MX8)
    return rp == 4 ? launch_d100<MODE_MX8, 4>(a, grid, st)
                   : rp == 8 ? launch_d100<MODE_MX8, 8>(a, grid, st) : launch_d100<MODE_MX8, 16>(a, grid, st);
  return cudaErrorInvalidValue;
}

}  // namespace b200
