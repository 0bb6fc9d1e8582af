// Paged decode attention over a quantised KV cache, sm_100a.
//
// Replaces the hot loop of the reference's fp8_paged_attention_kernel
// (fp8_paged_attention_kernel.cuh:24-151 in the reference project: one CTA per (seq, head)
// walking its pages serially, 16 of 128 threads active in QK, byte-granular strided loads)
// with a persistent, bandwidth-shaped kernel:
//
//  * Work unit = one *stage*: 32*TS consecutive tokens of one sequence for HG adjacent
//    KV heads (HG*TS = 8).  All units of the launch, in (sequence, head-group, tile) order,
//    are cut into equal contiguous ranges, one per CTA, so every SM streams the same number
//    of bytes whatever the context-length distribution is.  A sequence that straddles a cut
//    is finished by the split merge kernel.
//  * One producer warp walks the CTA's range, looks pages up in the block table and issues
//    1-D bulk (TMA) copies: per page one copy each for the K bytes, the V bytes and their
//    scales of all HG heads (contiguous in the reference layout
//    cache[num_blocks, heads, head_dim, page]).  Copies land in an NS-deep shared-memory
//    ring; full/empty mbarriers with byte counts hand stages to the consumers.
//  * Eight consumer warps; warp w owns KV head (w % HG) and the 32-token sub-tile (w / HG).
//    Per sub-tile it computes S^T[token, q] = K * Q^T and O^T[d, q] += V^T * P^T with
//    mma.sync m16n8k16 (f16 in, fp32 accumulate).  Tokens sit on the M side (always a full
//    16-row tile); the query rows (GQA group x q_len <= 8*NT) sit on the 8-wide N side.
//    E4M3 / E2M1 bytes are widened to f16 in registers (exact), fp32 per-token scales are
//    applied to the fp32 logits and folded into P, E8M0 block scales are applied to the fp32
//    partial logits (K) or to the f16 operand (V).
//  * Online softmax state (m, l) per query row lives in registers; partial results are
//    written normalised with a base-2 log-sum-exp and merged by merge_splits_kernel.
//
// Numerical notes.  E4M3 -> f16 and E2M1 -> f16 are exact.  Q is used in f16 (bf16 -> f16 is
// exact for |q| in [2^-14, 65504]); an fp32 Q is split into an f16 high and low part when
// PRECISE.  P is rounded to f16 (again hi+lo when PRECISE).  V * 2^e is formed in f16 and is
// exact for e in [-14, 7] (E4M3) or [-16, 8] (E2M1); smaller exponents flush to zero, larger
// ones overflow to inf.
#pragma once
#include "sm100_primitives.cuh"
#include "cuda_llm_b200.h"

namespace b200 {

constexpr int kConsumerWarps = 8;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 8;
constexpr int kMaxPagesPerStage = 16;
constexpr uint32_t kSmemBudget = 232448;  // 227 KB opt-in maximum per CTA

enum : int { MODE_PAGE_SCALE = 0, MODE_TOKEN_SCALE = 1, MODE_MX8 = 2, MODE_MX8K_MX4V = 3 };

enum : int { FLAG_NEW = 1, FLAG_LAST = 2, FLAG_DIRECT = 4 };

struct StageMeta {  // 32 ints
  int s, hg, tok0, ctx, flags, slot, qbase, qlen;
  int pad[8];
  int blk[kMaxPagesPerStage];
};

struct DecodeArgs {
  const void* q;
  const uint8_t* kc;
  const uint8_t* vc;
  const uint8_t* ks;
  const uint8_t* vs;
  const int32_t* bt;
  const int32_t* ctx;
  const int32_t* cuq;
  void* out;
  float* lse;
  int32_t* table;     // [S*n_hg][4] = {first cta, #ctas, direct, -}
  float* part_o;      // [slot*TS+ts][HG][rows_max][D]
  float* part_lse;    // [slot*TS+ts][HG][rows_max]   (base-2)
  uint32_t* status;
  int S, Hq, Hkv, group, max_blocks, num_blocks;
  int HG, TS, n_hg, rows_max;
  int q_dtype, out_dtype, per_block;
  float scale_log2;
  int n_stages;
  uint32_t stage_bytes, off_v, off_ks, off_vs;
  uint32_t k_page_stride, v_page_stride, ks_page_stride, vs_page_stride;  // smem, per page
  uint32_t k_chunk, v_chunk, ks_chunk, vs_chunk;                          // bytes per page copy
  uint64_t k_blk_stride, v_blk_stride, ks_blk_stride, vs_blk_stride;      // global, per block
};

__device__ __forceinline__ int eff_ctx(const DecodeArgs& a, int s, int page) {
  int c = a.ctx[s];
  long long cap = (long long)a.max_blocks * page;
  if (c > cap) {
    atomicOr(a.status, CUDA_LLM_ST_BAD_CTX);
    c = (int)cap;
  }
  return c < 0 ? 0 : c;
}
__device__ __forceinline__ void seq_q(const DecodeArgs& a, int s, int& qbase, int& qlen) {
  if (a.cuq) {
    qbase = a.cuq[s];
    qlen = a.cuq[s + 1] - qbase;
  } else {
    qbase = s;
    qlen = 1;
  }
  if (qlen < 0) qlen = 0;
  if (qlen * a.group > a.rows_max) {
    atomicOr(a.status, CUDA_LLM_ST_BAD_QLEN);
    qlen = a.rows_max / a.group;
  }
}

__device__ __forceinline__ float load_q_elem(const void* q, int dtype, size_t idx) {
  if (dtype == CUDA_LLM_F32) return reinterpret_cast<const float*>(q)[idx];
  if (dtype == CUDA_LLM_F16) return __half2float(reinterpret_cast<const __half*>(q)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[idx]);
}
__device__ __forceinline__ void store_out_elem(void* out, int dtype, size_t idx, float v) {
  if (dtype == CUDA_LLM_F32) reinterpret_cast<float*>(out)[idx] = v;
  else if (dtype == CUDA_LLM_F16) reinterpret_cast<__half*>(out)[idx] = __float2half(v);
  else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16(v);
}

// E8M0 byte pair (two 16-bit lanes holding 0..255) -> f16x2 of 2^(e-127+SHIFT), clamped to
// [2^-15 -> 0, 2^16 -> inf].
template <int SHIFT>
__device__ __forceinline__ uint32_t e8m0_pair_to_f16x2(uint32_t bytes_in_halves) {
  constexpr uint32_t LO = 112u - SHIFT;          // byte whose power of two has f16 exponent field 0
  constexpr uint32_t LO2 = LO | (LO << 16), HI2 = (LO + 31u) | ((LO + 31u) << 16);
  uint32_t x;
  asm("max.u16x2 %0, %1, %2;" : "=r"(x) : "r"(bytes_in_halves), "r"(LO2));
  asm("min.u16x2 %0, %1, %2;" : "=r"(x) : "r"(x), "r"(HI2));
  return (x - LO2) << 10;
}

// Packed E2M1 -> f16 by bit placement.  A nibble s.ee.m put at f16 bits 15 and 11..9 reads as
// the E2M1 value times 2^-14 (subnormal nibbles land on f16 subnormals, so this is exact for all
// 16 codes).  The kernel folds 2^7 into the block scale and 2^7 into the final normalisation.
// Each function turns a word of four bytes into the four f16 HIGH bytes of its low (even d) or
// high (odd d) nibbles.
constexpr int kE2M1ScaleShift = 7;
__device__ __forceinline__ uint32_t e2m1_lo_nibbles_to_f16_hi_bytes(uint32_t w) {
  return ((w << 4) & 0x80808080u) | ((w << 1) & 0x0E0E0E0Eu);
}
__device__ __forceinline__ uint32_t e2m1_hi_nibbles_to_f16_hi_bytes(uint32_t w) {
  return (w & 0x80808080u) | ((w >> 3) & 0x0E0E0E0Eu);
}

template <int D, int PAGE, int MODE, int NT, bool PRECISE>
__global__ void __launch_bounds__(kDecodeThreads, 1)
paged_decode_kernel(const __grid_constant__ DecodeArgs a) {
  constexpr int KT = D / 16;                     // k-tiles of QK  == m-tiles of PV
  constexpr bool V4 = (MODE == MODE_MX8K_MX4V);  // V stored as packed E2M1
  constexpr bool MX = (MODE == MODE_MX8 || MODE == MODE_MX8K_MX4V);
  constexpr int DV = V4 ? D / 2 : D;             // byte rows per head in the V slab
  constexpr int NB = D / 32;                     // scale blocks along head_dim
  constexpr float NEG_INF = -__builtin_huge_valf();

  extern __shared__ __align__(1024) uint8_t smem[];
  // layout: [0,64) full barriers, [64,128) empty barriers, [128,192) plan, [256, 256+NS*128) meta,
  //         then stages (1024-aligned)
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_bar = smem_base;
  const uint32_t empty_bar = smem_base + 64;
  volatile long long* plan = reinterpret_cast<volatile long long*>(smem + 128);
  StageMeta* metas = reinterpret_cast<StageMeta*>(smem + 256);
  const uint32_t stages_off = 256 + kMaxStages * sizeof(StageMeta);
  const uint32_t stage0 = smem_base + stages_off;
  long long* scan = reinterpret_cast<long long*>(smem + stages_off);  // prologue scratch (reused)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int NS = a.n_stages;
  const int TOK_STAGE = 32 * a.TS;

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(full_bar + 8 * i, 1);
      mbar_init(empty_bar + 8 * i, kConsumerWarps);
    }
    mbar_fence_init();
  }

  // ---------------------------------------------------------------- plan: equal unit ranges
  const int per = (a.S + kDecodeThreads - 1) / kDecodeThreads;
  const int s_lo = min(a.S, tid * per), s_hi = min(a.S, s_lo + per);
  long long my_units = 0;
  for (int s = s_lo; s < s_hi; ++s) {
    int qb, ql;
    seq_q(a, s, qb, ql);
    int c = eff_ctx(a, s, PAGE);
    if (ql > 0 && c > 0) my_units += (long long)((c + TOK_STAGE - 1) / TOK_STAGE) * a.n_hg;
  }
  scan[tid] = my_units;
  __syncthreads();
  if (tid == 0) {
    long long run = 0;
    for (int i = 0; i < kDecodeThreads; ++i) {
      long long v = scan[i];
      scan[i] = run;
      run += v;
    }
    plan[0] = run;
  }
  __syncthreads();
  const long long total_units = plan[0];
  const long long my_prefix = scan[tid];
  const long long per_cta = (total_units + gridDim.x - 1) / gridDim.x;
  const long long u_begin = min(total_units, (long long)blockIdx.x * per_cta);
  const long long u_end = min(total_units, u_begin + per_cta);
  if (u_begin < u_end && my_units > 0 && u_begin >= my_prefix && u_begin < my_prefix + my_units) {
    long long U = my_prefix;
    for (int s = s_lo; s < s_hi; ++s) {
      int qb, ql;
      seq_q(a, s, qb, ql);
      int c = eff_ctx(a, s, PAGE);
      long long n = (ql > 0 && c > 0) ? (long long)((c + TOK_STAGE - 1) / TOK_STAGE) * a.n_hg : 0;
      if (u_begin < U + n) {
        plan[1] = s;
        plan[2] = U;
        break;
      }
      U += n;
    }
  }
  __syncthreads();
  if (u_begin >= u_end) return;
  const int n_units = (int)(u_end - u_begin);

  if (warp == kConsumerWarps) {
    // =============================================================== producer warp
    int s = (int)plan[1];
    long long U_s = plan[2];
    int ctx_s = eff_ctx(a, s, PAGE);
    int qbase, qlen;
    seq_q(a, s, qbase, qlen);
    int tiles_s = (ctx_s + TOK_STAGE - 1) / TOK_STAGE;
    constexpr int NTYPES = (MODE == MODE_PAGE_SCALE) ? 2 : 4;
    const int PPS = (TOK_STAGE >= PAGE) ? TOK_STAGE / PAGE : 1;  // pages per stage

    auto locate = [&](long long u, int& hg, int& tile) {
      while (u - U_s >= (long long)tiles_s * a.n_hg) {
        U_s += (long long)tiles_s * a.n_hg;
        ++s;
        // skip empty sequences
        for (;;) {
          if (s >= a.S) {  // cannot happen while the plan and this walk agree; never read past the inputs
            s = a.S - 1;
            atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
            tiles_s = 1 << 24;
            break;
          }
          ctx_s = eff_ctx(a, s, PAGE);
          seq_q(a, s, qbase, qlen);
          tiles_s = (qlen > 0) ? (ctx_s + TOK_STAGE - 1) / TOK_STAGE : 0;
          if (tiles_s > 0) break;
          ++s;
        }
      }
      int local = (int)(u - U_s);
      hg = local / tiles_s;
      tile = local - hg * tiles_s;
    };
    auto load_blk = [&](int tile) -> int {
      int tok0 = tile * TOK_STAGE;
      int np = min(PPS, (ctx_s - tok0 + PAGE - 1) / PAGE);
      int b = 0;
      if (lane < np) {
        b = a.bt[(size_t)s * a.max_blocks + min(tok0 / PAGE + lane, a.max_blocks - 1)];
        if (b < 0 || b >= a.num_blocks) {
          atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
          b = 0;
        }
      }
      return b;
    };

    int hg, tile;
    locate(u_begin, hg, tile);
    int blk = load_blk(tile);
    bool ok = true;
    int issued = 0;
    for (int it = 0; it < n_units; ++it) {
      const int slot = it % NS;
      const uint32_t phase = (it / NS) & 1;
      // snapshot of the current unit
      const int c_s = s, c_hg = hg, c_tile = tile, c_ctx = ctx_s, c_tiles = tiles_s;
      const int c_qbase = qbase, c_qlen = qlen;
      const long long c_U = U_s;
      const int c_blk = blk;
      // look one unit ahead so that its block-table read overlaps the wait below
      if (it + 1 < n_units) {
        locate(u_begin + it + 1, hg, tile);
        blk = load_blk(tile);
      }
      if (it >= NS) {
        if (!mbar_wait(empty_bar + 8 * slot, phase ^ 1)) {
          ok = false;
          break;
        }
      }
      const int tok0 = c_tile * TOK_STAGE;
      const int np = min(PPS, (c_ctx - tok0 + PAGE - 1) / PAGE);
      const long long seg_first = c_U + (long long)c_hg * c_tiles;
      const int cta_first = (int)(seg_first / per_cta);
      const int cta_last = (int)((seg_first + c_tiles - 1) / per_cta);
      const bool direct = (a.TS == 1) && (cta_first == cta_last);
      const bool is_new = (it == 0) || (c_tile == 0);
      const bool is_last = (it == n_units - 1) || (c_tile == c_tiles - 1);
      StageMeta* m = metas + slot;
      if (lane == 0) {
        m->s = c_s;
        m->hg = c_hg;
        m->tok0 = tok0;
        m->ctx = c_ctx;
        m->flags = (is_new ? FLAG_NEW : 0) | (is_last ? FLAG_LAST : 0) | (direct ? FLAG_DIRECT : 0);
        m->slot = c_s * a.n_hg + c_hg + (int)blockIdx.x;
        m->qbase = c_qbase;
        m->qlen = c_qlen;
        if (c_tile == 0) {
          int32_t* t = a.table + 4 * (size_t)(c_s * a.n_hg + c_hg);
          t[0] = cta_first;
          t[1] = cta_last - cta_first + 1;
          t[2] = direct ? 1 : 0;
        }
      }
      if (lane < kMaxPagesPerStage) m->blk[lane] = c_blk;
      const uint32_t fb = full_bar + 8 * slot;
      if (lane == 0) {
        uint32_t bytes = (uint32_t)np * (a.k_chunk + a.v_chunk);
        if (NTYPES == 4) bytes += (uint32_t)np * (a.ks_chunk + a.vs_chunk);
        mbar_arrive_expect_tx(fb, bytes);
      }
      __syncwarp();
      const uint32_t sb = stage0 + slot * a.stage_bytes;
      // every lane takes part in the shuffle; only lanes with work issue a copy
      for (int base = 0; base < np * NTYPES; base += 32) {
        const int idx = base + lane;
        const int pi = (idx < np * NTYPES) ? idx % np : 0;
        const int ty = idx / np;
        const int b = __shfl_sync(0xffffffffu, c_blk, pi);
        if (idx < np * NTYPES) {
          if (ty == 0) {
            bulk_g2s(sb + pi * a.k_page_stride,
                     a.kc + (uint64_t)b * a.k_blk_stride + (uint64_t)c_hg * a.k_chunk, a.k_chunk, fb);
          } else if (ty == 1) {
            bulk_g2s(sb + a.off_v + pi * a.v_page_stride,
                     a.vc + (uint64_t)b * a.v_blk_stride + (uint64_t)c_hg * a.v_chunk, a.v_chunk, fb);
          } else if (ty == 2) {
            bulk_g2s(sb + a.off_ks + pi * a.ks_page_stride,
                     a.ks + (uint64_t)b * a.ks_blk_stride + (uint64_t)c_hg * a.ks_chunk, a.ks_chunk, fb);
          } else {
            bulk_g2s(sb + a.off_vs + pi * a.vs_page_stride,
                     a.vs + (uint64_t)b * a.vs_blk_stride + (uint64_t)c_hg * a.vs_chunk, a.vs_chunk, fb);
          }
        }
      }
      issued = it + 1;
    }
    if (!ok) {
      if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      // wait (bounded) for this warp's own copies still in flight before leaving
      for (int it = max(0, issued - NS); it < issued; ++it)
        (void)mbar_wait(full_bar + 8 * (it % NS), (it / NS) & 1);
    }
    return;
  }

  // ================================================================= consumer warps
  const int g = lane >> 2, t = lane & 3;
  const int h = warp % a.HG;      // head within the CTA's head group
  const int ts = warp / a.HG;     // 32-token sub-tile within the stage
  // K: this thread owns tokens 4g..4g+3 of the sub-tile (S^T rows g / g+8 of two m-tiles)
  const int Tk = ts * 32 + 4 * g;
  const int pik = Tk / PAGE, pok = Tk % PAGE;
  // V: this thread owns tokens 8t..8t+7 of the sub-tile (k index of the PV mma)
  const int Tv = ts * 32 + 8 * t;
  const int piv = Tv / PAGE, pov = Tv % PAGE;
  const uint32_t k_off = pik * a.k_page_stride + h * (D * PAGE) + pok + t * PAGE;
  const uint32_t v_off = a.off_v + piv * a.v_page_stride + h * (DV * PAGE) + pov + g * PAGE;
  uint32_t ks_off, vs_off;
  if (MODE == MODE_TOKEN_SCALE) {
    ks_off = a.off_ks + pik * a.ks_page_stride + (h * PAGE + pok) * 4;
    vs_off = a.off_vs + pik * a.vs_page_stride + (h * PAGE + pok) * 4;
  } else {
    ks_off = a.off_ks + pik * a.ks_page_stride + h * (NB * PAGE) + pok;  // + b*PAGE
    vs_off = a.off_vs + piv * a.vs_page_stride + h * (NB * PAGE) + pov;  // + b*PAGE
  }

  uint32_t qf[NT][KT][2];
  uint32_t ql[PRECISE ? NT : 1][PRECISE ? KT : 1][2];
  float oacc[NT][KT][4];
  float m_run[NT][2], l_run[NT][2];
  float vref = 1.f, inv_vref = 1.f;
  bool need_vref = false;
  float kscale_head = 1.f;

  for (int it = 0; it < n_units; ++it) {
    const int slot = it % NS;
    const uint32_t phase = (it / NS) & 1;
    if (!mbar_wait(full_bar + 8 * slot, phase)) {
      if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      return;
    }
    const StageMeta* mp = metas + slot;
    const int s = mp->s, hg = mp->hg, tok0 = mp->tok0, ctx = mp->ctx, flags = mp->flags;
    const int mslot = mp->slot, qbase = mp->qbase, qlen = mp->qlen;
    const int kvh = hg * a.HG + h;
    const int R = a.group * qlen;  // live query rows
    const uint32_t sb = stage0 + slot * a.stage_bytes;

    if (flags & FLAG_NEW) {
      // ---- Q fragments: B operand of S^T = K * Q^T.  k index (kt, slot sl, t) <-> d = kt*16 + sl*4 + t
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int r = nt * 8 + g;
        const bool live = r < R;
        const int j = live ? r / a.group : 0;
        const int i = live ? r - j * a.group : 0;
        const size_t base = ((size_t)(qbase + j) * a.Hq + (size_t)kvh * a.group + i) * D;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          float x[4];
#pragma unroll
          for (int sl = 0; sl < 4; ++sl)
            x[sl] = live ? load_q_elem(a.q, a.q_dtype, base + kt * 16 + sl * 4 + t) : 0.f;
          qf[nt][kt][0] = pack_f16x2(x[0], x[1]);
          qf[nt][kt][1] = pack_f16x2(x[2], x[3]);
          if (PRECISE) {
            __half2 h01 = *reinterpret_cast<__half2*>(&qf[nt][kt][0]);
            __half2 h23 = *reinterpret_cast<__half2*>(&qf[nt][kt][1]);
            ql[PRECISE ? nt : 0][PRECISE ? kt : 0][0] =
                pack_f16x2(x[0] - __low2float(h01), x[1] - __high2float(h01));
            ql[PRECISE ? nt : 0][PRECISE ? kt : 0][1] =
                pack_f16x2(x[2] - __low2float(h23), x[3] - __high2float(h23));
          }
        }
        m_run[nt][0] = m_run[nt][1] = NEG_INF;
        l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < KT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) oacc[nt][mt][c] = 0.f;
      }
      vref = 1.f;
      inv_vref = 1.f;
      need_vref = (MODE == MODE_TOKEN_SCALE) || (MODE == MODE_PAGE_SCALE);
      if (MODE == MODE_PAGE_SCALE && !a.per_block)
        kscale_head = reinterpret_cast<const float*>(a.ks)[kvh];
    }

    const int nv = min(32, ctx - tok0 - ts * 32);  // valid tokens of this warp's sub-tile
    if (nv > 0) {
      const bool tail = nv < 32;
      // causal limit: query row r = j*group + i sees positions < ctx - qlen + 1 + j
      const int pos0 = tok0 + ts * 32;                       // absolute position of sub-tile token 0
      const bool need_causal = (qlen > 1) && (pos0 + 32 > ctx - qlen + 1);

      // ------------------------------------------------------------ S^T = K * Q^T
      float sacc[NT][2][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) sacc[nt][mt][c] = 0.f;

      const uint32_t kb = sb + k_off;
#pragma unroll
      for (int b2 = 0; b2 < KT / 2; ++b2) {
        float tacc[NT][2][4];
        if (MX) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
              for (int c = 0; c < 4; ++c) tacc[nt][mt][c] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int kt = b2 * 2 + kk;
          const uint32_t w0 = lds32(kb + (kt * 16 + 0) * PAGE);
          const uint32_t w1 = lds32(kb + (kt * 16 + 4) * PAGE);
          const uint32_t w2 = lds32(kb + (kt * 16 + 8) * PAGE);
          const uint32_t w3 = lds32(kb + (kt * 16 + 12) * PAGE);
          const uint32_t x01a = prmt(w0, w1, 0x5140), x01b = prmt(w0, w1, 0x7362);
          const uint32_t x23a = prmt(w2, w3, 0x5140), x23b = prmt(w2, w3, 0x7362);
          // m-tile 0: rows g -> token 4g, g+8 -> token 4g+1 ; m-tile 1: tokens 4g+2, 4g+3
          const uint32_t a00 = e4m3x2_to_f16x2_lo(x01a), a01 = e4m3x2_to_f16x2_hi(x01a);
          const uint32_t a02 = e4m3x2_to_f16x2_lo(x23a), a03 = e4m3x2_to_f16x2_hi(x23a);
          const uint32_t a10 = e4m3x2_to_f16x2_lo(x01b), a11 = e4m3x2_to_f16x2_hi(x01b);
          const uint32_t a12 = e4m3x2_to_f16x2_lo(x23b), a13 = e4m3x2_to_f16x2_hi(x23b);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            if (MX) {
              mma_f16(tacc[nt][0], a00, a01, a02, a03, qf[nt][kt][0], qf[nt][kt][1]);
              mma_f16(tacc[nt][1], a10, a11, a12, a13, qf[nt][kt][0], qf[nt][kt][1]);
              if (PRECISE) {
                mma_f16(tacc[nt][0], a00, a01, a02, a03, ql[PRECISE ? nt : 0][PRECISE ? kt : 0][0],
                        ql[PRECISE ? nt : 0][PRECISE ? kt : 0][1]);
                mma_f16(tacc[nt][1], a10, a11, a12, a13, ql[PRECISE ? nt : 0][PRECISE ? kt : 0][0],
                        ql[PRECISE ? nt : 0][PRECISE ? kt : 0][1]);
              }
            } else {
              mma_f16(sacc[nt][0], a00, a01, a02, a03, qf[nt][kt][0], qf[nt][kt][1]);
              mma_f16(sacc[nt][1], a10, a11, a12, a13, qf[nt][kt][0], qf[nt][kt][1]);
              if (PRECISE) {
                mma_f16(sacc[nt][0], a00, a01, a02, a03, ql[PRECISE ? nt : 0][PRECISE ? kt : 0][0],
                        ql[PRECISE ? nt : 0][PRECISE ? kt : 0][1]);
                mma_f16(sacc[nt][1], a10, a11, a12, a13, ql[PRECISE ? nt : 0][PRECISE ? kt : 0][0],
                        ql[PRECISE ? nt : 0][PRECISE ? kt : 0][1]);
              }
            }
          }
        }
        if (MX) {
          const uint32_t e4 = lds32(sb + ks_off + b2 * PAGE);  // E8M0 of tokens 4g..4g+3, block b2
          float sc[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) sc[j] = e8m0_to_f32((e4 >> (8 * j)) & 0xffu);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
              for (int c = 0; c < 4; ++c)
                sacc[nt][mt][c] = fmaf(tacc[nt][mt][c], sc[2 * mt + (c >> 1)], sacc[nt][mt][c]);
        }
      }

      // ------------------------------------------------------------ scales, mask, online softmax
      float ksc[4], vsc[4];
      if (MODE == MODE_TOKEN_SCALE) {
        const uint4 kq = lds128(sb + ks_off);
        const uint4 vq = lds128(sb + vs_off);
        ksc[0] = __uint_as_float(kq.x); ksc[1] = __uint_as_float(kq.y);
        ksc[2] = __uint_as_float(kq.z); ksc[3] = __uint_as_float(kq.w);
        vsc[0] = __uint_as_float(vq.x); vsc[1] = __uint_as_float(vq.y);
        vsc[2] = __uint_as_float(vq.z); vsc[3] = __uint_as_float(vq.w);
      } else if (MODE == MODE_PAGE_SCALE) {
        float kp = kscale_head, vp = 1.f;
        if (a.per_block) {
          const int bidx = mp->blk[pik];
          kp = reinterpret_cast<const float*>(a.ks)[(size_t)bidx * a.Hkv + kvh];
          vp = reinterpret_cast<const float*>(a.vs)[(size_t)bidx * a.Hkv + kvh];
        } else {
          vp = reinterpret_cast<const float*>(a.vs)[kvh];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { ksc[j] = kp; vsc[j] = vp; }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) { ksc[j] = 1.f; vsc[j] = 1.f; }
      }
      if (need_vref) {
        // reference magnitude of the V scales of this segment: max over the first sub-tile
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = (4 * g + j < nv) ? vsc[j] : 0.f;
          mx = fmaxf(mx, (v == v && v < 3.0e38f) ? v : 0.f);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        vref = (mx > 0.f) ? mx : 1.f;
        inv_vref = 1.f / vref;
        need_vref = false;
      }

      uint32_t pb[NT][4];                 // B fragments of P^T (two PV k-tiles x {b0,b1})
      uint32_t pbl[PRECISE ? NT : 1][4];  // low parts when PRECISE
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float sv[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = 2 * mt + (c >> 1);  // token 4g + j
            float x = sacc[nt][mt][c] * (ksc[j] * a.scale_log2);
            if (tail || need_causal) {
              const int tok = 4 * g + j;
              bool vis = tok < nv;
              if (need_causal) {
                const int r = nt * 8 + 2 * t + (c & 1);
                const int jq = r / a.group;
                vis = vis && (pos0 + tok < ctx - qlen + 1 + jq);
              }
              x = vis ? x : NEG_INF;
            }
            sv[mt][c] = x;
          }
        // column (query row) maxima: columns 2t (c even) and 2t+1 (c odd)
        float mx0 = fmaxf(fmaxf(sv[0][0], sv[0][2]), fmaxf(sv[1][0], sv[1][2]));
        float mx1 = fmaxf(fmaxf(sv[0][1], sv[0][3]), fmaxf(sv[1][1], sv[1][3]));
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
        const float mu0 = (mn0 == NEG_INF) ? 0.f : mn0, mu1 = (mn1 == NEG_INF) ? 0.f : mn1;
        const float al0 = fast_exp2(m_run[nt][0] - mu0), al1 = fast_exp2(m_run[nt][1] - mu1);
        m_run[nt][0] = mn0;
        m_run[nt][1] = mn1;
        float ps0 = 0.f, ps1 = 0.f;
        float pv[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float p = fast_exp2(sv[mt][c] - ((c & 1) ? mu1 : mu0));
            if (c & 1) ps1 += p; else ps0 += p;
            float pp = p;
            if (MODE == MODE_TOKEN_SCALE || MODE == MODE_PAGE_SCALE) {
              const int j = 2 * mt + (c >> 1);
              pp = p * (vsc[j] * inv_vref);
              if (tail) pp = (4 * g + j < nv) ? pp : 0.f;   // scale of a dead slot may be NaN
            }
            pv[mt][c] = pp;
          }
        l_run[nt][0] = l_run[nt][0] * al0 + ps0;
        l_run[nt][1] = l_run[nt][1] * al1 + ps1;
        if (__any_sync(0xffffffffu, (al0 != 1.f) || (al1 != 1.f))) {
#pragma unroll
          for (int mt = 0; mt < KT; ++mt) {
            oacc[nt][mt][0] *= al0; oacc[nt][mt][1] *= al1;
            oacc[nt][mt][2] *= al0; oacc[nt][mt][3] *= al1;
          }
        }
        // P^T fragments through an 8x8 transpose of the packed accumulators
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint32_t pk = pack_f16x2(pv[mt][2 * hf], pv[mt][2 * hf + 1]);
            pb[nt][2 * mt + hf] = movmatrix_trans(pk);
            if (PRECISE) {
              __half2 hh = *reinterpret_cast<const __half2*>(&pk);
              const uint32_t lo = pack_f16x2(pv[mt][2 * hf] - __low2float(hh),
                                             pv[mt][2 * hf + 1] - __high2float(hh));
              pbl[PRECISE ? nt : 0][2 * mt + hf] = movmatrix_trans(lo);
            }
          }
      }

      // ------------------------------------------------------------ O^T += V^T * P^T
      uint32_t mask_lo = 0xffffffffu, mask_hi = 0xffffffffu;
      if (tail) {
        const int kc = max(0, min(8, nv - 8 * t));
        mask_lo = kc >= 4 ? 0xffffffffu : ((1u << (8 * kc)) - 1u);
        mask_hi = kc <= 4 ? 0u : (kc >= 8 ? 0xffffffffu : ((1u << (8 * (kc - 4))) - 1u));
      }
      const uint32_t vb = sb + v_off;
#pragma unroll
      for (int b2 = 0; b2 < KT / 2; ++b2) {
        uint32_t sp[2][2];  // [PV k-tile][a0/a2 token pair] f16x2 block scales
        if (MX) {
          uint2 e = lds64(sb + vs_off + b2 * PAGE);  // E8M0 of tokens 8t..8t+7, block b2
          if (tail) {
            e.x = (e.x & mask_lo) | (0x7f7f7f7fu & ~mask_lo);
            e.y = (e.y & mask_hi) | (0x7f7f7f7fu & ~mask_hi);
          }
          const uint32_t ya = prmt(e.x, e.y, 0x5140), yb = prmt(e.x, e.y, 0x7362);
          constexpr int SH = V4 ? kE2M1ScaleShift : 0;
          sp[0][0] = e8m0_pair_to_f16x2<SH>(prmt(ya, 0u, 0x4140));
          sp[0][1] = e8m0_pair_to_f16x2<SH>(prmt(ya, 0u, 0x4342));
          sp[1][0] = e8m0_pair_to_f16x2<SH>(prmt(yb, 0u, 0x4140));
          sp[1][1] = e8m0_pair_to_f16x2<SH>(prmt(yb, 0u, 0x4342));
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int mt = b2 * 2 + kk;
          uint32_t A0[4], A1[4];  // PV k-tile 0 / 1
          if (!V4) {
            uint2 r0 = lds64(vb + (mt * 16) * PAGE);
            uint2 r1 = lds64(vb + (mt * 16 + 8) * PAGE);
            if (tail) {
              r0.x &= mask_lo; r0.y &= mask_hi;
              r1.x &= mask_lo; r1.y &= mask_hi;
            }
            const uint32_t x0a = prmt(r0.x, r0.y, 0x5140), x0b = prmt(r0.x, r0.y, 0x7362);
            const uint32_t x1a = prmt(r1.x, r1.y, 0x5140), x1b = prmt(r1.x, r1.y, 0x7362);
            A0[0] = e4m3x2_to_f16x2_lo(x0a); A0[1] = e4m3x2_to_f16x2_lo(x1a);
            A0[2] = e4m3x2_to_f16x2_hi(x0a); A0[3] = e4m3x2_to_f16x2_hi(x1a);
            A1[0] = e4m3x2_to_f16x2_lo(x0b); A1[1] = e4m3x2_to_f16x2_lo(x1b);
            A1[2] = e4m3x2_to_f16x2_hi(x0b); A1[3] = e4m3x2_to_f16x2_hi(x1b);
          } else {
            // packed E2M1: byte row (mt*8+g) holds d = mt*16+2g (low nibble) and +1 (high nibble)
            uint2 r = lds64(vb + (mt * 8) * PAGE);
            if (tail) { r.x &= mask_lo; r.y &= mask_hi; }
            const uint32_t ex = e2m1_lo_nibbles_to_f16_hi_bytes(r.x), ey = e2m1_lo_nibbles_to_f16_hi_bytes(r.y);
            const uint32_t ox = e2m1_hi_nibbles_to_f16_hi_bytes(r.x), oy = e2m1_hi_nibbles_to_f16_hi_bytes(r.y);
            // [t0,t4,t1,t5] and [t2,t6,t3,t7] of the even-d row (g) and the odd-d row (g+8)
            const uint32_t pea = prmt(ex, ey, 0x5140), peb = prmt(ex, ey, 0x7362);
            const uint32_t poa = prmt(ox, oy, 0x5140), pob = prmt(ox, oy, 0x7362);
            // k-tile kq: a0/a1 tokens (8t+2kq, 8t+4+2kq), a2/a3 tokens (8t+2kq+1, 8t+5+2kq)
            A0[0] = prmt(pea, 0u, 0x1404); A0[1] = prmt(poa, 0u, 0x1404);
            A0[2] = prmt(pea, 0u, 0x3424); A0[3] = prmt(poa, 0u, 0x3424);
            A1[0] = prmt(peb, 0u, 0x1404); A1[1] = prmt(pob, 0u, 0x1404);
            A1[2] = prmt(peb, 0u, 0x3424); A1[3] = prmt(pob, 0u, 0x3424);
          }
          if (MX) {
            A0[0] = hmul2(A0[0], sp[0][0]); A0[1] = hmul2(A0[1], sp[0][0]);
            A0[2] = hmul2(A0[2], sp[0][1]); A0[3] = hmul2(A0[3], sp[0][1]);
            A1[0] = hmul2(A1[0], sp[1][0]); A1[1] = hmul2(A1[1], sp[1][0]);
            A1[2] = hmul2(A1[2], sp[1][1]); A1[3] = hmul2(A1[3], sp[1][1]);
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_f16(oacc[nt][mt], A0[0], A0[1], A0[2], A0[3], pb[nt][0], pb[nt][1]);
            mma_f16(oacc[nt][mt], A1[0], A1[1], A1[2], A1[3], pb[nt][2], pb[nt][3]);
            if (PRECISE) {
              mma_f16(oacc[nt][mt], A0[0], A0[1], A0[2], A0[3], pbl[PRECISE ? nt : 0][0],
                      pbl[PRECISE ? nt : 0][1]);
              mma_f16(oacc[nt][mt], A1[0], A1[1], A1[2], A1[3], pbl[PRECISE ? nt : 0][2],
                      pbl[PRECISE ? nt : 0][3]);
            }
          }
        }
      }
    }

    // stage consumed: hand the slot back before the epilogue
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + 8 * slot);

    if (flags & FLAG_LAST) {
      // ------------------------------------------------------------ epilogue of the segment
      const bool direct = (flags & FLAG_DIRECT) != 0;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          l0 += __shfl_xor_sync(0xffffffffu, l0, o);
          l1 += __shfl_xor_sync(0xffffffffu, l1, o);
        }
        // packed-E2M1 rows were accumulated at 2^-(14-kE2M1ScaleShift) of their value
        const float unit = V4 ? vref * (float)(1 << (14 - kE2M1ScaleShift)) : vref;
        const float inv0 = (l0 > 0.f) ? unit / l0 : 0.f, inv1 = (l1 > 0.f) ? unit / l1 : 0.f;
        const float lse0 = (l0 > 0.f) ? m_run[nt][0] + log2f(l0) : NEG_INF;
        const float lse1 = (l1 > 0.f) ? m_run[nt][1] + log2f(l1) : NEG_INF;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int r = nt * 8 + 2 * t + cc;
          if (r >= R) continue;
          const float inv = cc ? inv1 : inv0;
          const float lse2 = cc ? lse1 : lse0;
          const int j = r / a.group, i = r - j * a.group;
          if (direct) {
            const size_t row = (size_t)(qbase + j) * a.Hq + (size_t)kvh * a.group + i;
#pragma unroll
            for (int mt = 0; mt < KT; ++mt) {
              const int d0 = V4 ? mt * 16 + 2 * g : mt * 16 + g;
              const int d1 = V4 ? d0 + 1 : d0 + 8;
              store_out_elem(a.out, a.out_dtype, row * D + d0, oacc[nt][mt][cc] * inv);
              store_out_elem(a.out, a.out_dtype, row * D + d1, oacc[nt][mt][2 + cc] * inv);
            }
            if (a.lse && g == 0) a.lse[row] = lse2 * 0.69314718055994531f;
          } else {
            const size_t prow = (((size_t)mslot * a.TS + ts) * a.HG + h) * a.rows_max + r;
            float* po = a.part_o + prow * D;
#pragma unroll
            for (int mt = 0; mt < KT; ++mt) {
              const int d0 = V4 ? mt * 16 + 2 * g : mt * 16 + g;
              const int d1 = V4 ? d0 + 1 : d0 + 8;
              po[d0] = oacc[nt][mt][cc] * inv;
              po[d1] = oacc[nt][mt][2 + cc] * inv;
            }
            if (g == 0) a.part_lse[prow] = lse2;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Split merge: one warp per (sequence, query head); combines the partials of every CTA that
// touched the sequence (algebra of combine_softmax_state, fused_online_softmax_kernel.cuh:40-49
// in the reference project, in base 2).
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
merge_splits_kernel(const __grid_constant__ DecodeArgs a, int page) {
  const int warp_global = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (warp_global >= a.S * a.Hq) return;
  const int s = warp_global / a.Hq, qh = warp_global - s * a.Hq;
  int qbase, qlen;
  seq_q(a, s, qbase, qlen);
  if (qlen <= 0) return;
  const int ctx = eff_ctx(a, s, page);
  constexpr int VPL = D / 32;  // values per lane
  if (ctx <= 0) {
    for (int j = 0; j < qlen; ++j) {
      const size_t row = (size_t)(qbase + j) * a.Hq + qh;
#pragma unroll
      for (int v = 0; v < VPL; ++v) store_out_elem(a.out, a.out_dtype, row * D + lane * VPL + v, 0.f);
      if (a.lse && lane == 0) a.lse[row] = -__builtin_huge_valf();
    }
    return;
  }
  const int kvh = qh / a.group, i = qh - kvh * a.group;
  const int hg = kvh / a.HG, h = kvh - hg * a.HG;
  const int sh = s * a.n_hg + hg;
  const int32_t* tb = a.table + 4 * (size_t)sh;
  const int cta_first = tb[0], n_cta = tb[1], direct = tb[2];
  if (direct) return;
  const int n_parts = n_cta * a.TS;
  for (int j = 0; j < qlen; ++j) {
    const int r = j * a.group + i;
    const size_t row = (size_t)(qbase + j) * a.Hq + qh;
    float mx = -__builtin_huge_valf();
    for (int p = lane; p < n_parts; p += 32) {
      const size_t prow = (((size_t)(sh + cta_first) * a.TS + p) * a.HG + h) * a.rows_max + r;
      mx = fmaxf(mx, a.part_lse[prow]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float mu = (mx == -__builtin_huge_valf()) ? 0.f : mx;
    float acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v] = 0.f;
    float wsum = 0.f;
    for (int p = 0; p < n_parts; ++p) {
      const size_t prow = (((size_t)(sh + cta_first) * a.TS + p) * a.HG + h) * a.rows_max + r;
      const float w = fast_exp2(a.part_lse[prow] - mu);
      if (w > 0.f) {
        wsum += w;
        const float* po = a.part_o + prow * D + lane * VPL;
#pragma unroll
        for (int v = 0; v < VPL; ++v) acc[v] = fmaf(w, po[v], acc[v]);
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      store_out_elem(a.out, a.out_dtype, row * D + lane * VPL + v, acc[v] * inv);
    if (a.lse && lane == 0)
      a.lse[row] = wsum > 0.f ? (mu + log2f(wsum)) * 0.69314718055994531f : -__builtin_huge_valf();
  }
}

}  // namespace b200
