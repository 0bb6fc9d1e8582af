// Paged decode attention over a quantised KV cache, sm_100a.
//
// Replaces the hot loop of the reference's fp8_paged_attention_kernel
// (fp8_paged_attention_kernel.cuh:24-151 in the reference project: one CTA per (seq, head)
// walking its pages serially, 16 of 128 threads active in QK, byte-granular strided loads)
// with a persistent, bandwidth-shaped kernel:
//
//  * Work unit = one *stage*: TOK_STAGE consecutive tokens of one sequence for HG adjacent KV
//    heads (HG * TOK_STAGE/32 = 8).  All units of the launch, in (sequence, head-group, tile)
//    order, are cut into contiguous ranges of equal cost, one per CTA, so every SM streams the
//    same number of bytes whatever the context-length distribution is (a unit costs 1, or 2
//    where a query of 9..16 rows makes both warps of a pair compute it).  A sequence that
//    straddles a cut is finished by the split merge kernel.
//  * One producer warp walks the CTA's range.  It prefetches block-table entries several
//    stages ahead into shared memory with 4-byte cp.async, and for every stage issues 1-D bulk
//    (TMA) copies: per page one copy each for the K bytes, the V bytes and their scales of all
//    HG heads (contiguous in the reference layout cache[num_blocks, heads, head_dim, page]).
//    Copies land in an NS-deep shared-memory ring; full/empty mbarriers with byte counts hand
//    stages to the consumers.
//  * Sixteen consumer warps.  With up to 8 query rows per KV head (NT == 1) a warp owns one KV
//    head and a 16-token sub-tile; with 9..16 rows (NT == 2) a warp owns one KV head, a
//    32-token sub-tile and one half (8) of the rows.  Per sub-tile it computes
//    S^T[token, q] = K * Q^T and O^T[d, q] += V^T * P^T with mma.sync m16n8k16 (f16 in, fp32
//    accumulate).  Tokens sit on the M side (always a full 16-row tile); the query rows (GQA
//    group x q_len) sit on the 8-wide N side.  E4M3 / E2M1 bytes are widened to f16 in
//    registers (exact), fp32 per-token scales are applied to the fp32 logits and folded into P,
//    E8M0 block scales are applied to the fp32 partial logits (K) or to P (V).
//  * Online softmax state (m, l) per query row lives in registers; every warp writes its
//    result normalised, with a base-2 log-sum-exp, and merge_splits_kernel combines them.
//
// Numerical notes.  E4M3 -> f16 and E2M1 -> f16 are exact.  Q is used in f16 (bf16 -> f16 is
// exact for |q| in [2^-14, 65504]); an fp32 Q is split into an f16 high and low part when
// PRECISE.  E8M0 K scales are placed into the fp32 exponent field (byte 0 acts as 0, not 2^-127;
// byte 255 as inf, not NaN).  P is rounded to f16 (again hi+lo when PRECISE).  E8M0 V scales: the
// largest block exponent of a token, e_ref, is folded into that token's softmax exponent exactly as
// an fp32 per-token V scale is (w = s + e_ref, running maximum over w, denominator accumulates
// P * 2^-e_ref), and P is multiplied in f16 by 2^(e_b - e_ref) <= 1 per 32-element block.  Nothing
// overflows whatever the exponents are; a block more than 2^14 below the largest block of its own
// token contributes zero.  Scale bytes of live tokens outside [32, 223] (2^-95 .. 2^96) set
// CUDA_LLM_ST_SCALE_RANGE: the fp32 denominator is not guaranteed there.
#pragma once
#include "sm100_primitives.cuh"
#include "cuda_llm_b200.h"

// Diagnostics (per-CTA timestamps, copy-only / math-only runs) exist only in builds made with
// -DCUDA_LLM_DIAGNOSTICS; the shipped library compiles every such branch away.
#ifdef CUDA_LLM_DIAGNOSTICS
#define B200_DIAG(x) (x)
#else
#define B200_DIAG(x) false
#endif

namespace b200 {

constexpr int kConsumerWarps = 16;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 8;
constexpr int kMaxPagesPerStage = 16;
constexpr uint32_t kSmemBudget = 232448;  // 227 KB opt-in maximum per CTA
constexpr int kBtAhead = 8;               // block-table prefetch distance, in stages
constexpr int kBtRing = 16;               // ring slots for prefetched block-table entries
constexpr int kSegGap = 2;                // cost units charged for starting a (sequence, head group) inside a range

enum : int {
  MODE_PAGE_SCALE = 0, MODE_TOKEN_SCALE = 1, MODE_MX8 = 2, MODE_MX8K_MX4V = 3,
  MODE_KV_F16 = 4, MODE_KV_BF16 = 5,       // unquantised 16-bit paged cache (no scales)
  MODE_KV_F16_TM = 6, MODE_KV_BF16_TM = 7  // unquantised 16-bit contiguous K/V [batch, heads, seq, head_dim]
};

enum : int { FLAG_NEW = 1, FLAG_LAST = 2, FLAG_DIRECT = 4, FLAG_END = 8, FLAG_QSMEM = 16 };

struct StageMeta {  // 32 ints
  int s, hg, tok0, ctx, flags, slot, qbase, qlen;
  int pad[8];
  int blk[kMaxPagesPerStage];
};

constexpr uint32_t kMetaOff = 256;
constexpr uint32_t kBtRingOff = kMetaOff + kMaxStages * sizeof(StageMeta);
// the stages start on a 1024-byte boundary: swizzled TMA boxes repeat their pattern every 1024 bytes
constexpr uint32_t kStagesOff = (kBtRingOff + kBtRing * kMaxPagesPerStage * 4 + 1023u) / 1024u * 1024u;

// Tensor maps of a 16-bit paged cache viewed as [num_blocks][Hkv * D][page] (innermost last here, first
// in the map): pages of 32 / 64 tokens are fetched as swizzled boxes so that the eight rows an
// ldmatrix phase touches fall into different banks.  Unused (zero) for every other mode.
struct alignas(64) KvTensorMaps {
  CUtensorMap k, v;
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
  float* part_o;      // [slot*SUBS+sub][HG][rows_max][D]
  float* part_lse;    // [slot*SUBS+sub][HG][rows_max]   (base-2)
  uint32_t* status;
  int S, Hq, Hkv, group, max_blocks, num_blocks;
  int HG, SUBS, n_hg, rows_max, tok_stage;
  int q_dtype, out_dtype, per_block;
  uint32_t q_smem_off;    // shared-memory offset of the per-slot query area (0: consumers read Q from global)
  uint32_t q_smem_bytes;  // bytes of one slot's query area
  int q_smem_tokens;      // query tokens per sequence the area was sized for
  int early_plan;         // plan and first table prefetch may run before the previous kernel has finished
  int fixed_ctx;     // context length of every sequence when `ctx` is null (contiguous K/V)
  int helper_pairs;  // 16-row kernels of the 8-bit modes pair two warps on a short query (two results per sub-tile)
  int debug;  // diagnostics: bit 0 = consumers skip the math, bit 1 = producer skips the copies,
              // bit 2 = per-CTA timestamps into `trace`, bit 4 = no scale copies, bit 5 = reversed ranges
  unsigned long long* trace;  // [grid][8]: ns of kernel entry, first stage landed, last stage consumed, exit;
                              // SM id; ns of table prefetches issued, first table entry landed, first copy issued
  float scale_log2;
  int n_stages;
  int grid, n_slots;    // CTAs of the decode launch; partial-result slots in the workspace
  const float* rope_cos;     // optional rotary tables [rope_positions][D] fp32 (rotate-half convention); null: none
  const float* rope_sin;
  const int32_t* rope_pos;   // optional position of every query token [total_q]; null: ctx - q_len + j
  int rope_positions;        // rows of the tables (positions are clamped to them, with a status bit)
  int tma_box_rows;     // 16-bit pages of 32 / 64 tokens: rows (head_dim lines) per TMA box, boxes per page
  int tma_boxes;
  int short_waits;      // every mbarrier wait gives up after kShortPolls polls instead of kMaxPolls
  int stall_test;       // failure-path test: the first stage of the launch is armed but no copies are issued for it
  uint32_t stage_bytes, off_v, off_ks, off_vs;
  uint32_t k_page_stride, v_page_stride, ks_page_stride, vs_page_stride;  // smem, per page
  uint32_t k_chunk, v_chunk, ks_chunk, vs_chunk;                          // bytes per page copy
  uint64_t k_blk_stride, v_blk_stride, ks_blk_stride, vs_blk_stride;      // global, per block
};

__device__ __forceinline__ int eff_ctx(const DecodeArgs& a, int s, int page) {
  if (!a.ctx) return a.fixed_ctx;
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

__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Two E8M0 bytes (in 16-bit lanes) relative to a reference exponent -> f16x2 of
// 2^(e - e_ref + SHIFT).  `c` holds (15 + SHIFT + 256) - e_ref per lane; e <= e_ref, so the f16
// exponent field 15 + SHIFT + e - e_ref never exceeds 15 + SHIFT, and a field below 1 gives +0.
__device__ __forceinline__ uint32_t e8m0_rel_pair_to_f16x2(uint32_t bytes_in_halves, uint32_t c) {
  const uint32_t x = max_u16x2(bytes_in_halves + c, 0x01000100u);
  return (x - 0x01000100u) << 10;
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

// Walks the (sequence, head-group, tile) units of a CTA's range in order.  Positions are in cost
// units: a unit advances the position by its weight `w` (1, or 2 where both row halves of a 16-row
// kernel have to compute it), and the launch is cut into ranges of equal cost.
struct UnitCursor {
  int s, hg, tile, tiles, ctx, qbase, qlen, w;
  long long pos;        // cost position of the current unit
  long long seg_first;  // cost position of (s, hg, tile 0)
};

template <int D, int PAGE, int MODE, int NT, bool PRECISE>
__global__ void __launch_bounds__(kDecodeThreads, 1)
paged_decode_kernel(const __grid_constant__ DecodeArgs a, const __grid_constant__ KvTensorMaps tmaps) {
  constexpr int KT = D / 16;                     // k-tiles of QK  == m-tiles of PV
  constexpr bool V4 = (MODE == MODE_MX8K_MX4V);  // V stored as packed E2M1
  constexpr bool MX = (MODE == MODE_MX8 || MODE == MODE_MX8K_MX4V);
  constexpr int DV = V4 ? D / 2 : D;             // byte rows per head in the V slab
  constexpr int NB = D / 32;                     // scale blocks along head_dim
  constexpr bool KV16 = (MODE >= MODE_KV_F16);  // 2-byte elements, no scales
  constexpr bool TM = (MODE >= MODE_KV_F16_TM);  // token-major rows [token][head_dim] instead of pages [head_dim][token]
  constexpr bool BF = (MODE == MODE_KV_BF16 || MODE == MODE_KV_BF16_TM);
  // 16-bit pages of 32 / 64 tokens: rows of 64 / 128 bytes, loaded as SWIZZLE_64B / SWIZZLE_128B boxes.
  // (Pages of 16 tokens stay on 1-D bulk copies: as SWIZZLE_32B boxes of 32-byte rows they were measured
  // at 5.0 TB/s against 6.2, the tiled copy engine being slow on 32-byte lines.)
  // 8-bit pages of 64 tokens have rows of 64 bytes too (four of the eight rows of an ldmatrix phase in the same
  // banks): the same swizzled boxes.  (Rows of 32 bytes stay on bulk copies, see above; packed E2M1 V as well.)
  constexpr bool TMA3D8 = !KV16 && !V4 && PAGE == 64;
  constexpr bool TMA3D = (KV16 && !TM && PAGE >= 32) || TMA3D8;
  constexpr int EB = KV16 ? 2 : 1;               // bytes per cache element
  constexpr uint32_t SWZ_MASK = (PAGE * EB >= 128) ? 7u : 3u;  // 16-byte chunk index ^= (address >> 7) & mask
  constexpr int SUB = (KV16 || NT == 1) ? 16 : 32;  // tokens per warp sub-tile
  constexpr int MT = SUB / 16;                   // m-tiles of S^T == k-tiles of PV per sub-tile
  constexpr float NEG_INF = -__builtin_huge_valf();
  constexpr float kMaxFloor = -1.0e30f;  // running maximum before any live token

  extern __shared__ __align__(1024) uint8_t smem[];
  // layout: [0,64) full barriers, [64,128) empty barriers, [128,192) plan, [256, +8*128) stage
  //         meta, block-table prefetch ring, then the stages
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full_bar = smem_base;
  const uint32_t empty_bar = smem_base + 64;
  volatile long long* plan = reinterpret_cast<volatile long long*>(smem + 128);
  const uint32_t stage0 = smem_base + kStagesOff;
  long long* scan = reinterpret_cast<long long*>(smem + kStagesOff);  // prologue scratch (reused)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int NS = a.n_stages;
  const int TOK_STAGE = a.tok_stage;

  // Launched as a programmatic dependent: nothing a previous kernel may still be writing (query,
  // K/V, the workspace the previous merge reads) is touched before griddepcontrol.wait.  Lengths,
  // query offsets and block tables are read before it only when the caller has promised that the
  // kernel in front of this one does not write them (early_plan): the plan and the first table
  // prefetch then overlap that kernel's tail.  Our own dependent, the split merge, may be
  // scheduled from here on.
  if (!a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const bool tracing = B200_DIAG((a.debug & 4) && a.trace != nullptr);
  if (tracing && threadIdx.x == 0) a.trace[blockIdx.x * 8 + 0] = globaltimer_ns();
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
  // cost of a sequence: its units, twice for a query of 9..16 rows in the 8-bit 16-row kernels
  // (both warps of a pair then compute every stage instead of alternating)
  constexpr bool WEIGHTED = (NT == 2) && !KV16;
  auto seq_cost = [&](int s) -> long long {
    int qb, ql;
    seq_q(a, s, qb, ql);
    const int c = eff_ctx(a, s, PAGE);
    if (ql <= 0 || c <= 0) return 0;
    const int w = (WEIGHTED && a.group * ql > 8) ? 2 : 1;
    // every (sequence, head group) also costs kSegGap units up front: finishing one inside a range
    // and starting the next (epilogue, partial rows, new query rows) was measured at 3-5 us, about two
    // stages, and the CTA whose range holds two such starts otherwise finishes last
    return ((long long)((c + TOK_STAGE - 1) / TOK_STAGE) * w + kSegGap) * a.n_hg;
  };
  long long my_units = 0;
  for (int s = s_lo; s < s_hi; ++s) my_units += seq_cost(s);
  // block-wide exclusive scan of my_units: warp shuffles, then the warp totals
  long long incl = my_units;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) scan[warp] = incl;
  __syncthreads();
  long long warp_base = 0, total_units = 0;
#pragma unroll
  for (int w = 0; w < kConsumerWarps + 1; ++w) {
    const long long v = scan[w];
    if (w < warp) warp_base += v;
    total_units += v;
  }
  const long long my_prefix = warp_base + incl - my_units;
  // unit counts fit 32 bits in practice (a unit moves at least 2 KB); 64-bit division is kept as
  // the fallback only
  const bool small_units = total_units < (1ll << 31) - (long long)gridDim.x;
  // a range is never narrower than the largest unit weight, so that every CTA between the first
  // and the last one of a (sequence, head group) owns at least one of its units
  const long long per_cta = max(small_units ? (long long)(((unsigned)total_units + gridDim.x - 1) / gridDim.x)
                                            : (total_units + gridDim.x - 1) / gridDim.x,
                                (long long)(WEIGHTED ? 2 : 1));
  const int vb = B200_DIAG(a.debug & 32) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;  // diagnostics: reversed ranges
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
  if (tracing && tid == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    a.trace[blockIdx.x * 8 + 4] = smid;
  }
  if (u_begin >= u_end) {
    // no work: still wait for the kernel in front, so that this grid (and with it the split merge,
    // which waits on this grid only) never completes before that kernel has
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");
    return;
  }

  if (warp == kConsumerWarps) {
    // =============================================================== producer warp
    // Two cursors walk the CTA's unit range: the issue cursor (the stage being filled now) and
    // a prefetch cursor kBtAhead units further on, which only pulls block-table entries into a
    // small shared-memory ring with 4-byte cp.async.  The block-table read is the one dependent
    // global load on the copy path; fetching it several stages early keeps it off the critical
    // path of every stage.
    const uint64_t stream_policy = l2_policy_evict_first();  // K/V bytes are read once
    constexpr int NTYPES = (MODE == MODE_PAGE_SCALE || KV16) ? 2 : 4;
    const int PPS = (TOK_STAGE >= PAGE) ? TOK_STAGE / PAGE : 1;  // pages per stage
    auto load_seq = [&](UnitCursor& c) {
      c.ctx = eff_ctx(a, c.s, PAGE);
      seq_q(a, c.s, c.qbase, c.qlen);
      c.tiles = (c.qlen > 0) ? (c.ctx + TOK_STAGE - 1) / TOK_STAGE : 0;
      c.w = (WEIGHTED && a.group * c.qlen > 8) ? 2 : 1;
    };
    // step to the next unit (tile -> head group -> sequence)
    auto advance = [&](UnitCursor& c) {
      c.pos += c.w;
      if (c.pos >= u_end) return;  // end of this CTA's range: the cursor is not used again
      if (++c.tile < c.tiles) return;
      c.tile = 0;
      c.pos += kSegGap;  // the gap in front of the next (sequence, head group)
      if (c.pos >= u_end) return;
      c.seg_first = c.pos;
      if (++c.hg < a.n_hg) return;
      c.hg = 0;
      for (;;) {  // next sequence with work
        ++c.s;
        if (c.s >= a.S) {  // past the last sequence: the position is now the total cost, nothing follows
          c.s = a.S - 1;
          c.tiles = 0;
          return;
        }
        load_seq(c);
        if (c.tiles > 0) return;
      }
    };
    // seat on the first unit whose cost position is >= u_begin (a weight-2 unit that starts before
    // the cut belongs to the previous CTA)
    UnitCursor ic;
    ic.s = (int)plan[1];
    load_seq(ic);
    {
      // inside the sequence every head group spans kSegGap + tiles * w cost units, its units start
      // behind the gap
      const long long base = plan[2];
      const int stride = kSegGap + ic.tiles * ic.w;
      const int o = (int)(u_begin - base);
      ic.hg = o / stride;
      const int rem = o - ic.hg * stride - kSegGap;           // offset behind the gap (negative: inside it)
      ic.tile = rem <= 0 ? 0 : (rem + ic.w - 1) / ic.w;
      ic.seg_first = base + (long long)ic.hg * stride + kSegGap;
      if (ic.tile >= ic.tiles) {  // the cut fell into the last unit of this head group: start at the next one
        ic.tile = ic.tiles - 1;
        ic.pos = ic.seg_first + (long long)ic.tile * ic.w;
        advance(ic);
      } else {
        ic.pos = ic.seg_first + (long long)ic.tile * ic.w;
      }
    }
    UnitCursor pc = ic;
    const uint32_t ring = smem_base + kBtRingOff;
    int pf_done = 0;  // units whose block-table entries have been requested
    auto prefetch = [&]() {
      if (TM) return;  // contiguous K/V: no block table
      if (pc.pos < u_end) {
        const int tok0 = pc.tile * TOK_STAGE;
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
    if (!TM && pc.pos + (long long)kBtAhead * pc.w <= u_end && pc.tile + kBtAhead <= pc.tiles) {
      // common start: the first kBtAhead units are consecutive tiles of one (sequence, head group),
      // so their table entries are fetched by the lanes in parallel instead of unit by unit
      for (int idx = lane; idx < kBtAhead * PPS; idx += 32) {
        const int j = idx / PPS, pg = idx - j * PPS;
        const int tok0 = (pc.tile + j) * TOK_STAGE;
        const int np = min(PPS, (pc.ctx - tok0 + PAGE - 1) / PAGE);
        if (pg < np) {
          const int32_t* src = a.bt + (size_t)pc.s * a.max_blocks + min(tok0 / PAGE + pg, a.max_blocks - 1);
          cp_async_4(ring + ((j % kBtRing) * kMaxPagesPerStage + pg) * 4, src);
        }
      }
#pragma unroll
      for (int j = 0; j < kBtAhead; ++j) cp_async_commit();
      pf_done = kBtAhead;
      pc.tile += kBtAhead - 1;
      pc.pos += (long long)(kBtAhead - 1) * pc.w;
      advance(pc);
    } else {
      for (int j = 0; j < kBtAhead; ++j) prefetch();
    }
    if (tracing && lane == 0) a.trace[blockIdx.x * 8 + 5] = globaltimer_ns();
    if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");  // K/V, Q and the workspace from here on

    // per-segment constants of the issue cursor
    int seg_cta_first = 0, seg_n_cta = 1;
    bool seg_direct = false, seg_fresh = true;
    bool ok = true;
    int issued = 0;
    // ring slot and phase are stepped, not divided out: NS is a run-time value
    int slot = 0;
    uint32_t phase = 0;
    for (int it = 0;; ++it, slot = (slot + 1 == NS) ? 0 : slot + 1, phase ^= (slot == 0) ? 1u : 0u) {
      if (ic.pos >= u_end) {
        // terminal stage: no bytes, tells the consumers that this CTA's range is done
        if (it >= NS && !mbar_wait(empty_bar + 8 * slot, phase ^ 1, a.short_waits)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          sts128(smem_base + kMetaOff + slot * (uint32_t)sizeof(StageMeta) + 16, FLAG_END, 0, 0, 0);
          mbar_arrive_expect_tx(full_bar + 8 * slot, 0u);
        }
        break;
      }
      cp_async_wait<kBtAhead - 1>();  // the group of unit `it` has landed
      __syncwarp();
      if (tracing && it == 0 && lane == 0) a.trace[blockIdx.x * 8 + 6] = globaltimer_ns();
      if (seg_fresh || ic.tile == 0) {
        const long long seg_last = ic.seg_first + (long long)(ic.tiles - 1) * ic.w;  // its last unit
        if (small_units) {
          seg_cta_first = (int)((unsigned)ic.seg_first / (unsigned)per_cta);
          seg_n_cta = (int)((unsigned)seg_last / (unsigned)per_cta) - seg_cta_first + 1;
        } else {
          seg_cta_first = (int)(ic.seg_first / per_cta);
          seg_n_cta = (int)(seg_last / per_cta) - seg_cta_first + 1;
        }
        // direct output needs one warp per (head, row): not when two warps share the rows of a
        // short query (NT == 2 kernel, at most 8 live rows)
        seg_direct = (a.SUBS == 1) && (seg_n_cta == 1) && !(!KV16 && NT == 2 && a.group * ic.qlen <= 8);
      }
      const int tok0 = ic.tile * TOK_STAGE;
      const int np = TM ? 1 : min(PPS, (ic.ctx - tok0 + PAGE - 1) / PAGE);
      int c_blk = 0;
      if (!TM && lane < np) {
        c_blk = (int)lds32(ring + ((it % kBtRing) * kMaxPagesPerStage + lane) * 4);
        if (c_blk < 0 || c_blk >= a.num_blocks) {
          atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
          c_blk = 0;
        }
      }
      if (it >= NS) {
        if (!mbar_wait(empty_bar + 8 * slot, phase ^ 1, a.short_waits)) {
          ok = false;
          break;
        }
      }
      const bool is_new = seg_fresh || (ic.tile == 0);
      const bool is_last = (ic.pos + ic.w >= u_end) || (ic.tile == ic.tiles - 1);
      const uint32_t meta = smem_base + kMetaOff + slot * (uint32_t)sizeof(StageMeta);
      // (a sequence with more query tokens than the query area was sized for keeps the global path)
      const bool q_to_smem = a.q_smem_bytes != 0 && is_new && ic.qlen <= a.q_smem_tokens;
      if (lane == 0) {
        const int flags = (is_new ? FLAG_NEW : 0) | (is_last ? FLAG_LAST : 0) | (seg_direct ? FLAG_DIRECT : 0) |
                          (q_to_smem ? FLAG_QSMEM : 0);
        sts128(meta, ic.s, ic.hg, tok0, ic.ctx);
        sts128(meta + 16, flags, ic.s * a.n_hg + ic.hg + vb, ic.qbase, ic.qlen);
        if (ic.tile == 0) {
          int32_t* t = a.table + 4 * (size_t)(ic.s * a.n_hg + ic.hg);
          t[0] = seg_cta_first;
          t[1] = seg_n_cta;
          t[2] = seg_direct ? 1 : 0;
        }
      }
      if (MODE == MODE_PAGE_SCALE && lane < kMaxPagesPerStage) sts32(meta + 64 + 4 * lane, c_blk);
      seg_fresh = false;
      const uint32_t fb = full_bar + 8 * slot;
      // failure-path test: the bytes are announced but never sent, so the consumers' wait runs out
      // (the very first unit of the launch: its cost position is the gap in front of it)
      const bool stalled = a.stall_test && ic.pos == kSegGap;
      const bool no_copy = B200_DIAG((a.debug & 2) != 0);  // diagnostics: math on whatever shared memory holds
      // the query rows of a new (sequence, head group) travel with its first stage, so that the
      // consumers find them in shared memory instead of waiting for a global load with the ring full
      const uint32_t q_row_bytes = (uint32_t)(a.HG * a.group * D) * (a.q_dtype == CUDA_LLM_F32 ? 4u : 2u);
      const uint32_t q_bytes = (q_to_smem && !no_copy) ? (uint32_t)ic.qlen * q_row_bytes : 0u;
      if (TM) {
        // per head of the group one copy each for the K and the V rows of the live tokens of the tile
        const uint32_t bytes = (uint32_t)min(TOK_STAGE, ic.ctx - tok0) * (D * 2);
        if (lane == 0) mbar_arrive_expect_tx(fb, no_copy ? 0u : 2u * (uint32_t)a.HG * bytes + q_bytes);
        __syncwarp();
        if (!no_copy && !stalled && lane < a.HG) {
          const uint32_t sb = stage0 + slot * a.stage_bytes + lane * a.k_chunk;
          const uint64_t off = (((uint64_t)ic.s * a.Hkv + (uint64_t)ic.hg * a.HG + lane) * a.fixed_ctx + tok0) * (D * 2);
          bulk_g2s_hint(sb, a.kc + off, bytes, fb, stream_policy);
          bulk_g2s_hint(sb + a.off_v, a.vc + off, bytes, fb, stream_policy);
        }
        __syncwarp();
      } else if (lane == 0) {
        uint32_t bytes = (uint32_t)np * (a.k_chunk + a.v_chunk);
        if (NTYPES == 4 && !B200_DIAG(a.debug & 16)) bytes += (uint32_t)np * (a.ks_chunk + a.vs_chunk);
        mbar_arrive_expect_tx(fb, no_copy ? 0u : bytes + q_bytes);
      }
      __syncwarp();
      if (q_bytes != 0 && !stalled && lane < ic.qlen) {  // lane j copies the rows of query token j (contiguous over the heads of the group)
        const uint8_t* src = reinterpret_cast<const uint8_t*>(a.q) +
                             ((size_t)(ic.qbase + lane) * a.Hq + (size_t)ic.hg * a.HG * a.group) * D *
                                 (a.q_dtype == CUDA_LLM_F32 ? 4 : 2);
        bulk_g2s(smem_base + a.q_smem_off + slot * a.q_smem_bytes + lane * q_row_bytes, src, q_row_bytes, fb);
      }
      if (TMA3D && !no_copy && !stalled) {
        // lane (page, box): one swizzled box of K and one of V, tensor-map coordinates
        // {token 0, row of the head group within the block, block}
        const uint32_t sb = stage0 + slot * a.stage_bytes;
        const int pg = lane / a.tma_boxes, bx = lane - pg * a.tma_boxes;
        const int blk_pg = __shfl_sync(0xffffffffu, c_blk, pg < np ? pg : 0);
        if (pg < np) {
          const uint32_t box_bytes = (uint32_t)a.tma_box_rows * (PAGE * EB);
          const int row = ic.hg * a.HG * D + bx * a.tma_box_rows;
          tma_load_3d_hint(sb + pg * a.k_page_stride + bx * box_bytes, &tmaps.k, 0, row, blk_pg, fb, stream_policy);
          tma_load_3d_hint(sb + a.off_v + pg * a.v_page_stride + bx * box_bytes, &tmaps.v, 0, row, blk_pg, fb,
                           stream_policy);
        }
        if (TMA3D8 && NTYPES == 4 && lane < np && !B200_DIAG(a.debug & 16)) {  // the scales stay on bulk copies
          const uint64_t b = (uint64_t)c_blk;
          bulk_g2s_hint(sb + a.off_ks + lane * a.ks_page_stride, a.ks + b * a.ks_blk_stride + (uint64_t)ic.hg * a.ks_chunk,
                        a.ks_chunk, fb, stream_policy);
          bulk_g2s_hint(sb + a.off_vs + lane * a.vs_page_stride, a.vs + b * a.vs_blk_stride + (uint64_t)ic.hg * a.vs_chunk,
                        a.vs_chunk, fb, stream_policy);
        }
      } else if (!TM && !no_copy && !stalled) {
        const uint32_t sb = stage0 + slot * a.stage_bytes;
        // lane pi issues the copies of page pi
        if (lane < np) {
          const uint64_t b = (uint64_t)c_blk;
          bulk_g2s_hint(sb + lane * a.k_page_stride, a.kc + b * a.k_blk_stride + (uint64_t)ic.hg * a.k_chunk,
                   a.k_chunk, fb, stream_policy);
          bulk_g2s_hint(sb + a.off_v + lane * a.v_page_stride,
                   a.vc + b * a.v_blk_stride + (uint64_t)ic.hg * a.v_chunk, a.v_chunk, fb, stream_policy);
          if (NTYPES == 4 && !B200_DIAG(a.debug & 16)) {
            bulk_g2s_hint(sb + a.off_ks + lane * a.ks_page_stride,
                     a.ks + b * a.ks_blk_stride + (uint64_t)ic.hg * a.ks_chunk, a.ks_chunk, fb, stream_policy);
            bulk_g2s_hint(sb + a.off_vs + lane * a.vs_page_stride,
                     a.vs + b * a.vs_blk_stride + (uint64_t)ic.hg * a.vs_chunk, a.vs_chunk, fb, stream_policy);
          }
        }
      }
      if (tracing && it == 0 && lane == 0) a.trace[blockIdx.x * 8 + 7] = globaltimer_ns();
      issued = it + 1;
      prefetch();  // table entries of unit it + kBtAhead
      advance(ic);
    }
    cp_async_wait<0>();
    if (!ok) {
      if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      // wait (bounded) for this warp's own copies still in flight before leaving
      for (int it = max(0, issued - NS); it < issued; ++it)
        (void)mbar_wait(full_bar + 8 * (it % NS), (it / NS) & 1, a.short_waits);
    }
    return;
  }

  // ================================================================= consumer warps
  if (a.early_plan) asm volatile("griddepcontrol.wait;" ::: "memory");  // before any store to the workspace or out
  const int g = lane >> 2, t = lane & 3;
  // 16-bit cache: a stage holds 128 (token, head) pairs, half of the 8-bit stage.  With up to 8
  // query rows the two groups of 8 warps take alternate stages (`par`); with 9..16 rows every
  // stage is computed by both groups, one row half each.
  const int wl = (NT == 1 && !KV16) ? warp : (warp & 7);  // index among the warps that share a stage's rows
  const int nt_w = (NT == 1) ? 0 : (warp >> 3);           // which 8 query rows this warp owns
  const int par = (KV16 && NT == 1) ? (warp >> 3) : -1;   // stage parity this warp computes (-1: all)
  const int h = wl % a.HG;                       // head within the CTA's head group
  const int ts = wl / a.HG;                      // sub-tile within the stage
  const int psub = (NT == 1) ? warp / a.HG : ts;  // index of this warp's result among those of a (CTA, head)
  // Every m-tile is 16 consecutive tokens of one page: token 16*mt + 2g (+1) sits on S^T rows
  // g (g+8) of m-tile mt.  Shared-memory offsets of this thread, per m-tile:
  uint32_t k_lm[MT];   // K ldmatrix row address: lane l <-> row (32*ks + l) of the head slab
  uint32_t v_lm[MT];   // V ldmatrix row address (E4M3 V): lane l <-> row (32*dp + l)
  uint32_t ks_t[MT], vs_t[MT];    // fp32 per-token scales of tokens 2g, 2g+1
  uint32_t ks_mx[MT], vs_mx[MT];  // E8M0: K tokens 2g, 2g+1; V tokens 4t..4t+3  (+ b*PAGE)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int T = ts * SUB + 16 * mt;
    const int pi = T / PAGE, po = T % PAGE;
    k_lm[mt] = pi * a.k_page_stride + h * (D * PAGE) + lane * PAGE + po;
    v_lm[mt] = a.off_v + pi * a.v_page_stride + h * (DV * PAGE) + lane * PAGE + po;
    ks_t[mt] = a.off_ks + pi * a.ks_page_stride + (h * PAGE + po + 2 * g) * 4;
    vs_t[mt] = a.off_vs + pi * a.vs_page_stride + (h * PAGE + po + 2 * g) * 4;
    ks_mx[mt] = a.off_ks + pi * a.ks_page_stride + h * (NB * PAGE) + po + 2 * g;
    vs_mx[mt] = a.off_vs + pi * a.vs_page_stride + h * (NB * PAGE) + po + 4 * t;
    if (TM) {
      // row = token, 2*D bytes.  Thread (g,t) reads 16-byte chunks t, t+4, ... of token rows g and
      // g+8 of its sub-tile: eight consecutive head_dim values each, used as two k-tile column
      // pairs (Q.K) or, after an 8x8 transpose across the warp, as rows of O^T (P.V).
      k_lm[mt] = h * a.k_chunk + (ts * 16 + g) * (D * 2) + t * 16;
      v_lm[mt] = a.off_v + h * a.k_chunk + (ts * 16 + g) * (D * 2) + t * 16;
    } else if (KV16) {
      // row = head_dim index, 2*PAGE bytes; a 16-token m-tile is 32 bytes of a row.  Four 8x8
      // matrices per ldmatrix.x4 -- K (transposed on load): lanes 8..15 the upper 8 tokens, lanes
      // 16..31 the upper 8 head_dim rows; V: lanes 8..15 the upper 8 rows, lanes 16..31 the upper
      // 8 tokens -- so the four registers are the A fragment of mma.m16n8k16 in order.
      k_lm[mt] = pi * a.k_page_stride + h * (D * PAGE * 2) + (((lane >> 4) * 8 + (lane & 7)) * PAGE + po) * 2 +
                 ((lane >> 3) & 1) * 16;
      v_lm[mt] = a.off_v + pi * a.v_page_stride + h * (D * PAGE * 2) +
                 ((((lane >> 3) & 1) * 8 + (lane & 7)) * PAGE + po) * 2 + (lane >> 4) * 16;
      if (TMA3D) {
        // the boxes arrive swizzled: the 16-byte chunk index is XORed with the row bits of the
        // address.  Steps of 16 rows (k-tiles, m-tiles) are multiples of 1024 bytes and leave the
        // XOR term unchanged, so it is applied once here.
        k_lm[mt] ^= ((k_lm[mt] >> 7) & SWZ_MASK) << 4;
        v_lm[mt] ^= ((v_lm[mt] >> 7) & SWZ_MASK) << 4;
      }
    } else if (TMA3D8) {
      // 8-bit rows of 64 bytes, swizzled the same way; steps of 32 rows are multiples of 1024 bytes
      k_lm[mt] ^= ((k_lm[mt] >> 7) & SWZ_MASK) << 4;
      v_lm[mt] ^= ((v_lm[mt] >> 7) & SWZ_MASK) << 4;
    }
  }

  // E8M0 V scales are also read where the softmax runs: bytes of tokens 2g, 2g+1, one block per
  // thread of a quad (block t, or t & 1 when head_dim is 64), relative to vs_mx[]
  const int mx_delta = 2 * g - 4 * t + (t & (NB - 1)) * PAGE;
  uint32_t scale_range_bad = 0;  // MX: sticky, a live V scale byte outside [32, 223]

  constexpr int KS = D / 32;   // ldmatrix.x4 steps over head_dim (32 rows each)
  uint32_t qf[KT][2];
  uint32_t ql[PRECISE ? KT : 1][2];
  float oacc[KT][4];
  float m_run[2], l_run[2];
  float kscale_head = 1.f, vscale_head = 1.f;
  int kvh = 0, R = 0, qbase = 0, qlen = 0;
  bool live = false;  // this warp has query rows in the current segment
  // NT == 2 kernels: a segment with at most 8 live rows does not need two row halves; the two
  // warps of a pair then take alternate stages (all rows) instead of idling one of them
  bool helper = false;
  int rb = 0;  // first query row of this warp

  int slot = 0;
  uint32_t phase = 0;
  for (int it = 0;; ++it, slot = (slot + 1 == NS) ? 0 : slot + 1, phase ^= (slot == 0) ? 1u : 0u) {
    if (!mbar_wait(full_bar + 8 * slot, phase, a.short_waits)) {
      if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
      return;
    }
    if (tracing && it == 0 && warp == 0 && lane == 0) a.trace[blockIdx.x * 8 + 1] = globaltimer_ns();
    const uint32_t meta = smem_base + kMetaOff + slot * (uint32_t)sizeof(StageMeta);
    const uint4 m0 = lds128(meta);
    const uint4 m1 = lds128(meta + 16);
    const int hg = (int)m0.y, tok0 = (int)m0.z, ctx = (int)m0.w, flags = (int)m1.x;
    if (flags & FLAG_END) {  // the producer has no more work for this CTA
      if (tracing && warp == 0 && lane == 0) a.trace[blockIdx.x * 8 + 2] = globaltimer_ns();
      break;
    }
    const int mslot = (int)m1.y;
    const uint32_t sb = stage0 + slot * a.stage_bytes;

    if (flags & FLAG_NEW) {
      qbase = (int)m1.z;
      qlen = (int)m1.w;
      kvh = hg * a.HG + h;
      R = a.group * qlen;  // live query rows of this KV head
      helper = !KV16 && (NT == 2) && (R <= 8);
      rb = helper ? 0 : nt_w * 8;
      live = rb < R;
      // ---- Q fragments: B operand of S^T = K * Q^T, f16 pairs (d, d+1) with
      // b0: d = 16kt + 2t, b1: d = 16kt + 8 + 2t.  An fp32 Q keeps a second f16 word (PRECISE).
      const int r = rb + g;
      const bool row_live = r < R;
      const int jq = row_live ? r / a.group : 0;
      const int iq = row_live ? r - jq * a.group : 0;
      const size_t base = ((size_t)(qbase + jq) * a.Hq + (size_t)kvh * a.group + iq) * D;
      // Common case, kept small because this code runs once per (sequence, head group) and is cold
      // in the instruction cache every time: 16-bit query rows, from this slot's shared-memory area
      // when there is one, one 32-bit load and a branch-free conversion per fragment register.
      const bool q_fast = !PRECISE && a.q_dtype != CUDA_LLM_F32 && a.rope_cos == nullptr;
      if (q_fast) {
        const bool q_in_smem = (flags & FLAG_QSMEM) != 0;
        const uint32_t qrow = smem_base + a.q_smem_off + slot * a.q_smem_bytes +
                              (uint32_t)((jq * a.HG + h) * a.group + iq) * (D * 2);
        const uint32_t* qglob = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(a.q) + base);
        const bool src_f16 = (a.q_dtype == CUDA_LLM_F16);
#pragma unroll
        for (int kt = 0; kt < KT; ++kt)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int d = TM ? 8 * (t + 4 * (kt >> 1)) + 4 * (kt & 1) + 2 * hf : 16 * kt + 8 * hf + 2 * t;
            const uint32_t w = q_in_smem ? lds32(qrow + d * 2) : (row_live ? qglob[d >> 1] : 0u);
            uint32_t pk;
            if (BF) {  // bf16 operands: bf16 rows pass through, f16 rows are re-rounded
              const uint32_t conv = pack_bf16x2(f16x2_lo(w), f16x2_hi(w));
              pk = src_f16 ? conv : w;
            } else {   // f16 operands: f16 rows pass through, bf16 rows are re-rounded
              const uint32_t conv = pack_f16x2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
              pk = src_f16 ? w : conv;
            }
            qf[kt][hf] = row_live ? pk : 0u;
          }
      }
      if (!q_fast) {
        // general path: any query dtype, shared-memory or global source, optional rotary embedding
        auto load_pair = [&](int d, float& lo, float& hi) {  // elements d, d + 1 of this thread's query row
          lo = 0.f; hi = 0.f;
          if (row_live && (flags & FLAG_QSMEM)) {
            // row (jq, h, iq) of this slot's query area
            const uint32_t el = (uint32_t)((jq * a.HG + h) * a.group + iq) * D + d;
            const uint32_t qa = smem_base + a.q_smem_off + slot * a.q_smem_bytes;
            if (a.q_dtype == CUDA_LLM_F32) {
              const uint2 v = lds64(qa + el * 4);
              lo = __uint_as_float(v.x); hi = __uint_as_float(v.y);
            } else {
              const uint32_t v = lds32(qa + el * 2);
              if (a.q_dtype == CUDA_LLM_F16) { lo = f16x2_lo(v); hi = f16x2_hi(v); }
              else { lo = __uint_as_float(v << 16); hi = __uint_as_float(v & 0xffff0000u); }
            }
          } else if (row_live) {
            if (a.q_dtype == CUDA_LLM_F32) {
              const float2 v = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(a.q) + base + d);
              lo = v.x; hi = v.y;
            } else if (a.q_dtype == CUDA_LLM_F16) {
              const __half2 v = *reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(a.q) + base + d);
              lo = __low2float(v); hi = __high2float(v);
            } else {
              const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(
                  reinterpret_cast<const __nv_bfloat16*>(a.q) + base + d);
              lo = __low2float(v); hi = __high2float(v);
            }
          }
        };
        auto store_frag = [&](int kt, int hf, float lo, float hi) {
          const uint32_t pk = BF ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
          qf[kt][hf] = pk;
          if (PRECISE) ql[PRECISE ? kt : 0][hf] = pack_f16x2(lo - f16x2_lo(pk), hi - f16x2_hi(pk));
        };
        // token-major K: the thread's 16-byte chunk (t + 4*(kt/2)) holds the columns of two k-tiles
        auto frag_d = [&](int kt, int hf) {
          return TM ? 8 * (t + 4 * (kt >> 1)) + 4 * (kt & 1) + 2 * hf : 16 * kt + 8 * hf + 2 * t;
        };
        if (a.rope_cos != nullptr) {
          // Rotary embedding of the query (rotate-half: q' = q * cos + rot(q) * sin with
          // rot(q) = [-q[D/2:], q[:D/2]], fused_rope_flash_attention_kernel.cuh:56-74 in the reference
          // project), in fp32 before the rounding to the MMA operand type.  Element d and its partner
          // d + D/2 belong to k-tiles kt and kt + KT/2 of the same thread.
          int pos = a.rope_pos ? (row_live ? a.rope_pos[qbase + jq] : 0) : ctx - qlen + jq;
          if (pos < 0 || pos >= a.rope_positions) {
            if (row_live) atomicOr(a.status, CUDA_LLM_ST_BAD_POSITION);
            pos = max(0, min(pos, a.rope_positions - 1));
          }
          const float* ct = a.rope_cos + (size_t)pos * D;
          const float* st = a.rope_sin + (size_t)pos * D;
#pragma unroll
          for (int kt = 0; kt < KT / 2; ++kt)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int d = frag_d(kt, hf);
              float x0, x1, y0, y1;
              load_pair(d, x0, x1);
              load_pair(d + D / 2, y0, y1);
              const float2 c_lo = *reinterpret_cast<const float2*>(ct + d), s_lo = *reinterpret_cast<const float2*>(st + d);
              const float2 c_hi = *reinterpret_cast<const float2*>(ct + d + D / 2),
                           s_hi = *reinterpret_cast<const float2*>(st + d + D / 2);
              store_frag(kt, hf, x0 * c_lo.x - y0 * s_lo.x, x1 * c_lo.y - y1 * s_lo.y);
              store_frag(kt + KT / 2, hf, y0 * c_hi.x + x0 * s_hi.x, y1 * c_hi.y + x1 * s_hi.y);
            }
        } else {
#pragma unroll
          for (int kt = 0; kt < KT; ++kt)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              float lo, hi;
              load_pair(frag_d(kt, hf), lo, hi);
              store_frag(kt, hf, lo, hi);
            }
        }
      }
      // a finite floor instead of -inf: max - max never becomes inf - inf, no special case below
      m_run[0] = m_run[1] = kMaxFloor;
      l_run[0] = l_run[1] = 0.f;
#pragma unroll
      for (int mt = 0; mt < KT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) oacc[mt][c] = 0.f;
      if (MODE == MODE_PAGE_SCALE && !a.per_block) {
        kscale_head = reinterpret_cast<const float*>(a.ks)[kvh];
        vscale_head = reinterpret_cast<const float*>(a.vs)[kvh];
      }
    }

    const int nv = min(SUB, ctx - tok0 - ts * SUB);  // valid tokens of this warp's sub-tile
    if (nv > 0 && live && !B200_DIAG(a.debug & 1) && (par < 0 || (it & 1) == par) && (!helper || (it & 1) == nt_w)) {
      const bool tail = nv < SUB;  // masking path (dead tokens)
      // causal limit: query row r = j*group + i sees positions < ctx - qlen + 1 + j
      const int pos0 = tok0 + ts * SUB;  // absolute position of sub-tile token 0
      const bool need_causal = (qlen > 1) && (pos0 + SUB > ctx - qlen + 1);

      // ------------------------------------------------------------ S^T = K * Q^T
      // One transposed ldmatrix.x4 brings 32 head_dim rows of the 16 tokens of an m-tile; thread
      // (g,t) receives, per 8-row matrix m, the bytes K[8m+2t][2g], K[8m+2t][2g+1], K[8m+2t+1][2g],
      // K[8m+2t+1][2g+1]: after one byte shuffle the low half is the (d, d+1) pair of token 2g and
      // the high half that of token 2g+1, ready for the exact E4M3 -> f16 widening.
      float sacc[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[mt][c] = 0.f;
      if (TM) {
#pragma unroll
        for (int j = 0; j < D / 32; ++j) {
          const uint4 lo = lds128(sb + k_lm[0] + j * 64), hi = lds128(sb + k_lm[0] + 8 * (D * 2) + j * 64);
          if (BF) {
            mma_bf16(sacc[0], lo.x, hi.x, lo.y, hi.y, qf[2 * j][0], qf[2 * j][1]);
            mma_bf16(sacc[0], lo.z, hi.z, lo.w, hi.w, qf[2 * j + 1][0], qf[2 * j + 1][1]);
          } else {
            mma_f16(sacc[0], lo.x, hi.x, lo.y, hi.y, qf[2 * j][0], qf[2 * j][1]);
            mma_f16(sacc[0], lo.z, hi.z, lo.w, hi.w, qf[2 * j + 1][0], qf[2 * j + 1][1]);
          }
        }
      } else if (KV16) {
        // 16-bit K: token g (g+8) of the sub-tile on S^T rows g (g+8)
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          uint32_t r4[4];
          ldmatrix_x4_trans(r4, sb + k_lm[0] + kt * 16 * PAGE * 2);
          if (BF) mma_bf16(sacc[0], r4[0], r4[1], r4[2], r4[3], qf[kt][0], qf[kt][1]);
          else mma_f16(sacc[0], r4[0], r4[1], r4[2], r4[3], qf[kt][0], qf[kt][1]);
        }
      }
#pragma unroll
      for (int ks = 0; ks < (KV16 ? 0 : KS); ++ks) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t r4[4];
          ldmatrix_x4_trans(r4, sb + k_lm[mt] + ks * 32 * PAGE);
          float tacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            const int kt = 2 * ks + kk;
            const uint32_t x0 = prmt(r4[2 * kk], 0u, 0x3120), x1 = prmt(r4[2 * kk + 1], 0u, 0x3120);
            const uint32_t a0 = e4m3x2_to_f16x2_lo(x0), a1 = e4m3x2_to_f16x2_hi(x0);
            const uint32_t a2 = e4m3x2_to_f16x2_lo(x1), a3 = e4m3x2_to_f16x2_hi(x1);
            float (&acc)[4] = MX ? tacc : sacc[mt];
            mma_f16(acc, a0, a1, a2, a3, qf[kt][0], qf[kt][1]);
            if (PRECISE) mma_f16(acc, a0, a1, a2, a3, ql[PRECISE ? kt : 0][0], ql[PRECISE ? kt : 0][1]);
          }
          if (MX) {
            // E8M0 of tokens 2g, 2g+1, block ks, placed straight into the fp32 exponent field
            // (byte 0 reads as 0 instead of 2^-127, byte 255 as inf instead of NaN)
            const uint32_t e2 = lds16(sb + ks_mx[mt] + ks * PAGE);
            const float s0 = __uint_as_float((e2 & 0xffu) << 23), s1 = __uint_as_float((e2 << 15) & 0x7f800000u);
            sacc[mt][0] = fmaf(tacc[0], s0, sacc[mt][0]);
            sacc[mt][1] = fmaf(tacc[1], s0, sacc[mt][1]);
            sacc[mt][2] = fmaf(tacc[2], s1, sacc[mt][2]);
            sacc[mt][3] = fmaf(tacc[3], s1, sacc[mt][3]);
          }
        }
      }

      // ------------------------------------------------------------ scales, mask, online softmax
      // With fp32 V scales the scale is folded into the exponent: w = s + log2(v_scale), the running
      // maximum is taken over w, P = 2^(w - M) <= 1 multiplies the raw V codes, and the softmax
      // denominator accumulates P / v_scale.
      float ksc[MT][2], vlg[MT][2], vrc[MT][2];
      uint32_t eref[MX ? MT : 1];  // MX: reference exponents of tokens 2g | 2g+1 << 16
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (MODE == MODE_TOKEN_SCALE) {
          const uint2 kq = lds64(sb + ks_t[mt]);
          const uint2 vq = lds64(sb + vs_t[mt]);
          ksc[mt][0] = __uint_as_float(kq.x); ksc[mt][1] = __uint_as_float(kq.y);
          float v0 = __uint_as_float(vq.x), v1 = __uint_as_float(vq.y);
          if (tail) {  // a dead slot may hold anything
            v0 = (16 * mt + 2 * g < nv) ? v0 : 1.f;
            v1 = (16 * mt + 2 * g + 1 < nv) ? v1 : 1.f;
          }
          v0 = fmaxf(v0, 1e-30f); v1 = fmaxf(v1, 1e-30f);
          vlg[mt][0] = fast_log2(v0); vlg[mt][1] = fast_log2(v1);
          vrc[mt][0] = fast_rcp(v0); vrc[mt][1] = fast_rcp(v1);
        } else if (MODE == MODE_PAGE_SCALE) {
          float kp = kscale_head, vl = 0.f, vr = 1.f;
          if (a.per_block) {
            const int bidx = (int)lds32(meta + 64 + 4 * ((ts * SUB + 16 * mt) / PAGE));
            kp = reinterpret_cast<const float*>(a.ks)[(size_t)bidx * a.Hkv + kvh];
            const float vp = fmaxf(reinterpret_cast<const float*>(a.vs)[(size_t)bidx * a.Hkv + kvh], 1e-30f);
            vl = fast_log2(vp);
            vr = fast_rcp(vp);
          }
          ksc[mt][0] = ksc[mt][1] = kp;
          vlg[mt][0] = vlg[mt][1] = vl;
          vrc[mt][0] = vrc[mt][1] = vr;
        } else if (MX) {
          // reference exponent of a token = its largest V block exponent: the quad reduces the NB
          // bytes of tokens 2g (low lane) and 2g+1 (high lane)
          uint32_t em = prmt(lds16(sb + vs_mx[mt] + mx_delta), 0u, 0x4140);
          em = max_u16x2(em, __shfl_xor_sync(0xffffffffu, em, 1));
          if (NB == 4) em = max_u16x2(em, __shfl_xor_sync(0xffffffffu, em, 2));
          if (tail) {  // a dead slot may hold anything
            em = ((16 * mt + 2 * g < nv) ? (em & 0xffffu) : 127u) |
                 ((16 * mt + 2 * g + 1 < nv) ? (em & 0xffff0000u) : (127u << 16));
          }
          eref[mt] = em;
          scale_range_bad |= ((em + 0x00200020u) | (em - 0x00200020u)) & 0x01000100u;
          ksc[mt][0] = ksc[mt][1] = 1.f;
          // e - 127 as fp32 (integer in the mantissa of 2^23), 2^(127 - e) by exponent placement
          vlg[mt][0] = __uint_as_float(0x4B000000u | (em & 0xffffu)) - 8388735.f;
          vlg[mt][1] = __uint_as_float(0x4B000000u | (em >> 16)) - 8388735.f;
          vrc[mt][0] = __uint_as_float(0x7F000000u - (em << 23));
          vrc[mt][1] = __uint_as_float(0x7F000000u - ((em << 7) & 0x7F800000u));
        } else {
          ksc[mt][0] = ksc[mt][1] = 1.f;
          vlg[mt][0] = vlg[mt][1] = 0.f;
          vrc[mt][0] = vrc[mt][1] = 1.f;
        }
      }

      float sv[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = c >> 1;  // token 16*mt + 2g + j
          float xx = fmaf(sacc[mt][c], ksc[mt][j] * a.scale_log2, vlg[mt][j]);
          if (tail || need_causal) {
            const int tok = KV16 ? g + 8 * j : 16 * mt + 2 * g + j;
            bool vis = tok < nv;
            if (need_causal) {
              const int r = rb + 2 * t + (c & 1);
              const int jq = r / a.group;
              vis = vis && (pos0 + tok < ctx - qlen + 1 + jq);
            }
            xx = vis ? xx : NEG_INF;
          }
          sv[mt][c] = xx;
        }
      // column (query row) maxima: columns 2t (c even) and 2t+1 (c odd)
      float mx0 = fmaxf(sv[0][0], sv[0][2]), mx1 = fmaxf(sv[0][1], sv[0][3]);
      if (MT == 2) {
        mx0 = fmaxf(mx0, fmaxf(sv[MT - 1][0], sv[MT - 1][2]));
        mx1 = fmaxf(mx1, fmaxf(sv[MT - 1][1], sv[MT - 1][3]));
      }
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float mu0 = mn0, mu1 = mn1;
      const float al0 = fast_exp2(m_run[0] - mu0), al1 = fast_exp2(m_run[1] - mu1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      float ps0 = 0.f, ps1 = 0.f;
      float pv[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float p = fast_exp2(sv[mt][c] - ((c & 1) ? mu1 : mu0));
          const float pl = p * vrc[mt][c >> 1];
          if (c & 1) ps1 += pl; else ps0 += pl;
          pv[mt][c] = p;
        }
      l_run[0] = l_run[0] * al0 + ps0;
      l_run[1] = l_run[1] * al1 + ps1;
      if (__any_sync(0xffffffffu, (al0 != 1.f) || (al1 != 1.f))) {
#pragma unroll
        for (int mt = 0; mt < KT; ++mt) {
          oacc[mt][0] *= al0; oacc[mt][1] *= al1;
          oacc[mt][2] *= al0; oacc[mt][3] *= al1;
        }
      }

      // ------------------------------------------------------------ O^T += V^T * P^T
      // P^T through an 8x8 transpose of the packed f16 accumulators.  k index <-> token of an
      // m-tile: {4t, 4t+2} (a0/a1, b0) and {4t+1, 4t+3} (a2/a3, b1); for E4M3 V the pairs are
      // regrouped below to {4t, 4t+1} and {4t+2, 4t+3}.  One plain ldmatrix.x4 brings
      // 32 rows of V (bytes 4t..4t+3 of row 8m+g per matrix m).
      uint32_t pb[MT][2];
      uint32_t pbl[PRECISE ? MT : 1][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint32_t pk = BF ? pack_bf16x2(pv[mt][2 * hf], pv[mt][2 * hf + 1])
                                                     : pack_f16x2(pv[mt][2 * hf], pv[mt][2 * hf + 1]);
          pb[mt][hf] = movmatrix_trans(pk);
          if (PRECISE)
            pbl[PRECISE ? mt : 0][hf] = movmatrix_trans(
                pack_f16x2(pv[mt][2 * hf] - f16x2_lo(pk), pv[mt][2 * hf + 1] - f16x2_hi(pk)));
        }
      if (!V4 && !KV16) {
        // E4M3 V arrives as bytes of tokens 4t..4t+3 and is widened in adjacent pairs; regrouping P
        // to {4t, 4t+1} / {4t+2, 4t+3} here (two byte shuffles) saves one shuffle per V register
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t p0 = pb[mt][0], p1 = pb[mt][1];
          pb[mt][0] = prmt(p0, p1, 0x5410);
          pb[mt][1] = prmt(p0, p1, 0x7632);
          if (PRECISE) {
            const uint32_t q0 = pbl[PRECISE ? mt : 0][0], q1 = pbl[PRECISE ? mt : 0][1];
            pbl[PRECISE ? mt : 0][0] = prmt(q0, q1, 0x5410);
            pbl[PRECISE ? mt : 0][1] = prmt(q0, q1, 0x7632);
          }
        }
      }
      // MX: the reference exponents follow P through the same 8x8 transpose and regrouping, so that
      // they sit beside the tokens whose block scales this thread reads (E4M3 V: {4t, 4t+1} and
      // {4t+2, 4t+3}; packed E2M1 V: {4t, 4t+2} and {4t+1, 4t+3}); c = (15 + shift + 256) - e_ref
      uint32_t c02[MX ? MT : 1], c13[MX ? MT : 1];
      if (MX) {
        constexpr uint32_t kRel = (15u + (V4 ? kE2M1ScaleShift : 0) + 256u) * 0x00010001u;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t r0 = movmatrix_trans(prmt(eref[MX ? mt : 0], 0u, 0x1010));
          const uint32_t r1 = movmatrix_trans(prmt(eref[MX ? mt : 0], 0u, 0x3232));
          c02[MX ? mt : 0] = kRel - (V4 ? r0 : prmt(r0, r1, 0x5410));
          c13[MX ? mt : 0] = kRel - (V4 ? r1 : prmt(r0, r1, 0x7632));
        }
      }
      uint32_t vmask[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        vmask[mt] = 0xffffffffu;
        if (tail) {
          const int kc = max(0, min(4, nv - 16 * mt - 4 * t));
          vmask[mt] = kc >= 4 ? 0xffffffffu : ((1u << (8 * kc)) - 1u);
        }
      }
      if (KV16) {
        // 16-bit V: registers 0,1 hold tokens 2t, 2t+1 (rows g, g+8), registers 2,3 tokens 2t+8, 2t+9;
        // P^T after the transpose: b0 = tokens 2t, 2t+1, b1 = tokens 2t+8, 2t+9
        const uint32_t m_lo = (2 * t < nv ? 0xffffu : 0u) | (2 * t + 1 < nv ? 0xffff0000u : 0u);
        const uint32_t m_hi = (2 * t + 8 < nv ? 0xffffu : 0u) | (2 * t + 9 < nv ? 0xffff0000u : 0u);
        if (TM) {
          // a register of token row g holds two head_dim values; the transpose turns the 8x8 block
          // (token g, value pair of thread t) into (value, token pair 2t, 2t+1): O^T row g of m-tile
          // 2j+rp is head_dim 8*((g>>1) + 4j) + 4rp + (g&1), row g+8 that + 2
#pragma unroll
          for (int j = 0; j < D / 32; ++j) {
            const uint4 lo = lds128(sb + v_lm[0] + j * 64), hi = lds128(sb + v_lm[0] + 8 * (D * 2) + j * 64);
#pragma unroll
            for (int rp = 0; rp < 2; ++rp) {
              uint32_t va[4];
              va[0] = movmatrix_trans(rp ? lo.z : lo.x);
              va[1] = movmatrix_trans(rp ? lo.w : lo.y);
              va[2] = movmatrix_trans(rp ? hi.z : hi.x);
              va[3] = movmatrix_trans(rp ? hi.w : hi.y);
              if (tail) {
                va[0] &= m_lo; va[1] &= m_lo; va[2] &= m_hi; va[3] &= m_hi;
              }
              if (BF) mma_bf16(oacc[2 * j + rp], va[0], va[1], va[2], va[3], pb[0][0], pb[0][1]);
              else mma_f16(oacc[2 * j + rp], va[0], va[1], va[2], va[3], pb[0][0], pb[0][1]);
            }
          }
        }
#pragma unroll
        for (int mo = 0; mo < (TM ? 0 : KT); ++mo) {
          uint32_t va[4];
          ldmatrix_x4(va, sb + v_lm[0] + mo * 16 * PAGE * 2);
          if (tail) {  // a dead slot may hold a NaN pattern: 0 * NaN must not reach the accumulator
            va[0] &= m_lo; va[1] &= m_lo; va[2] &= m_hi; va[3] &= m_hi;
          }
          if (BF) mma_bf16(oacc[mo], va[0], va[1], va[2], va[3], pb[0][0], pb[0][1]);
          else mma_f16(oacc[mo], va[0], va[1], va[2], va[3], pb[0][0], pb[0][1]);
        }
      }
      constexpr int ROWS_PER_LDSM = V4 ? 64 : 32;  // head_dim rows one ldmatrix.x4 covers
#pragma unroll
      for (int dp = 0; dp < (KV16 ? 0 : D / ROWS_PER_LDSM); ++dp) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t va[4];
          ldmatrix_x4(va, sb + v_lm[mt] + dp * 32 * PAGE);
          if (tail) {  // codes of dead slots may be NaN: 0 * NaN must not reach the accumulator
            va[0] &= vmask[mt]; va[1] &= vmask[mt]; va[2] &= vmask[mt]; va[3] &= vmask[mt];
          }
          if (!V4) {
            // va[0], va[1]: rows g, g+8 of O m-tile 2dp; va[2], va[3]: of m-tile 2dp+1 (one scale block)
            uint32_t s02 = 0u, s13 = 0u;
            if (MX) {
              // E8M0 of tokens 4t..4t+3, block dp.  A dead slot may hold any byte: it takes its token's
              // reference exponent (127), or the 16-bit lane beside it would be overrun
              uint32_t e = lds32(sb + vs_mx[mt] + dp * PAGE);
              if (tail) e = (e & vmask[mt]) | (0x7f7f7f7fu & ~vmask[mt]);
              s02 = e8m0_rel_pair_to_f16x2(prmt(e, 0u, 0x4140), c02[MX ? mt : 0]);  // tokens 4t, 4t+1
              s13 = e8m0_rel_pair_to_f16x2(prmt(e, 0u, 0x4342), c13[MX ? mt : 0]);  // tokens 4t+2, 4t+3
            }
            // a block scale multiplies P (two registers per 32 head_dim rows), not the V operand
            uint32_t b0 = pb[mt][0], b1 = pb[mt][1];
            uint32_t bl0 = pbl[PRECISE ? mt : 0][0], bl1 = pbl[PRECISE ? mt : 0][1];
            if (MX) {
              b0 = hmul2(b0, s02); b1 = hmul2(b1, s13);
              if (PRECISE) { bl0 = hmul2(bl0, s02); bl1 = hmul2(bl1, s13); }
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int mo = 2 * dp + kk;
              const uint32_t x0 = va[2 * kk], x1 = va[2 * kk + 1];  // bytes of tokens 4t..4t+3, rows g and g+8
              const uint32_t A0 = e4m3x2_to_f16x2_lo(x0), A1 = e4m3x2_to_f16x2_lo(x1);
              const uint32_t A2 = e4m3x2_to_f16x2_hi(x0), A3 = e4m3x2_to_f16x2_hi(x1);
              mma_f16(oacc[mo], A0, A1, A2, A3, b0, b1);
              if (PRECISE) mma_f16(oacc[mo], A0, A1, A2, A3, bl0, bl1);
            }
          } else {
            // packed E2M1: matrix m holds byte rows 32dp + 8m + g, i.e. O m-tile 4dp + m:
            // d = 16*mo + 2g in the low nibble (row g) and d + 1 in the high nibble (row g+8);
            // m-tiles 4dp, 4dp+1 share scale block 2dp, m-tiles 4dp+2, 4dp+3 share block 2dp+1
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
              uint32_t e = lds32(sb + vs_mx[mt] + (2 * dp + bb) * PAGE);
              if (tail) e = (e & vmask[mt]) | (0x7f7f7f7fu & ~vmask[mt]);
              const uint32_t s02 = e8m0_rel_pair_to_f16x2(prmt(e, 0u, 0x4240), c02[MX ? mt : 0]);
              const uint32_t s13 = e8m0_rel_pair_to_f16x2(prmt(e, 0u, 0x4341), c13[MX ? mt : 0]);
              // the block scale multiplies P; the codes go to the tensor core as placed (value * 2^-14)
              const uint32_t b0 = hmul2(pb[mt][0], s02), b1 = hmul2(pb[mt][1], s13);
#pragma unroll
              for (int mm = 0; mm < 2; ++mm) {
                const int m = 2 * bb + mm, mo = 4 * dp + m;
                const uint32_t ex = e2m1_lo_nibbles_to_f16_hi_bytes(va[m]), ox = e2m1_hi_nibbles_to_f16_hi_bytes(va[m]);
                mma_f16(oacc[mo], prmt(ex, 0u, 0x2404), prmt(ox, 0u, 0x2404), prmt(ex, 0u, 0x3414), prmt(ox, 0u, 0x3414),
                        b0, b1);
              }
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
      if (MX && scale_range_bad) {
        atomicOr(a.status, CUDA_LLM_ST_SCALE_RANGE);
        scale_range_bad = 0;
      }
      float l0 = l_run[0], l1 = l_run[1];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
      }
      // accumulator unit: packed-E2M1 rows were accumulated at 2^-(14-kE2M1ScaleShift) of their
      // value; a per-head V scale multiplies once at the end
      float unit = V4 ? (float)(1 << (14 - kE2M1ScaleShift)) : 1.f;
      if (MODE == MODE_PAGE_SCALE && !a.per_block) unit *= vscale_head;
      // (approximate reciprocal and logarithm: relative error below 2^-22, and far less code than the
      // IEEE sequences; this path is cold in the instruction cache every time it runs)
      const float inv0 = (l0 > 0.f) ? unit * fast_rcp(l0) : 0.f, inv1 = (l1 > 0.f) ? unit * fast_rcp(l1) : 0.f;
      const float lse0 = (l0 > 0.f) ? m_run[0] + fast_log2(l0) : NEG_INF;
      const float lse1 = (l1 > 0.f) ? m_run[1] + fast_log2(l1) : NEG_INF;
      if (!direct) {
        // the usual case, kept together: normalised partial rows for the split merge
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int r = rb + 2 * t + cc;
          if (r >= R) continue;
          const float inv = cc ? inv1 : inv0;
          // a helper pair stores its second result in the unused upper rows
          const size_t prow = (((size_t)mslot * a.SUBS + psub) * a.HG + h) * a.rows_max + r + (helper ? nt_w * 8 : 0);
          float* po = a.part_o + prow * D;
#pragma unroll
          for (int mt = 0; mt < KT; ++mt) {
            const int d0 = TM ? 8 * ((g >> 1) + 4 * (mt >> 1)) + 4 * (mt & 1) + (g & 1) : V4 ? mt * 16 + 2 * g : mt * 16 + g;
            const int d1 = TM ? d0 + 2 : V4 ? d0 + 1 : d0 + 8;
            po[d0] = oacc[mt][cc] * inv;
            po[d1] = oacc[mt][2 + cc] * inv;
          }
          if (g == 0) a.part_lse[prow] = cc ? lse1 : lse0;
        }
      } else {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int r = rb + 2 * t + cc;
          if (r >= R) continue;
          const float inv = cc ? inv1 : inv0;
          const int j = r / a.group, i = r - j * a.group;
          const size_t row = (size_t)(qbase + j) * a.Hq + (size_t)kvh * a.group + i;
#pragma unroll
          for (int mt = 0; mt < KT; ++mt) {
            const int d0 = TM ? 8 * ((g >> 1) + 4 * (mt >> 1)) + 4 * (mt & 1) + (g & 1) : V4 ? mt * 16 + 2 * g : mt * 16 + g;
            const int d1 = TM ? d0 + 2 : V4 ? d0 + 1 : d0 + 8;
            store_out_elem(a.out, a.out_dtype, row * D + d0, oacc[mt][cc] * inv);
            store_out_elem(a.out, a.out_dtype, row * D + d1, oacc[mt][2 + cc] * inv);
          }
          if (a.lse && g == 0) a.lse[row] = (cc ? lse1 : lse0) * 0.69314718055994531f;
        }
      }
    }
  }
  if (tracing && warp == 0 && lane == 0) a.trace[blockIdx.x * 8 + 3] = globaltimer_ns();
}

// ------------------------------------------------------------------------------------------
// Split merge: one block of W warps per (sequence, query head, query token); the warps share the partials of every
// CTA and sub-tile warp that touched the sequence and combine them (algebra of
// combine_softmax_state, fused_online_softmax_kernel.cuh:40-49 in the reference project, in
// base 2).  Launched as a programmatic dependent of the decode kernel: blocks may start early
// and wait at griddepcontrol.wait until the decode kernel's results are visible.
// ------------------------------------------------------------------------------------------
template <int D, int W>
__global__ void __launch_bounds__(32 * W)
merge_splits_kernel(const __grid_constant__ DecodeArgs a, int page) {
  constexpr float NEG_INF = -__builtin_huge_valf();
  constexpr int VPL = D / 32;  // values per lane
  __shared__ float s_max[W];
  __shared__ float s_sum[W];
  __shared__ float s_acc[W][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x / a.Hq, qh = blockIdx.x - s * a.Hq;
  int qbase, qlen;
  seq_q(a, s, qbase, qlen);
  const int ctx = eff_ctx(a, s, page);
  const int kvh = qh / a.group, i = qh - kvh * a.group;
  const int hg = kvh / a.HG, h = kvh - hg * a.HG;
  const int sh = s * a.n_hg + hg;
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (qlen <= 0 || (int)blockIdx.y >= qlen) return;
  if (ctx <= 0) {
    if (blockIdx.y != 0) return;
    for (int j = warp; j < qlen; j += W) {
      const size_t row = (size_t)(qbase + j) * a.Hq + qh;
#pragma unroll
      for (int v = 0; v < VPL; ++v) store_out_elem(a.out, a.out_dtype, row * D + lane * VPL + v, 0.f);
      if (a.lse && lane == 0) a.lse[row] = NEG_INF;
    }
    return;
  }
  const int32_t* tb = a.table + 4 * (size_t)sh;
  int cta_first = tb[0], n_cta = tb[1];
  const int direct = tb[2];
  // An entry is written by the CTA that owns the segment's first unit.  After a wait that gave up
  // it may be missing (stale or never-initialised memory): nothing outside the partial slots is
  // read, the rows come out as zeros and the status word says so.
  const bool entry_ok = cta_first >= 0 && n_cta >= 1 && n_cta <= a.grid && cta_first <= a.grid - n_cta &&
                        (long long)sh + cta_first + n_cta <= (long long)a.n_slots;
  if (!entry_ok) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(a.status, CUDA_LLM_ST_INCOMPLETE);
    n_cta = 0;
    cta_first = 0;
  } else if (direct) {
    return;
  }
  // a 16-row kernel leaves two results per sub-tile for a query of at most 8 rows (rows r, r + 8)
  const int dup = (a.helper_pairs && a.rows_max == 16 && a.group * qlen <= 8) ? 2 : 1;
  const int n_parts = n_cta * a.SUBS * dup;
  const size_t pstride = (size_t)a.HG * a.rows_max;  // rows between consecutive sub-tile results
  auto part_row = [&](size_t row0, int p) -> size_t { return row0 + (size_t)(p / dup) * pstride + (size_t)(p % dup) * 8; };
  for (int j = (int)blockIdx.y; j < qlen; j += (int)gridDim.y) {  // blockIdx.y: a share of the query tokens
    if (j != (int)blockIdx.y) __syncthreads();                  // the shared arrays are reused
    const int r = j * a.group + i;
    const size_t row = (size_t)(qbase + j) * a.Hq + qh;
    const size_t row0 = (((size_t)(sh + cta_first) * a.SUBS) * a.HG + h) * a.rows_max + r;
    // the log-sum-exp of the first 32 * W parts is loaded once, in the lane order the weighting loop
    // below uses (warp w, lane l <-> part W * l + w), and kept for it
    const int first = W * lane + warp;
    const float lse_first = first < n_parts ? a.part_lse[part_row(row0, first)] : NEG_INF;
    float mx = lse_first;
    for (int p = 32 * W + threadIdx.x; p < n_parts; p += 32 * W) mx = fmaxf(mx, a.part_lse[part_row(row0, p)]);
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
    // warp w takes parts w, w+W, ...: weights 32 of its parts at a time (one per lane), then every
    // lane walks the rows of those parts with independent loads
    for (int base = 0; base < n_parts; base += 32 * W) {
      const int mine = base + W * lane + warp;
      const float wl = mine < n_parts ? fast_exp2((base == 0 ? lse_first : a.part_lse[part_row(row0, mine)]) - mu) : 0.f;
      const int cnt = min(32, (n_parts - base - warp + W - 1) / W);
#pragma unroll 8
      for (int jj = 0; jj < cnt; ++jj) {
        const float w = __shfl_sync(0xffffffffu, wl, jj);
        wsum += w;
        const float* po = a.part_o + part_row(row0, base + W * jj + warp) * D + lane * VPL;
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
        store_out_elem(a.out, a.out_dtype, row * D + d, sum * inv);
      }
      if (a.lse && lane == 0)
        a.lse[row] = wsum > 0.f ? (mu + log2f(wsum)) * 0.69314718055994531f : NEG_INF;
    }
  }
}

}  // namespace b200
