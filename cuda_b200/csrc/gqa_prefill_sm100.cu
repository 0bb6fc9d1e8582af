// GQA prefill attention on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// TMA (tiled, 128-byte swizzled) operand loads, mbarrier pipelines.
//
// Same contract as gqa_prefill_kernel (the reference's fused_gqa_forward, fused_gqa_kernel.cuh:22-212
// in the reference project): q [B, Hq, S, D], k / v [B, Hkv, S, D], fp16 or bf16, causal mask
// "key position <= query position", fp32 softmax.
//
// One CTA per (batch, KV head, block of query positions).  Its 128 accumulator rows are the query
// heads that share the KV head (1, 2, 4 or 8 of them) times 128 / heads consecutive query positions,
// so a K / V tile is fetched once for the whole group.  Roles:
//   warp 8        TMA producer: Q once, then K / V tiles of 128 tokens into a two-deep ring
//   warp 9        allocates TMEM, issues S = Q K^T (M 128, N 128, K 16 x D/16) into one of two S
//                 buffers in TMEM and O += P V (N = D) into the O buffer
//   warps 0..7    two threads per row = per TMEM lane (warps w and w + 4 share lane quarter w, one takes
//                 columns 0..63 of the row, the other 64..127): read their half of the S row with
//                 tcgen05.ld (one round trip), online softmax in fp32 without any shuffle (the two halves
//                 exchange their maxima through shared memory), write P (16-bit) into one of two
//                 shared-memory buffers in the swizzled K-major layout the MMA reads, rescale O in TMEM when a row maximum moved, write the output
// Shared-memory operand layouts are the canonical 128-byte-swizzle layouts of the matrix
// descriptors: K-major rows of 64 elements for Q, K and P; MN-major (row = token, 64 head_dim
// elements per 128-byte line) for V, which is exactly how a [tokens, D] tile lands through TMA.
// Every wait is bounded; a wait that runs out raises a device-side counter, lets the CTA fall
// through to the common exit (TMEM is released there) and leaves garbage in that CTA's rows.
#include "tcgen05_primitives.cuh"
#include "cuda_llm_b200.h"

namespace b200 {

struct alignas(64) PrefillMaps {
  CUtensorMap q, k, v;
};

struct Prefill100Args {
  void* out;
  int B, Hq, Hkv, S, group;
  int gsz;   // query heads per CTA (1, 2, 4 or 8; divides group)
  int causal;
  int bf16;  // operand type: 1 bf16, 0 fp16
  int out_dtype;  // CUDA_LLM_F32 / F16 / BF16 (the 16-bit types need not equal the operand type)
  float scale_log2;
};

__device__ unsigned int g_prefill_wait_timeouts = 0;

constexpr int kP100Threads = 320;  // 8 softmax warps, 1 TMA warp, 1 MMA warp
constexpr int kP100Bc = 128;  // KV tokens per tile

// 2^x for x <= 0 on the FMA / ALU pipes instead of the special-function unit, which is the busiest
// unit of the softmax warps (one MUFU.EX2 per score is as many cycles per tile as the MMAs): round x
// to the nearest integer n with the 1.5 * 2^23 trick, evaluate a cubic fit of 2^f on f = x - n in
// [-0.5, 0.5] (relative error 8e-5, below what a 16-bit P keeps), add n to the exponent field.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.f);  // masked scores (-inf) and anything below 2^-126 end up at ~1e-38
  const float r = x + 12582912.f;
  const float f = x - (r - 12582912.f);
  float p = fmaf(f, 0.05508868396282196f, 0.24260404706001282f);
  p = fmaf(f, p, 0.6932762265205383f);
  p = fmaf(f, p, 0.9999289512634277f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(r) << 23));
}

// Packed fp32 arithmetic of sm_100 (two lanes per instruction) and the three-input maximum: the softmax
// warps are bound by the number of instructions they issue per tile, and these halve the scale / subtract,
// the row sum, the polynomial and the row maximum.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.ftz.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.ftz.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.ftz.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// exp2_poly on two values at once
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  float r0, r1, t0, t1, f0, f1;
  fadd2(r0, r1, x0, x1, 12582912.f, 12582912.f);
  fadd2(t0, t1, r0, r1, -12582912.f, -12582912.f);
  ffma2(f0, f1, t0, t1, -1.f, -1.f, x0, x1);
  ffma2(p0, p1, f0, f1, 0.05508868396282196f, 0.05508868396282196f, 0.24260404706001282f, 0.24260404706001282f);
  ffma2(p0, p1, f0, f1, p0, p1, 0.6932762265205383f, 0.6932762265205383f);
  ffma2(p0, p1, f0, f1, p0, p1, 0.9999289512634277f, 0.9999289512634277f);
  p0 = __int_as_float(__float_as_int(p0) + (__float_as_int(r0) << 23));
  p1 = __int_as_float(__float_as_int(p1) + (__float_as_int(r1) << 23));
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tensor_map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kP100Threads, 1)
gqa_prefill_sm100_kernel(const __grid_constant__ Prefill100Args a, const __grid_constant__ PrefillMaps maps) {
  constexpr int NCH = D / 64;                 // 64-element (128-byte) chunks of head_dim
  constexpr uint32_t QCH = 128 * 128;         // bytes of one [128 rows x 64 elements] swizzled block
  constexpr uint32_t Q_BYTES = NCH * QCH, KV_BYTES = NCH * QCH;
  constexpr int NKV = 3;                      // K and V tiles in flight each (P lives in tensor memory)
  constexpr float NEG_INF = -__builtin_huge_valf();
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);
  const uint32_t sQ = base, sK = sQ + Q_BYTES, sV = sK + NKV * KV_BYTES;
  const uint32_t bars = sV + NKV * KV_BYTES;  // 8-byte mbarriers
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 32, k_empty = bars + 56, v_empty = bars + 80,
                 s_full = bars + 104, s_empty = bars + 120, p_full = bars + 136, pv_done = bars + 152,
                 pair_bar = bars + 168, tmem_slot = bars + 200;
  // row maxima (per tile parity, per column half) and final row sums exchanged between the two threads of a row
  float* xchg = reinterpret_cast<float*>(smem + (bars - base) + 256);  // [2 parities][2 halves][128 rows]
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - base));
  volatile uint32_t* fail_ptr = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - base) + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z;
  const int n_chunks = a.group / a.gsz;
  const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
  const int BQ = 128 / a.gsz;
  const int qt = (int)(gridDim.x - 1 - blockIdx.x);  // heavy (late) causal blocks first
  const int q0 = qt * BQ;
  const int last_q = min(a.S, q0 + BQ) - 1;
  const int n_tiles = a.causal ? last_q / kP100Bc + 1 : (a.S + kP100Bc - 1) / kP100Bc;

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NKV; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
      mbar_init(v_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + 8 * i, 1);
      mbar_init(s_empty + 8 * i, 8);   // one arrival per softmax warp
      mbar_init(p_full + 8 * i, 8);
      mbar_init(pv_done + 8 * i, 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(pair_bar + 8 * i, 2);  // the two warps that share a lane quarter
    *fail_ptr = 0;
    mbar_fence_init();
  }
  if (warp == 9) {  // TMEM: S0 [0,128), S1 [128,256), O [256, 256 + D)
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  auto give_up = [&]() {
    *fail_ptr = 1;
    atomicAdd(&g_prefill_wait_timeouts, 1u);
  };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, (uint32_t)a.gsz * BQ * D * 2);
      for (int i = 0; i < a.gsz; ++i)
        for (int c = 0; c < NCH; ++c)
          tma_load_3d(sQ + c * QCH + i * BQ * 128, &maps.q, c * 64, q0, b * a.Hq + kvh * a.group + chunk * a.gsz + i, q_full);
      int st = 0;           // ring slot of tile j and the parity of its use: j % NKV, (j / NKV) & 1
      uint32_t par = 0;
      for (int j = 0; j < n_tiles; ++j) {
        // the K slot is free as soon as the S that read it is done, the V slot only after its P V
        if (j >= NKV && !tc_wait(k_empty + 8 * st, par ^ 1)) { give_up(); break; }
        mbar_arrive_expect_tx(k_full + 8 * st, KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(sK + st * KV_BYTES + c * QCH, &maps.k, c * 64, j * kP100Bc, b * a.Hkv + kvh, k_full + 8 * st);
        if (j >= NKV && !tc_wait(v_empty + 8 * st, par ^ 1)) { give_up(); break; }
        mbar_arrive_expect_tx(v_full + 8 * st, KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(sV + st * KV_BYTES + c * QCH, &maps.v, c * 64, j * kP100Bc, b * a.Hkv + kvh, v_full + 8 * st);
        if (++st == NKV) {
          st = 0;
          par ^= 1;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc_f16(a.bf16, 0, 128, kP100Bc);
      const uint32_t idesc_o = instr_desc_f16(a.bf16, 1, 128, D);
      bool ok = tc_wait(q_full, 0);
      // descriptor halves: the high word is a constant of the layout, the low word steps by (bytes >> 4)
      const uint32_t hi_k = smem_desc_hi_sw128(1024);                       // K-major operands and V alike
      const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo = smem_desc_lo(sK, 16);
      const uint32_t v_lo = smem_desc_lo(sV, QCH);
      int vst = 0;          // V ring slot of the next P V and the parity of its use
      uint32_t vpar = 0;
      auto issue_pv = [&](int j) -> bool {  // O (+)= P_j V_j
        const int st = j & 1;
        if (!tc_wait(p_full + 8 * st, (j >> 1) & 1) || !tc_wait(v_full + 8 * vst, vpar)) return false;
        tc_fence_after();
        // P comes from tensor memory: 16 tokens of a row are 8 columns
        const uint32_t pa = tmem + 384 + st * 64, vl = v_lo + vst * (KV_BYTES >> 4);
        if (j > 0) {
#pragma unroll
          for (int kk = 0; kk < kP100Bc / 16; ++kk)
            umma_f16_ts_parts(tmem + 256, pa + kk * 8, vl + ((kk * 2048) >> 4), hi_k, idesc_o, 1u);
        } else {
#pragma unroll
          for (int kk = 0; kk < kP100Bc / 16; ++kk)
            umma_f16_ts_parts(tmem + 256, pa + kk * 8, vl + ((kk * 2048) >> 4), hi_k, idesc_o, kk > 0 ? 1u : 0u);
        }
        umma_commit(pv_done + 8 * st);   // this P buffer free, O updated
        umma_commit(v_empty + 8 * vst);  // V stage free
        if (++vst == NKV) {
          vst = 0;
          vpar ^= 1;
        }
        return true;
      };
      int kst = 0;          // K ring slot of the next S
      uint32_t kpar = 0;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j & 1;
        ok = tc_wait(k_full + 8 * kst, kpar) && (j < 2 || tc_wait(s_empty + 8 * st, ((j >> 1) - 1) & 1));
        if (!ok) break;
        tc_fence_after();
        const uint32_t kl = k_lo + kst * (KV_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * QCH + (kk & 3) * 32) >> 4;
          umma_f16_parts(tmem + st * 128, q_lo + off, hi_k, kl + off, hi_k, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full + 8 * st);
        umma_commit(k_empty + 8 * kst);  // K stage free once S is done
        if (++kst == NKV) {
          kst = 0;
          kpar ^= 1;
        }
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok) ok = issue_pv(n_tiles - 1);
      if (!ok) give_up();
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: two threads per row
    const int row = tid & 127, half = tid >> 7;  // TMEM lane; which 64 columns of S / which half of O
    const int quarter = warp & 3;
    const int hi = row / BQ, qpos = q0 + row - hi * BQ;
    const int qh = kvh * a.group + chunk * a.gsz + hi;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    constexpr int OC = D / 2;                     // O columns of this thread
    float m_run = -1.0e30f, l_run = 0.f;
    bool ok = true;
    uint32_t pair_phase = 0;
    // both warps of a quarter: write, then meet (bounded) before reading the other's values
    auto pair_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(pair_bar + 8 * quarter);
      const bool done = tc_wait(pair_bar + 8 * quarter, pair_phase);
      pair_phase ^= 1;
      return done;
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1, kv0 = j * kP100Bc;
      if (!tc_wait(s_full + 8 * st, (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (kv0 + kP100Bc > a.S) || (a.causal && kv0 + kP100Bc - 1 > q0);
      // this thread's half of the S row in one TMEM round trip
      uint32_t sr[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld32(tmem + lane_base + st * 128 + half * 64 + c * 32, sr[c]);
      tc_wait_ld();
      // S buffer consumed: the next-but-one S may be issued into it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + 8 * st);
      if (need_mask) {  // diagonal / last tile only
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kv0 + half * 64 + c * 32 + i;
            if (key >= a.S || (a.causal && key > qpos)) sr[c][i] = __float_as_uint(NEG_INF);
          }
      }
      // row maximum of the raw scores with eight independent chains (the softmax scale is positive),
      // then the maximum of the other half of the row
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = NEG_INF;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx8[(i >> 1) & 7] = fmax3(mx8[(i >> 1) & 7], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
      float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      xchg[(st * 2 + half) * 128 + row] = mx;
      if (!pair_sync()) { ok = false; break; }
      mx = fmaxf(mx, xchg[(st * 2 + (half ^ 1)) * 128 + row]);
      // The reference maximum of a row only moves when the tile exceeds it by more than 2^8: P = 2^(s - m)
      // then stays below 256 (exact in 16 bits as far as its rounding goes, harmless in the fp32 sums), and O
      // in tensor memory is rescaled in the first tile or two of a row instead of whenever a maximum creeps up.
      const float m_tile = mx * a.scale_log2;
      const float m_new = (m_tile > m_run + 8.f) ? m_tile : m_run;
      const float alpha = fast_exp2(m_run - m_new);
      m_run = m_new;
      // O is rescaled only when a row maximum of this warp moved, and only after the previous P V is done
      if (j >= 1 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!tc_wait(pv_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + lane_base + 256 + half * OC + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tmem + lane_base + 256 + half * OC + c * 32, r);
        }
        tc_wait_st();
      }
      // this P buffer was read by the P V of two tiles ago
      if (j >= 2 && !tc_wait(pv_done + 8 * st, ((j >> 1) - 1) & 1)) { ok = false; break; }
      // P = 2^(s - m), row sum, P (16-bit) into the swizzled K-major operand buffer (64-token chunk `half`)
      float ps8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // four packed accumulators
      const float neg_m = -m_new;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          // every fourth pair of exponentials on the FMA pipe (packed), the others on the special-function unit
          float x0, x1, p0, p1;
          ffma2(x0, x1, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]), a.scale_log2, a.scale_log2, neg_m, neg_m);
          if ((i & 6) == 6) {
            exp2_poly2(x0, x1, p0, p1);
          } else {
            p0 = fast_exp2(x0);
            p1 = fast_exp2(x1);
          }
          const int k = (i >> 1) & 3;
          fadd2(ps8[2 * k], ps8[2 * k + 1], ps8[2 * k], ps8[2 * k + 1], p0, p1);
          pk[i >> 1] = a.bf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
        }
        // 32 tokens of this half row = 16 columns of the P buffer in tensor memory
        tmem_st16(tmem + lane_base + 384 + st * 64 + half * 32 + c * 16, pk);
      }
      tc_wait_st();
      l_run = l_run * alpha + (((ps8[0] + ps8[1]) + (ps8[2] + ps8[3])) + ((ps8[4] + ps8[5]) + (ps8[6] + ps8[7])));
      // P written and O rescaled: the P V of this tile may go
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + 8 * st);
    }
    // epilogue: the two halves add their row sums, then O / l -> out (each thread its half of the row)
    if (ok) {
      xchg[((n_tiles & 1) * 2 + half) * 128 + row] = l_run;  // the parity slot the last tile did not use
      ok = pair_sync();
    }
    if (ok && !tc_wait(pv_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1)) ok = false;
    if (!ok) {
      if (lane == 0) give_up();
    } else {
      tc_fence_after();
      const float l_tot = l_run + xchg[((n_tiles & 1) * 2 + (half ^ 1)) * 128 + row];
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      const bool store = qpos < a.S;
      const size_t orow = (((size_t)b * a.Hq + qh) * (size_t)a.S + (store ? qpos : 0)) * D + half * OC;
      uint4* og = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.out) + orow);
      float4* ogf = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + orow);
      const bool out_bf16 = a.out_dtype == CUDA_LLM_BF16, out_f32 = a.out_dtype == CUDA_LLM_F32;
#pragma unroll 1
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + 256 + half * OC + c * 32, r);
        tc_wait_ld();
        if (store && out_f32) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            ogf[c * 8 + u] = make_float4(__uint_as_float(r[4 * u]) * inv, __uint_as_float(r[4 * u + 1]) * inv,
                                         __uint_as_float(r[4 * u + 2]) * inv, __uint_as_float(r[4 * u + 3]) * inv);
        } else if (store) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float x0 = __uint_as_float(r[8 * u + 2 * e]) * inv, x1 = __uint_as_float(r[8 * u + 2 * e + 1]) * inv;
              w[e] = out_bf16 ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
            }
            og[c * 4 + u] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  // common exit: every thread arrives here, also after a wait that ran out
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// ---- host side -------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder();  // api.cu

static bool encode_bhsd(EncodeTiledFn enc, CUtensorMap* m, const void* p, long long bh, int S, int D, int box_rows) {
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)bh};
  const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)S * D * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(p), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Query heads of a KV head that share a CTA: the largest of 8, 4, 2, 1 that divides the group (a group of 3, 5 or
// 7 heads runs one head per CTA like MHA, a group of 6 two, a group of 12 four).
static int heads_per_cta(int group) { return group % 8 == 0 ? 8 : group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1; }

// Whether the tcgen05 kernel takes this shape: 16-bit tensors, any group size.
bool gqa_prefill_sm100_supported(int Hq, int Hkv, int D, int dtype) {
  if (dtype != CUDA_LLM_F16 && dtype != CUDA_LLM_BF16) return false;
  if (D != 64 && D != 128) return false;
  return Hkv > 0 && Hq % Hkv == 0;
}

// dtype: the 16-bit type of q, k, v; out_dtype: any of the three output types.
cudaError_t run_gqa_prefill_sm100(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hkv, int S,
                                  int D, float softmax_scale, bool causal, int dtype, int out_dtype, cudaStream_t st) {
  if (B == 0 || S == 0) return cudaSuccess;
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return cudaErrorNotSupported;
  Prefill100Args a;
  a.out = out; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.group = Hq / Hkv;
  a.gsz = heads_per_cta(a.group);
  a.causal = causal ? 1 : 0;
  a.bf16 = dtype == CUDA_LLM_BF16 ? 1 : 0;
  a.out_dtype = out_dtype;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  const int bq = 128 / a.gsz;
  PrefillMaps maps;
  if (!encode_bhsd(enc, &maps.q, q, (long long)B * Hq, S, D, bq) || !encode_bhsd(enc, &maps.k, k, (long long)B * Hkv, S, D, kP100Bc) ||
      !encode_bhsd(enc, &maps.v, v, (long long)B * Hkv, S, D, kP100Bc))
    return cudaErrorInvalidValue;
  const int nch = D / 64;
  size_t smem = (size_t)nch * 16384 * 7 + 256 + 512 * 4;  // Q, 3 x K, 3 x V, barriers, exchange
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: a CTA allocates all 512 TMEM columns
  auto kern = D == 64 ? gqa_prefill_sm100_kernel<64> : gqa_prefill_sm100_kernel<128>;
  static int configured[2][64] = {{0}};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[D == 128][dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[D == 128][dev] = 1;
  }
  dim3 grid((S + bq - 1) / bq, Hkv * (a.group / a.gsz), B);
  kern<<<grid, kP100Threads, smem, st>>>(a, maps);
  return cudaGetLastError();
}

cudaError_t prefill_wait_timeouts(unsigned int* count) {
  return cudaMemcpyFromSymbol(count, g_prefill_wait_timeouts, sizeof(unsigned int));
}

}  // namespace b200
