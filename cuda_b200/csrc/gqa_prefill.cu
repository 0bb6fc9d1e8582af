// Grouped-query prefill attention with an optional paged, quantised KV-cache write.
//
// Replaces the reference's fused_gqa_forward_kernel / dispatch_fused_gqa
// (fused_gqa_kernel.cuh:22-212, 215-249 in the reference project: one thread per query row, scalar
// FP32 dot products over fp32 copies of the tiles in 80/160 KB of static shared memory -- it does not
// assemble for sm_100a).  Semantics kept: q [B, Hq, S, D], k / v [B, Hkv, S, D], out [B, Hq, S, D],
// kv_head = q_head / (Hq / Hkv), causal mask "key position <= query position", fp32 softmax.
//
// Shape of this kernel: one CTA per (batch, KV head, block of query positions).  Its eight warps cover
// the query heads that share the KV head (up to 8 per CTA), 16 query rows each, so that a K/V tile is
// brought into shared memory once for the whole group.  K/V tiles of 64 tokens arrive through 16-byte
// cp.async into a two-deep ring with XOR-swizzled rows; S = Q K^T and O += P V run on warp MMA
// (m16n8k16, f16 or bf16 in, fp32 accumulate) with ldmatrix operand loads; P never leaves registers.
// The same host call can write the new K / V into the paged cache the decode path reads
// (kv_append_kernel: quantise with the cache's recipe, store into cache[block][head][d][offset]).
#include "paged_decode_kernel.cuh"

namespace b200 {

struct PrefillArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int B, Hq, Hkv, S, group, n_chunks;
  int causal;
  float scale_log2;
  // microscaled inputs (MXQ kernels): q / k / v are E4M3 bytes, one fp32 scale per 32 elements of head_dim
  const float* qs;  // [B, Hq, S, D/32]
  const float* ks;  // [B, Hkv, S, D/32]
  const float* vs;
  int out_dtype;    // CudaLlmDType of `out` (MXQ kernels; the 16-bit kernels write their input dtype)
};

constexpr int kPfWarps = 8;
constexpr int kPfBc = 64;  // KV tokens per tile

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  // zero-fills the 16 bytes when !valid (src-size 0)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}

// 16 E4M3 codes (one 16-byte load) times their block scale -> 16 f16 values (two 16-byte chunks).
// E4M3 -> f16 is exact; the product is rounded to f16 once.
__device__ __forceinline__ void dequant16(const uint4 codes, float scale, uint4& lo, uint4& hi) {
  auto two = [&](uint32_t h2) -> uint32_t { return pack_f16x2(f16x2_lo(h2) * scale, f16x2_hi(h2) * scale); };
  lo.x = two(e4m3x2_to_f16x2_lo(codes.x)); lo.y = two(e4m3x2_to_f16x2_hi(codes.x));
  lo.z = two(e4m3x2_to_f16x2_lo(codes.y)); lo.w = two(e4m3x2_to_f16x2_hi(codes.y));
  hi.x = two(e4m3x2_to_f16x2_lo(codes.z)); hi.y = two(e4m3x2_to_f16x2_hi(codes.z));
  hi.z = two(e4m3x2_to_f16x2_lo(codes.w)); hi.w = two(e4m3x2_to_f16x2_hi(codes.w));
}
__device__ __forceinline__ void sts128u(uint32_t addr, const uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// MXQ: the tensors are E4M3 bytes with fp32 block scales; tiles are dequantised to f16 on their way
// into shared memory (dispatch_fused_microscaled_attention, kernels_api.h:103-108 in the reference
// project, declared there without a definition).
template <int D, bool BF, bool MXQ>
__global__ void __launch_bounds__(kPfWarps * 32) gqa_prefill_kernel(const PrefillArgs a) {
  constexpr int PITCH = D * 2;          // bytes per row
  constexpr int CHUNKS = PITCH / 16;    // 16-byte chunks per row
  constexpr int KT = D / 16;            // k-tiles of Q K^T
  constexpr int NT = kPfBc / 8;         // n-tiles of S per KV tile
  constexpr int DT = D / 8;             // n-tiles of O
  constexpr float NEG_INF = -__builtin_huge_valf();
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);                       // [8 warps][16 rows][D]
  const uint32_t sK = sQ + kPfWarps * 16 * PITCH;           // [2][64][D]
  const uint32_t sV = sK + 2 * kPfBc * PITCH;               // [2][64][D]
  auto swz = [](int row, int chunk) -> uint32_t { return (uint32_t)row * PITCH + (uint32_t)((chunk ^ (row & 7)) * 16); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.z;
  const int kvh = blockIdx.y / a.n_chunks, chunk = blockIdx.y - kvh * a.n_chunks;
  const int gsz = min(8, a.group - chunk * 8);              // query heads of this CTA
  const int wph = kPfWarps / gsz;                           // warps (16-row tiles) per head
  const int BQ = 16 * wph;                                  // query positions per CTA
  const int qt = (int)(gridDim.x - 1 - blockIdx.x);         // heavy (late) causal tiles first
  const int q0 = qt * BQ;
  if (q0 >= a.S) return;
  const int hi = warp / wph, jw = warp - hi * wph;
  const bool active = hi < gsz;
  const int qh = kvh * a.group + chunk * 8 + (active ? hi : 0);
  const int qrow0 = q0 + 16 * jw;                           // first query position of this warp

  constexpr int EB = MXQ ? 1 : 2;                           // bytes per element in global memory
  const size_t kv_base = ((size_t)b * a.Hkv + kvh) * (size_t)a.S * D;
  const uint8_t* kg = reinterpret_cast<const uint8_t*>(a.k) + kv_base * EB;
  const uint8_t* vg = reinterpret_cast<const uint8_t*>(a.v) + kv_base * EB;
  const float* ksg = MXQ ? a.ks + kv_base / 32 : nullptr;
  const float* vsg = MXQ ? a.vs + kv_base / 32 : nullptr;

  const int last_q = min(a.S, q0 + BQ) - 1;
  const int n_tiles = a.causal ? min((a.S + kPfBc - 1) / kPfBc, last_q / kPfBc + 1) : (a.S + kPfBc - 1) / kPfBc;

  auto load_tile = [&](int tile, int stage) {
    const int kv0 = tile * kPfBc;
    if (MXQ) {
      // 16 codes per thread and step: one 16-byte load, one scale, two swizzled 16-byte stores
      for (int i = tid; i < kPfBc * (D / 16); i += kPfWarps * 32) {
        const int r = i / (D / 16), c16 = i - r * (D / 16);
        uint4 klo = make_uint4(0, 0, 0, 0), khi = klo, vlo = klo, vhi = klo;
        if (kv0 + r < a.S) {
          const size_t row = (size_t)(kv0 + r);
          dequant16(*reinterpret_cast<const uint4*>(kg + row * D + c16 * 16), ksg[row * (D / 32) + (c16 >> 1)], klo, khi);
          dequant16(*reinterpret_cast<const uint4*>(vg + row * D + c16 * 16), vsg[row * (D / 32) + (c16 >> 1)], vlo, vhi);
        }
        sts128u(sK + stage * (kPfBc * PITCH) + swz(r, 2 * c16), klo);
        sts128u(sK + stage * (kPfBc * PITCH) + swz(r, 2 * c16 + 1), khi);
        sts128u(sV + stage * (kPfBc * PITCH) + swz(r, 2 * c16), vlo);
        sts128u(sV + stage * (kPfBc * PITCH) + swz(r, 2 * c16 + 1), vhi);
      }
      return;
    }
    for (int i = tid; i < kPfBc * CHUNKS; i += kPfWarps * 32) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const bool ok = kv0 + r < a.S;
      const size_t off = ((size_t)(ok ? kv0 + r : 0) * D) * 2 + c * 16;
      cp_async_16(sK + stage * (kPfBc * PITCH) + swz(r, c), kg + off, ok);
      cp_async_16(sV + stage * (kPfBc * PITCH) + swz(r, c), vg + off, ok);
    }
  };

  // Q rows of this warp -> shared memory -> A fragments (kept in registers for the whole CTA)
  if (MXQ) {
    const size_t qb = ((size_t)b * a.Hq + qh) * (size_t)a.S;
    const uint8_t* qg = reinterpret_cast<const uint8_t*>(a.q) + qb * D;
    for (int i = lane; i < 16 * (D / 16); i += 32) {
      const int r = i / (D / 16), c16 = i - r * (D / 16);
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (active && qrow0 + r < a.S) {
        const size_t row = (size_t)(qrow0 + r);
        dequant16(*reinterpret_cast<const uint4*>(qg + row * D + c16 * 16), a.qs[(qb + row) * (D / 32) + (c16 >> 1)], lo, hi);
      }
      sts128u(sQ + warp * (16 * PITCH) + swz(r, 2 * c16), lo);
      sts128u(sQ + warp * (16 * PITCH) + swz(r, 2 * c16 + 1), hi);
    }
  } else {
    const uint8_t* qg = reinterpret_cast<const uint8_t*>(a.q) + (((size_t)b * a.Hq + qh) * (size_t)a.S) * D * 2;
    for (int i = lane; i < 16 * CHUNKS; i += 32) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const bool ok = active && qrow0 + r < a.S;
      cp_async_16(sQ + warp * (16 * PITCH) + swz(r, c), qg + ((size_t)(ok ? qrow0 + r : 0) * D) * 2 + c * 16, ok);
    }
  }
  load_tile(0, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KT][4];
#pragma unroll
  for (int kt = 0; kt < KT; ++kt)
    ldmatrix_x4(qf[kt], sQ + warp * (16 * PITCH) + swz((lane & 7) + 8 * ((lane >> 3) & 1), 2 * kt + (lane >> 4)));

  float oacc[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) oacc[i][c] = 0.f;
  float m_run[2] = {-1.0e30f, -1.0e30f}, l_run[2] = {0.f, 0.f};

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) load_tile(tile + 1, stage ^ 1);
    cp_async_commit();
    const int kv0 = tile * kPfBc;
    // a warp whose rows all lie before this tile (causal) has nothing to do in it
    const bool skip = !active || (a.causal && kv0 > qrow0 + 15);
    if (!skip) {
      const uint32_t kb = sK + stage * (kPfBc * PITCH), vb = sV + stage * (kPfBc * PITCH);
      float sacc[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[i][c] = 0.f;
#pragma unroll
      for (int kt = 0; kt < KT; ++kt)
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t r4[4];  // b0, b1 of n-tile 2np, then of n-tile 2np + 1
          ldmatrix_x4(r4, kb + swz(16 * np + (lane & 7) + 8 * (lane >> 4), 2 * kt + ((lane >> 3) & 1)));
          if (BF) {
            mma_bf16(sacc[2 * np], qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3], r4[0], r4[1]);
            mma_bf16(sacc[2 * np + 1], qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3], r4[2], r4[3]);
          } else {
            mma_f16(sacc[2 * np], qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3], r4[0], r4[1]);
            mma_f16(sacc[2 * np + 1], qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3], r4[2], r4[3]);
          }
        }
      // scale, mask (key beyond the sequence, or after the query position when causal), row maxima
      const bool need_mask = (kv0 + kPfBc > a.S) || (a.causal && kv0 + kPfBc - 1 > qrow0);
      float mx[2] = {NEG_INF, NEG_INF};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float x = sacc[nt][c] * a.scale_log2;
          if (need_mask) {
            const int key = kv0 + 8 * nt + 2 * t + (c & 1), qpos = qrow0 + g + 8 * (c >> 1);
            if (key >= a.S || (a.causal && key > qpos)) x = NEG_INF;
          }
          sacc[nt][c] = x;
          mx[c >> 1] = fmaxf(mx[c >> 1], x);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float al[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float mn = fmaxf(m_run[r], mx[r]);
        al[r] = fast_exp2(m_run[r] - mn);
        m_run[r] = mn;
      }
      float ps[2] = {0.f, 0.f};
      uint32_t pa[NT][2];  // P as A-operand halves: [nt][0] = row g, [nt][1] = row g + 8 (cols 2t, 2t+1 of n-tile nt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float p0 = fast_exp2(sacc[nt][0] - m_run[0]), p1 = fast_exp2(sacc[nt][1] - m_run[0]);
        const float p2 = fast_exp2(sacc[nt][2] - m_run[1]), p3 = fast_exp2(sacc[nt][3] - m_run[1]);
        ps[0] += p0 + p1;
        ps[1] += p2 + p3;
        pa[nt][0] = BF ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
        pa[nt][1] = BF ? pack_bf16x2(p2, p3) : pack_f16x2(p2, p3);
      }
      l_run[0] = l_run[0] * al[0] + ps[0];
      l_run[1] = l_run[1] * al[1] + ps[1];
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        oacc[i][0] *= al[0]; oacc[i][1] *= al[0];
        oacc[i][2] *= al[1]; oacc[i][3] *= al[1];
      }
      // O += P V: k index = token; two adjacent n-tiles of S form one 16-token A fragment
#pragma unroll
      for (int kt = 0; kt < kPfBc / 16; ++kt)
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {
          uint32_t r4[4];  // b0, b1 of d n-tile 2dp, then of 2dp + 1
          ldmatrix_x4_trans(r4, vb + swz(16 * kt + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * dp + (lane >> 4)));
          if (BF) {
            mma_bf16(oacc[2 * dp], pa[2 * kt][0], pa[2 * kt][1], pa[2 * kt + 1][0], pa[2 * kt + 1][1], r4[0], r4[1]);
            mma_bf16(oacc[2 * dp + 1], pa[2 * kt][0], pa[2 * kt][1], pa[2 * kt + 1][0], pa[2 * kt + 1][1], r4[2], r4[3]);
          } else {
            mma_f16(oacc[2 * dp], pa[2 * kt][0], pa[2 * kt][1], pa[2 * kt + 1][0], pa[2 * kt + 1][1], r4[0], r4[1]);
            mma_f16(oacc[2 * dp + 1], pa[2 * kt][0], pa[2 * kt][1], pa[2 * kt + 1][0], pa[2 * kt + 1][1], r4[2], r4[3]);
          }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  if (!active) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv[2] = {l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, l_run[1] > 0.f ? 1.f / l_run[1] : 0.f};
  uint32_t* og = reinterpret_cast<uint32_t*>(a.out);
  const int odt = MXQ ? a.out_dtype : (BF ? CUDA_LLM_BF16 : CUDA_LLM_F16);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qpos = qrow0 + g + 8 * r;
    if (qpos >= a.S) continue;
    const size_t row = (((size_t)b * a.Hq + qh) * (size_t)a.S + qpos) * D;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      const float x0 = oacc[i][2 * r] * inv[r], x1 = oacc[i][2 * r + 1] * inv[r];
      const size_t e = row + 8 * i + 2 * t;
      if (odt == CUDA_LLM_F32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + e) = make_float2(x0, x1);
      else og[e >> 1] = (odt == CUDA_LLM_BF16) ? pack_bf16x2(x0, x1) : pack_f16x2(x0, x1);
    }
  }
}

template <int D, bool BF, bool MXQ = false>
static cudaError_t launch_prefill(const PrefillArgs& a, cudaStream_t st) {
  auto kern = gqa_prefill_kernel<D, BF, MXQ>;
  constexpr int smem = (kPfWarps * 16 + 4 * kPfBc) * D * 2;
  static int configured[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured[dev] = 1;
  }
  const int gsz0 = a.group < 8 ? a.group : 8;
  const int bq = 16 * (kPfWarps / gsz0);  // query positions per CTA of a full chunk (the smallest block any chunk uses)
  dim3 grid((a.S + bq - 1) / bq, a.Hkv * a.n_chunks, a.B);
  kern<<<grid, kPfWarps * 32, smem, st>>>(a);
  return cudaGetLastError();
}

// fp32 tensors: a plain SIMT kernel (no tensor-core operand form keeps fp32 accuracy without a
// three-way split).  One warp per query row, four rows of one (batch, query head) per CTA; K/V
// tiles of 32 tokens in shared memory; lane = token for Q.K, lane = head_dim slice for P.V.
template <int D>
__global__ void __launch_bounds__(128) gqa_prefill_f32_kernel(const PrefillArgs a) {
  constexpr int E = D / 32;
  constexpr float NEG_INF = -__builtin_huge_valf();
  __shared__ float sK[32][D + 1];
  __shared__ float sV[32][D + 1];
  __shared__ float sQ[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, qh = blockIdx.y, kvh = qh / a.group;
  const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * 4, qpos = q0 + warp;
  const float* qg = reinterpret_cast<const float*>(a.q) + (((size_t)b * a.Hq + qh) * (size_t)a.S) * D;
  const float* kg = reinterpret_cast<const float*>(a.k) + (((size_t)b * a.Hkv + kvh) * (size_t)a.S) * D;
  const float* vg = reinterpret_cast<const float*>(a.v) + (((size_t)b * a.Hkv + kvh) * (size_t)a.S) * D;
  const bool row_ok = qpos < a.S;
#pragma unroll
  for (int e = 0; e < E; ++e) sQ[warp][lane + 32 * e] = row_ok ? qg[(size_t)qpos * D + lane + 32 * e] : 0.f;
  float m = -1.0e30f, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  const int last_q = min(a.S, q0 + 4) - 1;
  const int n_keys = a.causal ? min(a.S, last_q + 1) : a.S;
  for (int kv0 = 0; kv0 < n_keys; kv0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * D; i += 128) {
      const int r = i / D, c = i - r * D;
      const bool ok = kv0 + r < a.S;
      sK[r][c] = ok ? kg[(size_t)(kv0 + r) * D + c] : 0.f;
      sV[r][c] = ok ? vg[(size_t)(kv0 + r) * D + c] : 0.f;
    }
    __syncthreads();
    const int key = kv0 + lane;
    float s = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; ++d) s = fmaf(sQ[warp][d], sK[lane][d], s);
    s *= a.scale_log2;
    if (!row_ok || key >= a.S || (a.causal && key > qpos)) s = NEG_INF;
    float mx = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float mn = fmaxf(m, mx);
    const float al = exp2f(m - mn);
    const float p = exp2f(s - mn);
    m = mn;
    float ps = p;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * al + ps;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] *= al;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = fmaf(pj, sV[j][lane + 32 * e], acc[e]);
    }
  }
  if (!row_ok) return;
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* og = reinterpret_cast<float*>(a.out) + (((size_t)b * a.Hq + qh) * (size_t)a.S + qpos) * D;
#pragma unroll
  for (int e = 0; e < E; ++e) og[lane + 32 * e] = acc[e] * inv;
}

cudaError_t run_gqa_prefill(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hkv, int S,
                            int D, float softmax_scale, bool causal, int dtype, cudaStream_t st) {
  PrefillArgs a;
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.qs = a.ks = a.vs = nullptr; a.out_dtype = dtype;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.group = Hq / Hkv;
  a.n_chunks = (a.group + 7) / 8;
  a.causal = causal ? 1 : 0;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  if (B == 0 || S == 0) return cudaSuccess;
  if (dtype == CUDA_LLM_F32) {
    dim3 grid((S + 3) / 4, Hq, B);
    if (D == 64) gqa_prefill_f32_kernel<64><<<grid, 128, 0, st>>>(a);
    else gqa_prefill_f32_kernel<128><<<grid, 128, 0, st>>>(a);
    return cudaGetLastError();
  }
  if (dtype == CUDA_LLM_BF16) return D == 64 ? launch_prefill<64, true>(a, st) : launch_prefill<128, true>(a, st);
  return D == 64 ? launch_prefill<64, false>(a, st) : launch_prefill<128, false>(a, st);
}

// E4M3 codes with one fp32 scale per 32 consecutive elements -> f16, code times scale rounded once.  A thread
// takes 16 codes (one 16-byte load, two 16-byte stores); n_elems is a multiple of 32.
__global__ void __launch_bounds__(256) mx_to_f16_kernel(const uint4* __restrict__ codes, const float* __restrict__ scales,
                                                        uint4* __restrict__ out, size_t n16) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n16) return;
  const uint4 c = codes[i];
  const float sc = scales[i >> 1];
  const uint32_t w[4] = {c.x, c.y, c.z, c.w};
  uint32_t h[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t lo = e4m3x2_to_f16x2_lo(w[j]), hi = e4m3x2_to_f16x2_hi(w[j]);
    h[2 * j] = pack_f16x2(f16x2_lo(lo) * sc, f16x2_hi(lo) * sc);
    h[2 * j + 1] = pack_f16x2(f16x2_lo(hi) * sc, f16x2_hi(hi) * sc);
  }
  out[2 * i] = make_uint4(h[0], h[1], h[2], h[3]);
  out[2 * i + 1] = make_uint4(h[4], h[5], h[6], h[7]);
}

cudaError_t launch_mx_to_f16(const void* codes, const float* scales, void* out, size_t n_elems, cudaStream_t st) {
  const size_t n16 = n_elems / 16;
  if (n16 == 0) return cudaSuccess;
  mx_to_f16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const uint4*>(codes), scales,
                                                                 reinterpret_cast<uint4*>(out), n16);
  return cudaGetLastError();
}

cudaError_t run_mx_attention(const void* q, const float* qs, const void* k, const float* ks, const void* v,
                             const float* vs, void* out, int B, int Hq, int Hkv, int S, int D, float softmax_scale,
                             bool causal, int out_dtype, cudaStream_t st) {
  PrefillArgs a;
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.qs = qs; a.ks = ks; a.vs = vs; a.out_dtype = out_dtype;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.group = Hq / Hkv;
  a.n_chunks = (a.group + 7) / 8;
  a.causal = causal ? 1 : 0;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  if (B == 0 || S == 0) return cudaSuccess;
  return D == 64 ? launch_prefill<64, false, true>(a, st) : launch_prefill<128, false, true>(a, st);
}

}  // namespace b200
