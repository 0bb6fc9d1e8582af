// Writes new K/V tokens into the paged, quantised cache: the step that precedes the decode path.
// The reference has no such kernel (its tests quantise with torch on the host,
// tests/test_kernels_misc.py:51-55, and page with make_paged_cache, tests/_utils.py:107-133); this
// one reproduces that recipe bit for bit on the device:
//   per-token fp32 scale : scale = max(amax / 448, 1e-8); code = E4M3(x / scale), round to nearest even
//   E8M0 block scale     : e = floor(log2(amax_block)) - emax (8 for E4M3, 2 for E2M1), code = x / 2^e
//   per-head fp32 scale  : the given scale is used, code = E4M3(x / scale)
// One warp per (token, KV head, K | V) quantises; lanes split head_dim; codes go to cache[block][head][d][offset],
// as 16-byte rows of 16 tokens where the new tokens fill whole pages.
#include <type_traits>

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
  int aligned;  // set by the launcher: caches and scales allow 16-byte rows
  int src_vec;  // set by the launcher: the source tensors allow 8-byte loads
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

// E consecutive elements of a source row, as loaded (one vector load where the tensors allow it) ...
template <int E>
__device__ __forceinline__ uint4 load_raw(const void* src, int dtype, size_t idx, bool vec) {
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (!vec) {  // element by element, kept as fp32 bits
    r.x = __float_as_uint(load_q_elem(src, dtype, idx));
    r.y = __float_as_uint(load_q_elem(src, dtype, idx + 1));
    if (E == 4) {
      r.z = __float_as_uint(load_q_elem(src, dtype, idx + 2));
      r.w = __float_as_uint(load_q_elem(src, dtype, idx + 3));
    }
  } else if (dtype == CUDA_LLM_F32) {
    if (E == 4) {
      r = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(src) + idx);
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const float*>(src) + idx);
      r.x = v.x; r.y = v.y;
    }
  } else if (E == 4) {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(src) + idx);
    r.x = v.x; r.y = v.y;
  } else {
    r.x = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(src) + idx);
  }
  return r;
}
// ... and widened to fp32
template <int E>
__device__ __forceinline__ void raw_to_float(const uint4& r, int dtype, bool vec, float (&x)[E]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
  if (!vec || dtype == CUDA_LLM_F32) {
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = __uint_as_float(w[e]);
  } else {
#pragma unroll
    for (int e = 0; e < E; e += 2) {
      if (dtype == CUDA_LLM_F16) {
        x[e] = f16x2_lo(w[e / 2]);
        x[e + 1] = f16x2_hi(w[e / 2]);
      } else {
        x[e] = __uint_as_float(w[e / 2] << 16);
        x[e + 1] = __uint_as_float(w[e / 2] & 0xffff0000u);
      }
    }
  }
}
__device__ __forceinline__ size_t source_row(const AppendArgs& a, long long tok, int h) {
  return a.seq_len > 0 ? ((size_t)(tok / a.seq_len) * a.Hkv + h) * a.seq_len + (tok % a.seq_len) : (size_t)tok * a.Hkv + h;
}

// One token row of one head, quantised by a warp: lane owns d = lane*E .. lane*E+E-1.  Returns the lane's
// code bytes packed little-endian (E bytes of E4M3, E/2 bytes of nibble pairs for E2M1), the per-token fp32
// scale (SCALE_PER_TOKEN) and the E8M0 byte of the lane's 32-element block (SCALE_MX_E8M0).
template <int D>
__device__ __forceinline__ uint32_t quantise_row(const AppendArgs& a, const uint4& raw, int h, int is_v, int blk, int lane,
                                                 float& tok_scale, uint32_t& eb_out) {
  constexpr int E = D / 32;
  float x[E];
  raw_to_float<E>(raw, a.in_dtype, a.src_vec != 0, x);
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) amax = fmaxf(amax, fabsf(x[e]));
  const bool fp4 = is_v && a.v_format == CUDA_LLM_KV_FP4_E2M1;
  const void* scale = is_v ? a.vs : a.ks;
  tok_scale = 0.f;
  eb_out = 0;
  if (a.scale_mode == CUDA_LLM_SCALE_MX_E8M0) {
    // a 32-element block = 32/E consecutive lanes
#pragma unroll
    for (int o = 1; o < 32 / E; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 7.888609052210118e-31f);  // 2^-100, as the host recipe clamps
    const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2(amax))
    const int eb = min(254, max(0, ef - (fp4 ? 2 : 8) + 127));
    const float inv = __uint_as_float((uint32_t)(254 - eb) << 23);      // 2^-(eb-127); eb in [0,254] -> exact except eb=254
    eb_out = (uint32_t)eb;
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = (eb == 0) ? x[e] * 1.7014118346046923e38f : x[e] * inv;
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc;
    if (a.scale_mode == CUDA_LLM_SCALE_PER_TOKEN) {
      sc = fmaxf(__fdiv_rn(amax, 448.f), 1e-8f);
      tok_scale = sc;
    } else if (a.scale_mode == CUDA_LLM_SCALE_PER_BLOCK) {
      sc = reinterpret_cast<const float*>(scale)[(size_t)blk * a.Hkv + h];
    } else {
      sc = reinterpret_cast<const float*>(scale)[h];
    }
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = __fdiv_rn(x[e], sc);
  }
  uint32_t packed = 0;
  if (!fp4) {
#pragma unroll
    for (int e = 0; e < E; e += 2) packed |= f32x2_to_e4m3x2(x[e], x[e + 1]) << (8 * e);
  } else {
#pragma unroll
    for (int e = 0; e < E; e += 2) packed |= (quant_e2m1_nibble(x[e]) | (quant_e2m1_nibble(x[e + 1]) << 4)) << (4 * e);
  }
  return packed;
}

// Few new tokens (a decode step appends one per sequence): one warp per (token, KV head, K | V), every code
// byte stored on its own.
template <int D>
__global__ void __launch_bounds__(128) kv_append_token_kernel(const AppendArgs a) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  // the decode kernel that follows is launched as a programmatic dependent: let it be scheduled now (it does
  // not touch the cache before its own griddepcontrol.wait, i.e. before this grid has completed)
  asm volatile("griddepcontrol.launch_dependents;");
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= 2LL * a.n * a.Hkv) return;
  const int is_v = (int)(item & 1);
  const int h = (int)((item >> 1) % a.Hkv);
  const long long tok = (item >> 1) / a.Hkv;
  const int blk = a.slot_block[tok], off = a.slot_offset[tok];
  if (blk < 0 || blk >= a.num_blocks || off < 0 || off >= a.page) {
    if (a.status && lane == 0) atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
    return;
  }
  float tsc;
  uint32_t eb;
  const uint4 raw = load_raw<E>(is_v ? a.v_new : a.k_new, a.in_dtype, source_row(a, tok, h) * D + lane * E, a.src_vec != 0);
  const uint32_t packed = quantise_row<D>(a, raw, h, is_v, blk, lane, tsc, eb);
  const bool fp4 = is_v && a.v_format == CUDA_LLM_KV_FP4_E2M1;
  uint8_t* cache = is_v ? a.vc : a.kc;
  void* scale = is_v ? a.vs : a.ks;
  if (a.scale_mode == CUDA_LLM_SCALE_PER_TOKEN && lane == 0)
    reinterpret_cast<float*>(scale)[((size_t)blk * a.Hkv + h) * a.page + off] = tsc;
  if (a.scale_mode == CUDA_LLM_SCALE_MX_E8M0 && (lane * E) % 32 == 0)
    reinterpret_cast<uint8_t*>(scale)[(((size_t)blk * a.Hkv + h) * (D / 32) + (lane * E) / 32) * a.page + off] = (uint8_t)eb;
  if (!fp4) {
    uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * D + lane * E) * a.page + off;
#pragma unroll
    for (int e = 0; e < E; ++e) dst[(size_t)e * a.page] = (uint8_t)(packed >> (8 * e));
  } else {
    uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * (D / 2) + lane * (E / 2)) * a.page + off;
#pragma unroll
    for (int e = 0; e < E / 2; ++e) dst[(size_t)e * a.page] = (uint8_t)(packed >> (8 * e));
  }
}

// x / sc, correctly rounded, for many x and one sc: y = RN(1 / sc) once, then q = RN(x y), r = x - q sc (exact,
// one FMA), q' = RN(q + r y).  q' equals the IEEE quotient whenever y is the correctly rounded reciprocal, q
// is within an ulp of the quotient and nothing leaves the normal range (Markstein's division theorem); the one
// divisor the theorem excludes (a significand of all ones) and divisors whose reciprocal is not normal take
// the IEEE division.  Callers guarantee sc > 0 and |x / sc| far below the overflow threshold.
struct Divisor {
  float sc, y;
  bool fast;
  __device__ __forceinline__ explicit Divisor(float s) : sc(s) {
    asm("rcp.rn.f32 %0, %1;" : "=f"(y) : "f"(s));  // IEEE reciprocal, round to nearest even
    const uint32_t b = __float_as_uint(s), e = (b >> 23) & 0xffu, ey = (__float_as_uint(y) >> 23) & 0xffu;
    fast = (b & 0x7fffffu) != 0x7fffffu && e >= 1 && e <= 253 && ey >= 1 && ey <= 253;
  }
  // x[e] /= sc for N values; one test of `fast` for all of them
  template <int N>
  __device__ __forceinline__ void div_all(float (&x)[N]) const {
    if (fast) {
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const float q = __fmul_rn(x[e], y);
        const float qq = __fmaf_rn(__fmaf_rn(-q, sc, x[e]), y, q);
        // the divisor is positive, so the quotient has the sign of x; the sums above turn -0 into +0
        x[e] = __uint_as_float((__float_as_uint(qq) & 0x7fffffffu) | (__float_as_uint(x[e]) & 0x80000000u));
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) x[e] = __fdiv_rn(x[e], sc);
    }
  }
};

// A CTA takes 16 consecutive new tokens of one KV head, K and V: 32 rows of head_dim values.  A row is
// quantised by head_dim / 16 adjacent lanes, 16 values each (four or eight rows per warp at a time, so the
// per-row work -- the maximum, its scale, a reciprocal -- is shared by 16 values per lane instead of 4).
// When the 16 tokens fill 16 consecutive slots of one page (a prefill writes whole pages), their codes are
// collected in shared memory as [token][head_dim] and written out transposed, 16 bytes (16 tokens) per
// head_dim row, so that a page slab is written with full-width stores; per-token and E8M0 scales likewise, as
// rows of 16.  Otherwise (ragged ends, sequences that start inside a page) every code byte is stored on its own.
template <int D, int DT, int SMODE>
__global__ void __launch_bounds__(128) kv_append_tile_kernel(const AppendArgs a) {
  // DT: source dtype (CUDA_LLM_F32 / F16 / BF16) when the source allows vector loads, -1 for element loads of
  // any dtype; SMODE: the scale mode.  Compile-time so that the unrolled per-value code has no run-time switches.
  constexpr int NB = D / 32;
  constexpr int LPR = D / 16;        // lanes per row
  constexpr int RPP = 32 / LPR;      // rows per warp and pass
  constexpr int PASSES = 32 / (4 * RPP);
  __shared__ __align__(16) uint32_t tile[2][16][D / 4];   // codes: [K | V][token][head_dim byte rows]
  __shared__ __align__(16) float tok_scales[2][16];
  __shared__ __align__(16) uint8_t mx_scales[2][NB][16];
  __shared__ int s_fast, s_blk, s_off0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = (int)(blockIdx.x % a.Hkv);
  const long long t0 = (long long)(blockIdx.x / a.Hkv) * 16;
  if (warp == 0) {
    const long long tok = t0 + (lane & 15);
    bool ok = tok < a.n;
    const int blk = ok ? a.slot_block[tok] : -1, off = ok ? a.slot_offset[tok] : -1;
    const int blk0 = __shfl_sync(0xffffffffu, blk, 0), off0 = __shfl_sync(0xffffffffu, off, 0);
    ok = ok && blk == blk0 && off == off0 + (lane & 15) && blk0 >= 0 && blk0 < a.num_blocks && off0 >= 0 &&
         (off0 & 15) == 0 && off0 + 16 <= a.page;
    const bool fast = __all_sync(0xffffffffu, ok) && a.aligned;
    if (lane == 0) {
      s_fast = fast ? 1 : 0;
      s_blk = blk0;
      s_off0 = off0;
    }
  }
  const int sub = lane % LPR, d0 = sub * 16;
  constexpr bool vec = DT >= 0;
  constexpr bool wide = DT == CUDA_LLM_F32;
  // the rows of this lane (row r: token r / 2, K for even r, V for odd r), all requested before the first is used
  uint4 raw[PASSES][4];
#pragma unroll
  for (int ps = 0; ps < PASSES; ++ps) {
    const int r = (ps * 4 + warp) * RPP + lane / LPR;
    const long long tok = t0 + (r >> 1);
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[ps][j] = make_uint4(0u, 0u, 0u, 0u);
    if (tok < a.n) {
      const void* src = (r & 1) ? a.v_new : a.k_new;
      const size_t idx = source_row(a, tok, h) * D + d0;
      if (!vec) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          raw[ps][j] = make_uint4(__float_as_uint(load_q_elem(src, a.in_dtype, idx + 4 * j)),
                                  __float_as_uint(load_q_elem(src, a.in_dtype, idx + 4 * j + 1)),
                                  __float_as_uint(load_q_elem(src, a.in_dtype, idx + 4 * j + 2)),
                                  __float_as_uint(load_q_elem(src, a.in_dtype, idx + 4 * j + 3)));
      } else if (wide) {
#pragma unroll
        for (int j = 0; j < 4; ++j) raw[ps][j] = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(src) + idx)[j];
      } else {
        raw[ps][0] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(src) + idx)[0];
        raw[ps][1] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(src) + idx)[1];
      }
    }
  }
  __syncthreads();
  const bool fast = s_fast != 0;
  const bool fp4v = a.v_format == CUDA_LLM_KV_FP4_E2M1;
#pragma unroll
  for (int ps = 0; ps < PASSES; ++ps) {
    const int r = (ps * 4 + warp) * RPP + lane / LPR;
    const int tl = r >> 1, is_v = r & 1;
    const long long tok = t0 + tl;
    const bool row_live = tok < a.n;
    int blk = s_blk, off = s_off0 + tl;
    bool slot_ok = row_live;
    if (!fast && row_live) {
      blk = a.slot_block[tok];
      off = a.slot_offset[tok];
      slot_ok = blk >= 0 && blk < a.num_blocks && off >= 0 && off < a.page;
      if (!slot_ok && a.status && sub == 0) atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
    }
    // ---- the 16 values of this lane as fp32
    float x[16];
    if (!vec || wide) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[4 * j] = __uint_as_float(raw[ps][j].x); x[4 * j + 1] = __uint_as_float(raw[ps][j].y);
        x[4 * j + 2] = __uint_as_float(raw[ps][j].z); x[4 * j + 3] = __uint_as_float(raw[ps][j].w);
      }
    } else {
      const uint32_t w[8] = {raw[ps][0].x, raw[ps][0].y, raw[ps][0].z, raw[ps][0].w,
                             raw[ps][1].x, raw[ps][1].y, raw[ps][1].z, raw[ps][1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (DT == CUDA_LLM_F16) {
          x[2 * j] = f16x2_lo(w[j]);
          x[2 * j + 1] = f16x2_hi(w[j]);
        } else {
          x[2 * j] = __uint_as_float(w[j] << 16);
          x[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(x[e]));
    const bool fp4 = is_v && fp4v;
    void* scale = is_v ? a.vs : a.ks;
    float tsc = 0.f;
    uint32_t eb = 0;
    if (SMODE == CUDA_LLM_SCALE_MX_E8M0) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // a 32-element block = two adjacent lanes
      amax = fmaxf(amax, 7.888609052210118e-31f);  // 2^-100, as the host recipe clamps
      const int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2(amax))
      eb = (uint32_t)min(254, max(0, ef - (fp4 ? 2 : 8) + 127));
      const float inv = __uint_as_float((uint32_t)(254 - eb) << 23);      // 2^-(eb-127); eb in [0,254] -> exact except eb=254
#pragma unroll
      for (int e = 0; e < 16; ++e) x[e] = (eb == 0) ? x[e] * 1.7014118346046923e38f : x[e] * inv;
    } else {
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (SMODE == CUDA_LLM_SCALE_PER_TOKEN) {
        tsc = fmaxf(__fdiv_rn(amax, 448.f), 1e-8f);
        const Divisor dv(tsc);  // |x / tsc| <= 448 (1 + 2^-23)
        dv.div_all(x);
      } else {
        const float sc = (SMODE == CUDA_LLM_SCALE_PER_BLOCK)
                             ? reinterpret_cast<const float*>(scale)[(size_t)(slot_ok ? blk : 0) * a.Hkv + h]
                             : reinterpret_cast<const float*>(scale)[h];
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] = __fdiv_rn(x[e], sc);
      }
    }
    // ---- codes: 16 bytes of E4M3, or 8 bytes of E2M1 nibble pairs (low nibble = even d)
    uint32_t c[4] = {0u, 0u, 0u, 0u};
    if (!fp4) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        c[j] = f32x2_to_e4m3x2(x[4 * j], x[4 * j + 1]) | (f32x2_to_e4m3x2(x[4 * j + 2], x[4 * j + 3]) << 16);
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          c[j] |= (quant_e2m1_nibble(x[8 * j + 2 * e]) | (quant_e2m1_nibble(x[8 * j + 2 * e + 1]) << 4)) << (8 * e);
    }
    if (!slot_ok) continue;
    if (fast) {
      if (!fp4) *reinterpret_cast<uint4*>(&tile[is_v][tl][d0 / 4]) = make_uint4(c[0], c[1], c[2], c[3]);
      else *reinterpret_cast<uint2*>(&tile[is_v][tl][d0 / 8]) = make_uint2(c[0], c[1]);
      if (SMODE == CUDA_LLM_SCALE_PER_TOKEN && sub == 0) tok_scales[is_v][tl] = tsc;
      if (SMODE == CUDA_LLM_SCALE_MX_E8M0 && (sub & 1) == 0) mx_scales[is_v][sub >> 1][tl] = (uint8_t)eb;
    } else {
      uint8_t* cache = is_v ? a.vc : a.kc;
      if (SMODE == CUDA_LLM_SCALE_PER_TOKEN && sub == 0)
        reinterpret_cast<float*>(scale)[((size_t)blk * a.Hkv + h) * a.page + off] = tsc;
      if (SMODE == CUDA_LLM_SCALE_MX_E8M0 && (sub & 1) == 0)
        reinterpret_cast<uint8_t*>(scale)[(((size_t)blk * a.Hkv + h) * NB + (sub >> 1)) * a.page + off] = (uint8_t)eb;
      if (!fp4) {
        uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * D + d0) * a.page + off;
#pragma unroll
        for (int e = 0; e < 16; ++e) dst[(size_t)e * a.page] = (uint8_t)(c[e >> 2] >> (8 * (e & 3)));
      } else {
        uint8_t* dst = cache + (((size_t)blk * a.Hkv + h) * (D / 2) + d0 / 2) * a.page + off;
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[(size_t)e * a.page] = (uint8_t)(c[e >> 2] >> (8 * (e & 3)));
      }
    }
  }
  if (!fast) return;
  __syncthreads();
  const int blk = s_blk, off0 = s_off0;
  const int is_v = warp & 1;
  if (warp < 2) {
    // ---- codes: lane takes byte rows 4*lane .. 4*lane+3 of the tile, all 16 tokens
    const int rows = (is_v && fp4v) ? D / 2 : D;
    if (4 * lane < rows) {
      uint32_t o[4][4];  // [row][token quad]
#pragma unroll
      for (int tq = 0; tq < 4; ++tq) {
        const uint32_t w0 = tile[is_v][4 * tq][lane], w1 = tile[is_v][4 * tq + 1][lane];
        const uint32_t w2 = tile[is_v][4 * tq + 2][lane], w3 = tile[is_v][4 * tq + 3][lane];
        // 4 x 4 byte transpose: word j of the result = byte j of w0, w1, w2, w3
        const uint32_t lo01 = prmt(w0, w1, 0x5140), lo23 = prmt(w2, w3, 0x5140);
        const uint32_t hi01 = prmt(w0, w1, 0x7362), hi23 = prmt(w2, w3, 0x7362);
        o[0][tq] = prmt(lo01, lo23, 0x5410);
        o[1][tq] = prmt(lo01, lo23, 0x7632);
        o[2][tq] = prmt(hi01, hi23, 0x5410);
        o[3][tq] = prmt(hi01, hi23, 0x7632);
      }
      uint8_t* dst = (is_v ? a.vc : a.kc) + (((size_t)blk * a.Hkv + h) * rows + 4 * lane) * a.page + off0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(dst + (size_t)j * a.page) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
    }
  } else {
    // ---- scales of the 16 tokens
    void* scale = is_v ? a.vs : a.ks;
    if (SMODE == CUDA_LLM_SCALE_PER_TOKEN) {
      if (lane < 16) reinterpret_cast<float*>(scale)[((size_t)blk * a.Hkv + h) * a.page + off0 + lane] = tok_scales[is_v][lane];
    } else if (SMODE == CUDA_LLM_SCALE_MX_E8M0) {
      if (lane < NB * 4) {
        const int b = lane >> 2, part = lane & 3;
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(scale) + (((size_t)blk * a.Hkv + h) * NB + b) * a.page + off0 + 4 * part) =
            *reinterpret_cast<const uint32_t*>(&mx_scales[is_v][b][4 * part]);
      }
    }
  }
}

constexpr int kAppendTileMinTokens = 1024;  // below this the per-token kernel has more warps in flight

cudaError_t launch_kv_append(AppendArgs a, int D, cudaStream_t st) {
  if (a.n == 0) return cudaSuccess;
  // full-width rows need 16-byte aligned caches (every page slab then is) and 4-byte aligned scales
  a.aligned = !(((uintptr_t)a.kc | (uintptr_t)a.vc) & 15) && !(((uintptr_t)a.ks | (uintptr_t)a.vs) & 3) && (a.page % 16 == 0);
  a.src_vec = !(((uintptr_t)a.k_new | (uintptr_t)a.v_new) & 15);
  if (a.n < kAppendTileMinTokens || !a.aligned) {
    const long long items = 2LL * a.n * a.Hkv;
    const unsigned grid = (unsigned)((items + 3) / 4);
    if (D == 64) kv_append_token_kernel<64><<<grid, 128, 0, st>>>(a);
    else kv_append_token_kernel<128><<<grid, 128, 0, st>>>(a);
    return cudaGetLastError();
  }
  const long long groups = ((long long)a.n + 15) / 16;
  const unsigned grid = (unsigned)(groups * a.Hkv);
  const int dt = a.src_vec ? a.in_dtype : -1;
  auto go = [&](auto d_tag, auto dt_tag) {
    constexpr int DD = decltype(d_tag)::value;
    constexpr int T = decltype(dt_tag)::value;
    switch (a.scale_mode) {
      case CUDA_LLM_SCALE_PER_HEAD: kv_append_tile_kernel<DD, T, CUDA_LLM_SCALE_PER_HEAD><<<grid, 128, 0, st>>>(a); break;
      case CUDA_LLM_SCALE_PER_BLOCK: kv_append_tile_kernel<DD, T, CUDA_LLM_SCALE_PER_BLOCK><<<grid, 128, 0, st>>>(a); break;
      case CUDA_LLM_SCALE_PER_TOKEN: kv_append_tile_kernel<DD, T, CUDA_LLM_SCALE_PER_TOKEN><<<grid, 128, 0, st>>>(a); break;
      default: kv_append_tile_kernel<DD, T, CUDA_LLM_SCALE_MX_E8M0><<<grid, 128, 0, st>>>(a); break;
    }
  };
  auto go_d = [&](auto d_tag) {
    if (dt == CUDA_LLM_F32) go(d_tag, std::integral_constant<int, CUDA_LLM_F32>{});
    else if (dt == CUDA_LLM_F16) go(d_tag, std::integral_constant<int, CUDA_LLM_F16>{});
    else if (dt == CUDA_LLM_BF16) go(d_tag, std::integral_constant<int, CUDA_LLM_BF16>{});
    else go(d_tag, std::integral_constant<int, -1>{});
  };
  if (D == 64) go_d(std::integral_constant<int, 64>{});
  else go_d(std::integral_constant<int, 128>{});
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
