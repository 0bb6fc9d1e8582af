// Decode attention over an fp32 paged cache with pages of 16 tokens: the float instantiation of the
// reference's paged_attention_kernel (paged_attention_kernel.cuh:20-145 in the reference project, layout
// cache[num_blocks, heads, head_dim, page], token innermost), shaped for HBM bandwidth.
//
// fp32 needs fp32 arithmetic (the reference's own tolerance for this dtype is 1e-4), and at 4 bytes per
// element the FMA pipe has room for it: a K or V element costs one FMA per query row of the GQA group,
// 17-34 % of the FMA rate at the HBM rate for groups of 4-8.  What the straightforward kernel lacked was
// bytes in flight, so this one is built around the copy engine:
//
// * One warp = one worker with its own ring of four shared-memory slots.  A slot holds the K or the V slab
//   of one (page, KV head): head_dim rows of 16 tokens, 64 contiguous bytes each, 8 KB for head_dim 128,
//   fetched by ONE bulk copy that signals the slot's mbarrier.  The warp that consumes a slot refills it, so
//   there is no producer warp and no empty barrier; seven warps per SM keep up to 168 KB in flight.
// * Work items are (sequence, KV head, token chunk, row group of four query rows), handed out through
//   an atomic counter, so the warps of the GPU finish together whatever the context lengths are.  An
//   item leaves a normalised partial row and its log-sum-exp per query row; merge_partials_kernel
//   combines the chunks.
// * Lane (tq, dl) = (lane & 3, lane >> 2) reads, for head_dim rows dl, dl + 8, ..., the 16 bytes of tokens
//   4tq .. 4tq+3: the eight lanes of a shared-memory phase cover 128 contiguous bytes (no bank conflicts),
//   both in Q.K (query values of the lane's rows in registers, partial dot products summed over dl with
//   three butterfly steps) and in P.V (the lane multiplies by the probabilities of exactly the tokens it
//   scored, so P never moves; partial outputs are summed over tq once per item).
//
// Waits are bounded (mbar_wait); a warp whose wait runs out records CUDA_LLM_ST_TIMEOUT in the status
// word, waits (bounded) for its own copies still in flight and returns.
#include "paged_decode_kernel.cuh"

namespace b200 {

cudaError_t launch_merge_partials(const float*, const float*, int, long long, int, void*, int, float*,
                                  cudaStream_t);

constexpr int kF32Warps = 7;    // workers per CTA
constexpr int kF32Slots = 4;    // ring slots per worker (K, V, K, V)
constexpr int kF32MinChunk = 8;       // pages per item, lower and upper bound
constexpr int kF32MaxSplits = 256;    // partial results per query row
constexpr long long kF32TargetItems = 8192;

struct PagedF32Args {
  const float* q;    // [S, Hq, D]
  const float* k;    // [num_blocks, Hkv, D, 16]
  const float* v;
  const int32_t* bt;
  const int32_t* ctx;
  float* part_o;     // [n_splits, S*Hq, D]
  float* part_lse;   // [n_splits, S*Hq]   natural log
  uint32_t* status;
  uint32_t* counter;  // next item
  int S, Hq, Hkv, group, max_blocks, num_blocks, n_splits, chunk_pages, n_rg;
  long long n_items;
  float scale_log2;
};

// (chunk_pages, n_splits) for a launch: about kF32TargetItems items when every sequence is full, chunks of
// at least kF32MinChunk pages, at most kF32MaxSplits chunks per sequence.
static void f32_split_plan(int S, int Hkv, int group, int max_pages, int& chunk_pages, int& n_splits) {
  const int n_rg = (group + 3) / 4;
  const long long total = (long long)S * Hkv * n_rg * (max_pages > 0 ? max_pages : 1);
  long long c = (total + kF32TargetItems - 1) / kF32TargetItems;
  if (c < kF32MinChunk) c = kF32MinChunk;
  const long long floor_c = ((long long)max_pages + kF32MaxSplits - 1) / kF32MaxSplits;
  if (c < floor_c) c = floor_c;
  if (c > max_pages && max_pages > 0) c = max_pages;
  if (c < 1) c = 1;
  chunk_pages = (int)c;
  n_splits = max_pages > 0 ? (int)((max_pages + c - 1) / c) : 1;
}

template <int D, int GP>
__global__ void __launch_bounds__(32 * kF32Warps, 1) paged_f32_decode_kernel(const PagedF32Args a) {
  constexpr int KK = D / 8;                  // head_dim rows per lane
  constexpr uint32_t SLOT = D * 16 * 4;      // bytes of a slab
  constexpr float NEG_INF = -__builtin_huge_valf();
  extern __shared__ __align__(128) uint8_t smem_f32[];
  __shared__ __align__(8) uint64_t bars[kF32Warps][kF32Slots];
  __shared__ int2 queue[kF32Warps][4];       // items issued and not yet consumed: (item, live tokens)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tq = lane & 3, dl = lane >> 2;
  uint8_t* ring = smem_f32 + (size_t)warp * kF32Slots * SLOT;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t bar0 = smem_u32(&bars[warp][0]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kF32Slots; ++i) mbar_init(bar0 + 8 * i, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const uint64_t policy = l2_policy_evict_first();
  const size_t rows_total = (size_t)a.S * a.Hq;

  // ---- issue side: a cursor over the pages of the item being fetched
  uint32_t iseq = 0, cseq = 0;  // slots issued / consumed
  int it_kvh = 0, it_page = 0, it_npages = 0, it_kv = 0, it_first_blk = 0, it_s = 0;
  int it_bt = 0;                // lane j: block of page (it_page & ~31) + j of the item
  bool it_have = false, it_done = false;
  int qw = 0, qr = 0;           // queue write / read positions
  int next_raw = 0;             // lane 0: the item the next acquire takes (fetched one item ahead)
  if (lane == 0) next_raw = (int)atomicAdd(a.counter, 1u);

  auto item_coords = [&](long long item, int& s, int& kvh, int& split, int& rg) {
    rg = (int)(item % a.n_rg);
    item /= a.n_rg;
    split = (int)(item % a.n_splits);
    item /= a.n_splits;
    kvh = (int)(item % a.Hkv);
    s = (int)(item / a.Hkv);
  };
  auto load_bt = [&]() {
    const int pg = it_first_blk + (it_page & ~31) + lane;
    int b = (pg < a.max_blocks && (it_page & ~31) + lane < it_npages) ? a.bt[(size_t)it_s * a.max_blocks + pg] : 0;
    if (b < 0 || b >= a.num_blocks) {
      atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
      b = 0;
    }
    it_bt = b;
  };
  auto acquire = [&]() {
    while (!it_done) {
      const long long item = __shfl_sync(0xffffffffu, next_raw, 0);
      if (item >= a.n_items) {
        it_done = true;
        break;
      }
      if (lane == 0) next_raw = (int)atomicAdd(a.counter, 1u);
      int s, kvh, split, rg;
      item_coords(item, s, kvh, split, rg);
      int ctx = a.ctx[s];
      ctx = max(0, min(ctx, a.max_blocks * 16));
      const int t0 = split * a.chunk_pages * 16;
      const int n_tok = max(0, min(ctx - t0, a.chunk_pages * 16));
      if (n_tok == 0) {
        // nothing to read: the partial rows of this chunk are zeros with weight zero
        for (int r = 0; r < GP; ++r) {
          const int gr = rg * GP + r;
          if (gr >= a.group) break;
          const size_t row = (size_t)split * rows_total + (size_t)s * a.Hq + (size_t)kvh * a.group + gr;
          for (int d = lane; d < D; d += 32) a.part_o[row * D + d] = 0.f;
          if (lane == 0) a.part_lse[row] = NEG_INF;
        }
        continue;
      }
      it_s = s;
      it_kvh = kvh;
      it_npages = (n_tok + 15) >> 4;
      it_page = 0;
      it_kv = 0;
      it_first_blk = t0 >> 4;
      it_have = true;
      load_bt();
      if (lane == 0) queue[warp][qw & 3] = make_int2((int)item, n_tok);
      ++qw;
      break;
    }
  };
  auto issue_one = [&]() {
    if (!it_have) acquire();
    if (!it_have) return;
    const int blk = __shfl_sync(0xffffffffu, it_bt, it_page & 31);
    const float* src = (it_kv ? a.v : a.k) + ((size_t)blk * a.Hkv + it_kvh) * (size_t)(D * 16);
    const uint32_t slot = iseq % kF32Slots;
    if (lane == 0) {
      mbar_arrive_expect_tx(bar0 + 8 * slot, SLOT);
      bulk_g2s_hint(ring_u32 + slot * SLOT, src, SLOT, bar0 + 8 * slot, policy);
    }
    ++iseq;
    it_kv ^= 1;
    if (it_kv == 0) {
      ++it_page;
      if (it_page == it_npages) it_have = false;
      else if ((it_page & 31) == 0) load_bt();
    }
  };
  auto fill = [&]() {
    while (iseq - cseq < (uint32_t)kF32Slots && !(it_done && !it_have)) {
      const uint32_t before = iseq;
      issue_one();
      if (iseq == before) break;
    }
  };
  auto give_up = [&]() {
    if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_TIMEOUT);
    // this warp's own copies still in flight: wait (bounded) for them before leaving
    for (uint32_t e = cseq; e != iseq; ++e) (void)mbar_wait(bar0 + 8 * (e % kF32Slots), (e / kF32Slots) & 1, 1);
  };

  // ---- consume side
  float qv[GP][KK], acc[GP][KK], m_run[GP], l_run[GP], p[GP][4];
  int c_page = 0, c_npages = 0, c_ntok = 0;
  size_t c_row0 = 0;   // partial row of query row 0 of this item
  int c_rows = 0;      // live query rows of this item

  for (;;) {
    fill();
    if (cseq == iseq) break;
    // ------------------------------------------------------------ K slab: scores of 16 tokens
    {
      const uint32_t slot = cseq % kF32Slots;
      if (!mbar_wait(bar0 + 8 * slot, (cseq / kF32Slots) & 1, 0)) {
        give_up();
        return;
      }
      if (c_page == c_npages) {  // first page of the next item in the queue
        __syncwarp();
        const int2 qd = queue[warp][qr & 3];
        ++qr;
        int s, kvh, split, rg;
        item_coords(qd.x, s, kvh, split, rg);
        c_ntok = qd.y;
        c_npages = (c_ntok + 15) >> 4;
        c_page = 0;
        c_rows = min(GP, a.group - rg * GP);
        c_row0 = (size_t)split * rows_total + (size_t)s * a.Hq + (size_t)kvh * a.group + rg * GP;
        const float* qp = a.q + ((size_t)s * a.Hq + (size_t)kvh * a.group + rg * GP) * D;
#pragma unroll
        for (int r = 0; r < GP; ++r) {
#pragma unroll
          for (int kk = 0; kk < KK; ++kk) {
            qv[r][kk] = (r < c_rows) ? qp[(size_t)r * D + dl + 8 * kk] : 0.f;
            acc[r][kk] = 0.f;
          }
          m_run[r] = -1.0e30f;  // a finite floor: max - max never becomes inf - inf
          l_run[r] = 0.f;
        }
      }
      const float4* ks = reinterpret_cast<const float4*>(ring + slot * SLOT);
      float sc[GP][4];
#pragma unroll
      for (int r = 0; r < GP; ++r) sc[r][0] = sc[r][1] = sc[r][2] = sc[r][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        const float4 kv = ks[(dl + 8 * kk) * 4 + tq];
#pragma unroll
        for (int r = 0; r < GP; ++r) {
          sc[r][0] = fmaf(qv[r][kk], kv.x, sc[r][0]);
          sc[r][1] = fmaf(qv[r][kk], kv.y, sc[r][1]);
          sc[r][2] = fmaf(qv[r][kk], kv.z, sc[r][2]);
          sc[r][3] = fmaf(qv[r][kk], kv.w, sc[r][3]);
        }
      }
      __syncwarp();  // every lane has read the slab: the slot may be refilled
      ++cseq;
      fill();
      // sum over the eight dl lanes
#pragma unroll
      for (int o = 4; o < 32; o <<= 1)
#pragma unroll
        for (int r = 0; r < GP; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) sc[r][j] += __shfl_xor_sync(0xffffffffu, sc[r][j], o);
      const int tok = c_page * 16 + 4 * tq;  // first token of this lane within the item
      bool rescale = false;
      float alpha[GP];
#pragma unroll
      for (int r = 0; r < GP; ++r) {
        float x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = (tok + j < c_ntok) ? sc[r][j] * a.scale_log2 : NEG_INF;
        float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m_run[r], mx);
        alpha[r] = fast_exp2(m_run[r] - mn);
        rescale |= (alpha[r] != 1.f);
        m_run[r] = mn;
        float ps = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          p[r][j] = fast_exp2(x[j] - mn);
          ps += p[r][j];
        }
        l_run[r] = l_run[r] * alpha[r] + ps;  // over this lane's tokens; summed over tq at the end
      }
      if (rescale) {  // uniform over the warp: every lane holds the same maxima
#pragma unroll
        for (int r = 0; r < GP; ++r)
#pragma unroll
          for (int kk = 0; kk < KK; ++kk) acc[r][kk] *= alpha[r];
      }
    }
    // ------------------------------------------------------------ V slab: O += P V
    {
      const uint32_t slot = cseq % kF32Slots;
      if (!mbar_wait(bar0 + 8 * slot, (cseq / kF32Slots) & 1, 0)) {
        give_up();
        return;
      }
      const float4* vs = reinterpret_cast<const float4*>(ring + slot * SLOT);
      const int left = c_ntok - (c_page * 16 + 4 * tq);  // live tokens among this lane's four
      if (left >= 4) {
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          const float4 vv = vs[(dl + 8 * kk) * 4 + tq];
#pragma unroll
          for (int r = 0; r < GP; ++r)
            acc[r][kk] = fmaf(p[r][3], vv.w, fmaf(p[r][2], vv.z, fmaf(p[r][1], vv.y, fmaf(p[r][0], vv.x, acc[r][kk]))));
        }
      } else {
        // the tail of the sequence: a dead slot may hold anything, 0 * NaN must not reach the accumulator
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          float4 vv = vs[(dl + 8 * kk) * 4 + tq];
          vv.x = left > 0 ? vv.x : 0.f;
          vv.y = left > 1 ? vv.y : 0.f;
          vv.z = left > 2 ? vv.z : 0.f;
          vv.w = 0.f;
#pragma unroll
          for (int r = 0; r < GP; ++r)
            acc[r][kk] = fmaf(p[r][2], vv.z, fmaf(p[r][1], vv.y, fmaf(p[r][0], vv.x, acc[r][kk])));
        }
      }
      __syncwarp();
      ++cseq;
      ++c_page;
    }
    if (c_page == c_npages) {
      // ---------------------------------------------------------- end of the item: partial rows
#pragma unroll
      for (int r = 0; r < GP; ++r) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          float v = acc[r][kk];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          acc[r][kk] = v * inv;
        }
        if (r < c_rows) {
          float* po = a.part_o + (c_row0 + r) * D;
          // lane (tq, dl) stores head_dim rows dl + 8 * (4i + tq): 32 consecutive floats per instruction
#pragma unroll
          for (int i = 0; i < KK / 4; ++i) {
            const float v = tq == 0 ? acc[r][4 * i] : tq == 1 ? acc[r][4 * i + 1] : tq == 2 ? acc[r][4 * i + 2] : acc[r][4 * i + 3];
            po[dl + 8 * (4 * i + tq)] = v;
          }
          if (lane == 0) a.part_lse[c_row0 + r] = l > 0.f ? (m_run[r] + log2f(l)) * 0.69314718055994531f : NEG_INF;
        }
      }
    }
  }
}

template <int D, int GP>
static cudaError_t launch_f32(const PagedF32Args& a, int grid, cudaStream_t st) {
  const size_t dyn = (size_t)kF32Warps * kF32Slots * D * 16 * 4;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 64 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(paged_f32_decode_kernel<D, GP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
    if (e != cudaSuccess) return e;
    if (dev < 64) attr_set[dev] = true;
  }
  paged_f32_decode_kernel<D, GP><<<grid, 32 * kF32Warps, dyn, st>>>(a);
  return cudaGetLastError();
}

size_t paged_f32_decode_workspace_bytes(int S, int Hq, int Hkv, int D, int max_tokens) {
  int chunk, n;
  f32_split_plan(S, Hkv, Hq / (Hkv > 0 ? Hkv : 1), (max_tokens + 15) / 16, chunk, n);
  const size_t rows = (size_t)S * Hq;
  return 256 + ((size_t)n * rows * sizeof(float) + 255) / 256 * 256 + (size_t)n * rows * D * sizeof(float);
}

bool paged_f32_decode_supported(int D, int page, const void* k, const void* v) {
  return page == 16 && (D == 64 || D == 128) && !(((uintptr_t)k | (uintptr_t)v) & 15);
}

cudaError_t run_paged_f32_decode(const void* q, const void* k, const void* v, const int32_t* bt, const int32_t* ctx,
                                 void* out, int S, int Hq, int Hkv, int D, int max_blocks, int num_blocks,
                                 float softmax_scale, void* workspace, int num_sms, cudaStream_t st) {
  PagedF32Args a;
  a.q = reinterpret_cast<const float*>(q);
  a.k = reinterpret_cast<const float*>(k);
  a.v = reinterpret_cast<const float*>(v);
  a.bt = bt; a.ctx = ctx;
  a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.group = Hq / Hkv; a.max_blocks = max_blocks; a.num_blocks = num_blocks;
  f32_split_plan(S, Hkv, a.group, max_blocks, a.chunk_pages, a.n_splits);
  a.n_rg = (a.group + 3) / 4;
  a.n_items = (long long)S * Hkv * a.n_splits * a.n_rg;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  const size_t rows = (size_t)S * Hq;
  a.status = reinterpret_cast<uint32_t*>(ws);
  a.counter = reinterpret_cast<uint32_t*>(ws + 128);
  a.part_lse = reinterpret_cast<float*>(ws + 256);
  a.part_o = reinterpret_cast<float*>(ws + 256 + ((size_t)a.n_splits * rows * sizeof(float) + 255) / 256 * 256);
  if (a.n_items == 0) return cudaSuccess;
  cudaError_t e = cudaMemsetAsync(a.counter, 0, 4, st);
  if (e != cudaSuccess) return e;
  const int grid = num_sms > 0 ? num_sms : 148;
  const int gp = a.group >= 3 ? 4 : a.group;
  if (D == 64) e = gp == 1 ? launch_f32<64, 1>(a, grid, st) : gp == 2 ? launch_f32<64, 2>(a, grid, st) : launch_f32<64, 4>(a, grid, st);
  else e = gp == 1 ? launch_f32<128, 1>(a, grid, st) : gp == 2 ? launch_f32<128, 2>(a, grid, st) : launch_f32<128, 4>(a, grid, st);
  if (e != cudaSuccess) return e;
  return launch_merge_partials(a.part_o, a.part_lse, a.n_splits, (long long)rows, D, out, CUDA_LLM_F32, nullptr, st);
}

}  // namespace b200
