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
// Pages of 32 / 64 tokens (an extension; the reference supports 16 only) have rows of 128 / 256 bytes, so a
// 16-token tile of a slab is not contiguous: it is fetched as one TMA box (16 tokens x head_dim rows, no
// swizzle) through a tensor map over the cache and lands in the slot in the same [head_dim][16] shape.
//
// The same kernel serves the reference's contiguous fp32 K/V (async_flash_decode_kernel.cuh:29-220, tensors
// [B, H, S, D], one token = one row of head_dim floats) as its token-major mode: a slot then holds 16
// consecutive token rows, lane (dq, tl) = (lane & 7, lane >> 3) reads the 16 bytes of head_dim values
// 32kb + 4dq .. +3 of token rows tl, tl + 4, ... (again 128 contiguous bytes per phase), dot products are
// summed over dq and outputs over tl.
//
// Waits are bounded (mbar_wait); a warp whose wait runs out records CUDA_LLM_ST_TIMEOUT in the status
// word, waits (bounded) for its own copies still in flight and returns.
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "paged_decode_kernel.cuh"

namespace b200 {

cudaError_t launch_merge_partials(const float*, const float*, int, long long, int, void*, int, float*,
                                  cudaStream_t);

constexpr int kF32Warps = 7;    // workers per CTA
constexpr int kF32Slots = 4;    // ring slots per worker (K, V, K, V)
constexpr int kF32MinChunk = 8;       // pages per item, lower and upper bound
constexpr int kF32MaxSplits = 512;    // partial results per query row
constexpr long long kF32TargetItems = 8192;

struct F32TensorMaps {
  CUtensorMap k, v;   // cache [num_blocks][Hkv * D][page] fp32, box = 16 tokens x D rows (pages of 32 / 64 tokens)
};

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
  int S, Hq, Hkv, group, max_blocks, num_blocks, n_splits, chunk_pages, n_rg;  // chunk_pages: 16-token tiles per item
  int page;           // tokens per page (16: bulk copies of whole slabs; 32 / 64: TMA boxes)
  int seq_len;        // token-major mode: tokens of every sequence (bt and ctx are null)
  long long n_items;
  float scale_log2;
  int stall_test;     // failure-path test: the copy of the first K slab of sequence 0 is announced and never sent
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

template <int D, int GP, bool TM>
__global__ void __launch_bounds__(32 * kF32Warps, 1)
paged_f32_decode_kernel(const PagedF32Args a, const __grid_constant__ F32TensorMaps tmaps) {
  constexpr int KK = D / 8;                  // head_dim values per lane
  constexpr int KB = D / 32;                 // token-major: 32-wide head_dim blocks
  constexpr uint32_t SLOT = D * 16 * 4;      // bytes of a slab
  constexpr float NEG_INF = -__builtin_huge_valf();
  extern __shared__ __align__(128) uint8_t smem_f32[];
  __shared__ __align__(8) uint64_t bars[kF32Warps][kF32Slots];
  __shared__ int2 queue[kF32Warps][4];       // items issued and not yet consumed: (item, live tokens)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tq = lane & 3, dl = lane >> 2;   // paged: token quad, head_dim row
  const int dq = lane & 7, tl = lane >> 3;   // token-major: head_dim quad, token row
  uint8_t* ring = smem_f32 + ((128u - (smem_u32(smem_f32) & 127u)) & 127u) + (size_t)warp * kF32Slots * SLOT;
  const uint32_t ring_u32 = smem_u32(ring);
  const int tpp = a.page >> 4;  // 16-token tiles per page
  const uint32_t bar0 = smem_u32(&bars[warp][0]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kF32Slots; ++i) mbar_init(bar0 + 8 * i, 1);
    mbar_fence_init();
  }
  __syncwarp();
  asm volatile("griddepcontrol.launch_dependents;");  // the merge may be scheduled; it waits for this grid's end
  const uint64_t policy = l2_policy_evict_first();
  const size_t rows_total = (size_t)a.S * a.Hq;

  // ---- issue side: a cursor over the pages of the item being fetched
  uint32_t iseq = 0, cseq = 0;  // slots issued / consumed
  int it_kvh = 0, it_page = 0, it_npages = 0, it_kv = 0, it_first_blk = 0, it_s = 0, it_ntok = 0;
  int it_bt = 0;                // lane j: block-table entry bt_base + j of the sequence
  int bt_base = 0;
  bool it_have = false, it_done = false;
  int qw = 0, qr = 0;           // queue write / read positions
  int next_raw = 0;             // lane 0: the item the next acquire takes (fetched one item ahead)
  if (lane == 0) next_raw = (int)atomicAdd(a.counter, 1u);

  // Items are numbered chunk-major: every sequence's first chunk comes before any second chunk.  The
  // chunks handed out last are then the high ones, which short sequences do not have and longer ones
  // fill only partly, so the work left for the end is fine-grained and the warps finish together.
  auto item_coords = [&](long long item, int& s, int& kvh, int& split, int& rg) {
    rg = (int)(item % a.n_rg);
    item /= a.n_rg;
    kvh = (int)(item % a.Hkv);
    item /= a.Hkv;
    s = (int)(item % a.S);
    split = (int)(item / a.S);
  };
  auto load_bt = [&](int first_page) {  // the 32 block-table entries from `first_page` on
    if (TM) return;
    bt_base = first_page;
    const int pg = first_page + lane;
    int b = pg < a.max_blocks ? a.bt[(size_t)it_s * a.max_blocks + pg] : 0;
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
      int ctx = TM ? a.seq_len : a.ctx[s];
      if (!TM) ctx = max(0, min(ctx, a.max_blocks * a.page));
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
      it_ntok = n_tok;
      it_have = true;
      load_bt(it_first_blk / (TM ? 1 : tpp));
      if (lane == 0) queue[warp][qw & 3] = make_int2((int)item, n_tok);
      ++qw;
      break;
    }
  };
  auto issue_one = [&]() {
    if (!it_have) acquire();
    if (!it_have) return;
    const float* src;
    uint32_t bytes = SLOT;
    if (TM) {
      // 16 consecutive token rows of this (sequence, KV head); the last tile of a sequence may be shorter
      const size_t tok = (size_t)(it_first_blk + it_page) * 16;
      src = (it_kv ? a.v : a.k) + (((size_t)it_s * a.Hkv + it_kvh) * a.seq_len + tok) * D;
      bytes = (uint32_t)min(16, it_ntok - it_page * 16) * (D * 4);
    }
    int blk = 0, tile_in_page = 0;
    if (!TM) {
      const int tile = it_first_blk + it_page;   // 16-token tile of the sequence
      const int pg = tile / tpp;
      tile_in_page = tile - pg * tpp;
      if (pg - bt_base >= 32) load_bt(pg);
      blk = __shfl_sync(0xffffffffu, it_bt, pg - bt_base);
      if (blk < 0 || blk >= a.num_blocks) {
        if (lane == 0) atomicOr(a.status, CUDA_LLM_ST_BAD_BLOCK);
        blk = 0;
      }
      src = (it_kv ? a.v : a.k) + ((size_t)blk * a.Hkv + it_kvh) * (size_t)(D * 16);
    }
    const uint32_t slot = iseq % kF32Slots;
    if (lane == 0) {
      mbar_arrive_expect_tx(bar0 + 8 * slot, bytes);
      if (!(a.stall_test && (it_s | it_kvh | it_first_blk | it_page | it_kv) == 0)) {  // first K slab of the launch
        if (!TM && tpp > 1)
          tma_load_3d_hint(ring_u32 + slot * SLOT, it_kv ? &tmaps.v : &tmaps.k, tile_in_page * 16, it_kvh * D, blk,
                           bar0 + 8 * slot, policy);
        else
          bulk_g2s_hint(ring_u32 + slot * SLOT, src, bytes, bar0 + 8 * slot, policy);
      }
    }
    ++iseq;
    it_kv ^= 1;
    if (it_kv == 0) {
      ++it_page;
      if (it_page == it_npages) it_have = false;
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
      if (!mbar_wait(bar0 + 8 * slot, (cseq / kF32Slots) & 1, a.stall_test)) {
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
            // paged: head_dim dl + 8kk; token-major: head_dim 32 (kk / 4) + 4dq + kk % 4
            const int d = TM ? 32 * (kk >> 2) + 4 * dq + (kk & 3) : dl + 8 * kk;
            qv[r][kk] = (r < c_rows) ? qp[(size_t)r * D + d] : 0.f;
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
      if (TM) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int kb = 0; kb < KB; ++kb) {
            const float4 kv = ks[(tl + 4 * j) * (D / 4) + 8 * kb + dq];
#pragma unroll
            for (int r = 0; r < GP; ++r)
              sc[r][j] = fmaf(qv[r][4 * kb + 3], kv.w, fmaf(qv[r][4 * kb + 2], kv.z,
                         fmaf(qv[r][4 * kb + 1], kv.y, fmaf(qv[r][4 * kb], kv.x, sc[r][j]))));
          }
      } else {
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
      }
      __syncwarp();  // every lane has read the slab: the slot may be refilled
      ++cseq;
      fill();
      // sum over the eight lanes that share the tokens (paged: dl, token-major: dq)
#pragma unroll
      for (int o = TM ? 1 : 4; o < (TM ? 8 : 32); o <<= 1)
#pragma unroll
        for (int r = 0; r < GP; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) sc[r][j] += __shfl_xor_sync(0xffffffffu, sc[r][j], o);
      // token of sc[.][j] within the item: paged 4tq + j, token-major tl + 4j
      const int tok = c_page * 16 + (TM ? tl : 4 * tq);
      constexpr int TSTEP = TM ? 4 : 1;
      bool rescale = false;
      float alpha[GP];
#pragma unroll
      for (int r = 0; r < GP; ++r) {
        float x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = (tok + TSTEP * j < c_ntok) ? sc[r][j] * a.scale_log2 : NEG_INF;
        float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, TM ? 8 : 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, TM ? 16 : 2));
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
        l_run[r] = l_run[r] * alpha[r] + ps;  // over this lane's tokens; summed over tq / tl at the end
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
      if (!mbar_wait(bar0 + 8 * slot, (cseq / kF32Slots) & 1, a.stall_test)) {
        give_up();
        return;
      }
      const float4* vs = reinterpret_cast<const float4*>(ring + slot * SLOT);
      if (TM) {
        // a dead token row may hold anything (the copy of a short last tile leaves old bytes behind):
        // its probability is exactly 0, and its values are replaced by 0 so that 0 * NaN cannot occur
        const bool tail = c_ntok - c_page * 16 < 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool live_tok = !tail || (c_page * 16 + tl + 4 * j < c_ntok);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb) {
            float4 vv = vs[(tl + 4 * j) * (D / 4) + 8 * kb + dq];
            if (!live_tok) vv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < GP; ++r) {
              acc[r][4 * kb] = fmaf(p[r][j], vv.x, acc[r][4 * kb]);
              acc[r][4 * kb + 1] = fmaf(p[r][j], vv.y, acc[r][4 * kb + 1]);
              acc[r][4 * kb + 2] = fmaf(p[r][j], vv.z, acc[r][4 * kb + 2]);
              acc[r][4 * kb + 3] = fmaf(p[r][j], vv.w, acc[r][4 * kb + 3]);
            }
          }
        }
      } else if (c_ntok - (c_page * 16 + 4 * tq) >= 4) {
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          const float4 vv = vs[(dl + 8 * kk) * 4 + tq];
#pragma unroll
          for (int r = 0; r < GP; ++r)
            acc[r][kk] = fmaf(p[r][3], vv.w, fmaf(p[r][2], vv.z, fmaf(p[r][1], vv.y, fmaf(p[r][0], vv.x, acc[r][kk]))));
        }
      } else {
        // the tail of the sequence: a dead slot may hold anything, 0 * NaN must not reach the accumulator
        const int left = c_ntok - (c_page * 16 + 4 * tq);  // live tokens among this lane's four
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
        l += __shfl_xor_sync(0xffffffffu, l, TM ? 8 : 1);
        l += __shfl_xor_sync(0xffffffffu, l, TM ? 16 : 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
          float v = acc[r][kk];
          v += __shfl_xor_sync(0xffffffffu, v, TM ? 8 : 1);
          v += __shfl_xor_sync(0xffffffffu, v, TM ? 16 : 2);
          acc[r][kk] = v * inv;
        }
        if (r < c_rows && TM) {
          // lane (dq, tl) stores the four values of head_dim block tl: 32 consecutive floats per 8 lanes
          float* po = a.part_o + (c_row0 + r) * D;
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            if (tl == kb)
              *reinterpret_cast<float4*>(po + 32 * kb + 4 * dq) =
                  make_float4(acc[r][4 * kb], acc[r][4 * kb + 1], acc[r][4 * kb + 2], acc[r][4 * kb + 3]);
          if (lane == 0) a.part_lse[c_row0 + r] = l > 0.f ? (m_run[r] + log2f(l)) * 0.69314718055994531f : NEG_INF;
        } else if (r < c_rows) {
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

template <int D, int GP, bool TM>
static cudaError_t launch_f32(const PagedF32Args& a, const F32TensorMaps& maps, int grid, cudaStream_t st) {
  const size_t dyn = (size_t)kF32Warps * kF32Slots * D * 16 * 4 + 128;  // + room to align the rings to 128 bytes
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 64 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(paged_f32_decode_kernel<D, GP, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
    if (e != cudaSuccess) return e;
    if (dev < 64) attr_set[dev] = true;
  }
  paged_f32_decode_kernel<D, GP, TM><<<grid, 32 * kF32Warps, dyn, st>>>(a, maps);
  return cudaGetLastError();
}

size_t paged_f32_decode_workspace_bytes(int S, int Hq, int Hkv, int D, int max_tokens) {
  int chunk, n;
  f32_split_plan(S, Hkv, Hq / (Hkv > 0 ? Hkv : 1), (max_tokens + 15) / 16, chunk, n);
  const size_t rows = (size_t)S * Hq;
  return 256 + ((size_t)n * rows * sizeof(float) + 255) / 256 * 256 + (size_t)n * rows * D * sizeof(float);
}

bool paged_f32_decode_supported(int D, int page, const void* k, const void* v) {
  return (page == 16 || page == 32 || page == 64) && (D == 64 || D == 128) && !(((uintptr_t)k | (uintptr_t)v) & 15);
}

// `paged`: K/V are caches [num_blocks, Hkv, D, page] read through bt / ctx (`maps`: their tensor maps, used for
// pages of 32 / 64 tokens, may be null for 16); otherwise contiguous tensors [S, Hkv, seq_len, D] (bt and ctx unused,
// page 16, max_blocks = tiles that cover seq_len).
cudaError_t run_paged_f32_decode(bool paged, const void* q, const void* k, const void* v, const int32_t* bt,
                                 const int32_t* ctx, void* out, int S, int Hq, int Hkv, int D, int page, int max_blocks,
                                 int num_blocks, int seq_len, float softmax_scale, void* workspace, int num_sms,
                                 const F32TensorMaps* maps, cudaStream_t st) {
  PagedF32Args a;
  a.q = reinterpret_cast<const float*>(q);
  a.k = reinterpret_cast<const float*>(k);
  a.v = reinterpret_cast<const float*>(v);
  a.bt = bt; a.ctx = ctx;
  a.S = S; a.Hq = Hq; a.Hkv = Hkv; a.group = Hq / Hkv; a.max_blocks = max_blocks; a.num_blocks = num_blocks;
  a.seq_len = seq_len;
  a.page = page;
  f32_split_plan(S, Hkv, a.group, max_blocks * (page / 16), a.chunk_pages, a.n_splits);
  a.n_rg = (a.group + 3) / 4;
  a.n_items = (long long)S * Hkv * a.n_splits * a.n_rg;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  {  // CUDA_LLM_TEST_STALL=1: the failure-path test of this kernel (its entry points carry no flags word)
    const char* env = getenv("CUDA_LLM_TEST_STALL");
    a.stall_test = (env && env[0] == '1') ? 1 : 0;
  }
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
  F32TensorMaps tm;
  if (maps) tm = *maps;
  else memset(&tm, 0, sizeof(tm));
  auto go = [&](auto d_tag, auto tm_tag) -> cudaError_t {
    constexpr int DD = decltype(d_tag)::value;
    constexpr bool T = decltype(tm_tag)::value;
    return gp == 1 ? launch_f32<DD, 1, T>(a, tm, grid, st) : gp == 2 ? launch_f32<DD, 2, T>(a, tm, grid, st) : launch_f32<DD, 4, T>(a, tm, grid, st);
  };
  using I64 = std::integral_constant<int, 64>;
  using I128 = std::integral_constant<int, 128>;
  if (paged) e = (D == 64) ? go(I64{}, std::false_type{}) : go(I128{}, std::false_type{});
  else e = (D == 64) ? go(I64{}, std::true_type{}) : go(I128{}, std::true_type{});
  if (e != cudaSuccess) return e;
  return launch_merge_partials(a.part_o, a.part_lse, a.n_splits, (long long)rows, D, out, CUDA_LLM_F32, nullptr, st);
}

}  // namespace b200
