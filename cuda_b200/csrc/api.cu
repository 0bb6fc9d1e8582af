// C ABI of libcuda_llm_b200: argument validation, shared-memory / workspace layout and
// kernel selection for the paged decode path.  Mirrors the checks the reference binding makes
// before it calls dispatch_fp8_paged_attention (fused_softmax_binding.cpp:645-669 in the
// reference project) and turns the dispatcher's silent no-op on an unsupported shape
// (fp8_paged_attention_kernel.cuh:176-190) into an error code.
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <atomic>
#include <mutex>

#include "decode_launch.cuh"

namespace b200 {
cudaError_t launch_merge_partials(const float*, const float*, int, long long, int, void*, int,
                                  float*, cudaStream_t);
cudaError_t launch_dequant_pages(const void*, const void*, const int32_t*, int, int, int, int, int,
                                 int, float*, cudaStream_t);

cudaError_t run_gqa_prefill(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hkv, int S,
                            int D, float softmax_scale, bool causal, int dtype, cudaStream_t st);
bool gqa_prefill_sm100_supported(int Hq, int Hkv, int D, int dtype);
cudaError_t launch_mx_to_f16(const void* codes, const float* scales, void* out, size_t n_elems, cudaStream_t st);
cudaError_t run_gqa_prefill_sm100(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hkv, int S,
                                  int D, float softmax_scale, bool causal, int dtype, int out_dtype, cudaStream_t st);
cudaError_t prefill_wait_timeouts(unsigned int* count);
cudaError_t run_mx_attention(const void* q, const float* qs, const void* k, const float* ks, const void* v,
                             const float* vs, void* out, int B, int Hq, int Hkv, int S, int D, float softmax_scale,
                             bool causal, int out_dtype, cudaStream_t st);
cudaError_t run_kv_append_prefill(const void* k, const void* v, const CudaLlmKvCacheTarget& c, int B, int Hkv, int S,
                                  int D, int in_dtype, cudaStream_t st);
size_t dense_decode_workspace_bytes(int S, int Hq, int Hkv, int D, int max_tokens);
size_t paged_f32_decode_workspace_bytes(int S, int Hq, int Hkv, int D, int max_tokens);
bool paged_f32_decode_supported(int D, int page, const void* k, const void* v);
struct F32TensorMaps {
  CUtensorMap k, v;
};
cudaError_t run_paged_f32_decode(bool paged, const void* q, const void* k, const void* v, const int32_t* bt,
                                 const int32_t* ctx, void* out, int S, int Hq, int Hkv, int D, int page, int max_blocks,
                                 int num_blocks, int seq_len, float softmax_scale, void* workspace, int num_sms,
                                 const F32TensorMaps* maps, cudaStream_t st);
cudaError_t run_dense_decode(bool paged, const void* q, const void* k, const void* v, const int32_t* bt,
                             const int32_t* ctx, void* out, int S, int Hq, int Hkv, int D, int page,
                             int max_blocks, int num_blocks, int seq_len, float softmax_scale, int dtype,
                             void* workspace, cudaStream_t st);

static thread_local char g_err[256] = "";
static int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
  return CUDA_LLM_ECUDA;
}
static int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

void set_error_message(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct Layout {
  int HG, SUBS, tok_stage, n_hg, NT, rows_max, PPS, n_stages, grid;
  uint32_t stage_bytes, off_v, off_ks, off_vs;
  uint32_t k_page_stride, v_page_stride, ks_page_stride, vs_page_stride;
  uint32_t k_chunk, v_chunk, ks_chunk, vs_chunk;
  size_t smem_bytes;
  uint32_t q_smem_off, q_smem_bytes;  // per-slot query area behind the stages (0: does not fit)
  int q_smem_tokens;                  // query tokens per sequence one area holds
  // workspace
  size_t ws_table, ws_lse, ws_o, ws_total;
};

static int sm_count_cached() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 64) dev = 63;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    counts[dev] = n;
  }
  return counts[dev];
}

// CUDA_LLM_OK when the current device is an sm_100 part (the only target of this library).
static int check_device() {
  static int major_of[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  const int slot = dev < 64 ? dev : 63;
  if (!major_of[slot]) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceGetAttribute");
    major_of[slot] = major;
  }
  if (major_of[slot] != 10) return fail(CUDA_LLM_EDEVICE, "this library holds sm_100a code only; the current device is not an sm_100 GPU");
  return CUDA_LLM_OK;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point look-up (libcuda is not linked).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

EncodeTiledFn tensor_map_encoder() { return encode_tiled_fn(); }

// Tensor map of a paged cache [num_blocks][Hkv * D][page] of 1- or 2-byte elements: boxes of `box_rows`
// head_dim lines of one page, swizzled over the 64 or 128 bytes of a line.
static int encode_cache_map(CUtensorMap* map, const void* cache, int num_blocks, int Hkv, int D, int page, int box_rows,
                            int elem_bytes = 2) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(CUDA_LLM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t eb = (cuuint64_t)elem_bytes;
  const cuuint64_t dims[3] = {(cuuint64_t)page, (cuuint64_t)Hkv * D, (cuuint64_t)num_blocks};
  const cuuint64_t strides[2] = {(cuuint64_t)page * eb, (cuuint64_t)Hkv * D * page * eb};
  const cuuint32_t box[3] = {(cuuint32_t)page, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                         const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, page * elem_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[96];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return fail(CUDA_LLM_ECUDA, msg);
  }
  return CUDA_LLM_OK;
}

// Tensor map of an fp32 paged cache [num_blocks][Hkv * D][page]: boxes of 16 tokens x D head_dim rows, as stored.
static int encode_f32_cache_map(CUtensorMap* map, const void* cache, int num_blocks, int Hkv, int D, int page) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(CUDA_LLM_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {(cuuint64_t)page, (cuuint64_t)Hkv * D, (cuuint64_t)num_blocks};
  const cuuint64_t strides[2] = {(cuuint64_t)page * 4, (cuuint64_t)Hkv * D * page * 4};
  const cuuint32_t box[3] = {16, (cuuint32_t)D, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[96];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return fail(CUDA_LLM_ECUDA, msg);
  }
  return CUDA_LLM_OK;
}

// Pure arithmetic (no device access when num_ctas > 0): shared-memory stage layout and
// workspace carving for one problem shape.
static int make_layout(int S, int Hq, int Hkv, int D, int page, int max_q_len, int k_format, int v_format,
                       int scale_mode, int num_ctas, Layout& L, bool token_major = false, int q_elem_bytes = 2) {
  if (S < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return fail(CUDA_LLM_EINVAL, "num_q_heads must be a positive multiple of num_kv_heads");
  if (D != 64 && D != 128) return fail(CUDA_LLM_EINVAL, "Only head_dim 64 and 128 supported");
  if (page != 16 && page != 32 && page != 64) return fail(CUDA_LLM_EINVAL, "Only page_size 16, 32 and 64 supported");
  const int group = Hq / Hkv;
  if (max_q_len < 1) max_q_len = 1;
  if (group * max_q_len > 16) return fail(CUDA_LLM_EINVAL, "(num_q_heads/num_kv_heads) * max_q_len must be <= 16");
  L.NT = (group * max_q_len <= 8) ? 1 : 2;
  L.rows_max = 8 * L.NT;
  // An 8-bit stage holds 256 (token, head) pairs, a 16-bit stage 128: the same bytes.
  const bool kv16 = (k_format == CUDA_LLM_KV_F16 || k_format == CUDA_LLM_KV_BF16);
  const int eb = kv16 ? 2 : 1;
  const int pairs = 256 / eb;
  int HG = 8;
  while (Hkv % HG) HG >>= 1;
  while (pairs / HG < page) HG >>= 1;  // a stage must hold whole pages
  if (token_major) HG = (Hkv % 2 == 0) ? 2 : 1;  // contiguous K/V: a stage is 128 / HG consecutive tokens of HG heads
  L.HG = HG;
  // 16 consumer warps, 8 bit: NT == 1 -> (HG heads) x (16/HG sub-tiles of 16 tokens);
  //                           NT == 2 -> 2 row halves x (HG heads) x (8/HG sub-tiles of 32 tokens)
  //                    16 bit: NT == 1 -> 2 stage parities x (HG heads) x (8/HG sub-tiles of 16 tokens)
  //                           NT == 2 -> 2 row halves x the same
  // either way a (CTA, head) leaves SUBS results of rows_max rows
  L.SUBS = (L.NT == 1 ? 16 : 8) / HG;
  L.tok_stage = pairs / HG;
  L.n_hg = Hkv / HG;
  L.PPS = token_major ? 1 : (L.tok_stage >= page) ? L.tok_stage / page : 1;
  if (L.PPS > kMaxPagesPerStage) return fail(CUDA_LLM_EINVAL, "internal: too many pages per stage");
  const uint32_t pad = 0;  // every 16-token m-tile lies inside one page: no padding between pages
  const int DV = (v_format == CUDA_LLM_KV_FP4_E2M1) ? D / 2 : D;
  L.k_chunk = token_major ? (uint32_t)L.tok_stage * D * eb : (uint32_t)HG * D * page * eb;
  L.v_chunk = token_major ? L.k_chunk : (uint32_t)HG * DV * page * eb;
  if (kv16) L.ks_chunk = L.vs_chunk = 0;
  else if (scale_mode == CUDA_LLM_SCALE_PER_TOKEN) L.ks_chunk = L.vs_chunk = (uint32_t)HG * page * 4;
  else if (scale_mode == CUDA_LLM_SCALE_MX_E8M0) L.ks_chunk = L.vs_chunk = (uint32_t)HG * (D / 32) * page;
  else L.ks_chunk = L.vs_chunk = 0;
  L.k_page_stride = (token_major ? HG : 1) * L.k_chunk + pad;  // token-major: k_chunk is one head's rows
  L.v_page_stride = (token_major ? HG : 1) * L.v_chunk + pad;
  L.ks_page_stride = L.ks_chunk;
  L.vs_page_stride = L.vs_chunk;
  L.off_v = L.PPS * L.k_page_stride;
  L.off_ks = L.off_v + L.PPS * L.v_page_stride;
  L.off_vs = L.off_ks + L.PPS * L.ks_page_stride;
  L.stage_bytes = (uint32_t)align_up(L.off_vs + L.PPS * L.vs_page_stride, 128);
  const uint32_t stages_off = kStagesOff;
  int ns = (int)((kSmemBudget - stages_off) / L.stage_bytes);
  if (ns > kMaxStages) ns = kMaxStages;
  if (ns < 2) return fail(CUDA_LLM_EINVAL, "internal: stage does not fit in shared memory twice");
  L.n_stages = ns;
  L.smem_bytes = stages_off + (size_t)ns * L.stage_bytes;
  if (L.smem_bytes < stages_off + kDecodeThreads * 8) L.smem_bytes = stages_off + kDecodeThreads * 8;
  // Query rows of one (sequence, head group), one area per ring slot, in the shared memory that is
  // left: as many query tokens per sequence as fit (sequences with more keep the global path).  A
  // ring deeper than three stages gives one stage up if that makes room for at least one token.
  L.q_smem_off = L.q_smem_bytes = 0;
  L.q_smem_tokens = 0;
  for (;;) {
    const size_t token_bytes = (size_t)HG * group * D * q_elem_bytes;
    const size_t off = align_up(stages_off + (size_t)ns * L.stage_bytes, 128);
    const size_t room = off < kSmemBudget ? (kSmemBudget - off) / ns / 128 * 128 : 0;
    int tokens = (int)(room / token_bytes);
    if (tokens > max_q_len) tokens = max_q_len;
    if (tokens >= 1) {
      L.n_stages = ns;
      L.q_smem_off = (uint32_t)off;
      L.q_smem_bytes = (uint32_t)align_up((size_t)tokens * token_bytes, 128);
      L.q_smem_tokens = tokens;
      L.smem_bytes = off + (size_t)ns * L.q_smem_bytes;
      break;
    }
    if (ns <= 3) break;
    --ns;
  }
  if (num_ctas <= 0) num_ctas = sm_count_cached();
  if (num_ctas <= 0) return fail(CUDA_LLM_ECUDA, "cannot query the SM count");
  L.grid = num_ctas;
  const size_t n_slots = (size_t)S * L.n_hg + L.grid;
  const size_t rows = n_slots * L.SUBS * L.HG * L.rows_max;
  L.ws_table = 256;
  L.ws_lse = align_up(L.ws_table + (size_t)S * L.n_hg * 16, 256);
  L.ws_o = align_up(L.ws_lse + rows * 4, 256);
  L.ws_total = align_up(L.ws_o + rows * D * 4, 256);
  return CUDA_LLM_OK;
}

// Work layout of the tcgen05 decode kernel (paged_decode_sm100.cu): two adjacent KV heads per unit, tiles of
// 128 tokens, one result of `rows_max` rows per (CTA, sequence, KV head).
// `q_lens_given`: the call carries cu_q_lens.  A query may then be longer than max_q_len declares and still be
// served as long as it fits the rows of the launch, so the four-row variant is for calls without query lengths only
// (one token per sequence); with them the launch has the 8 or 16 rows the default kernel would have.
static int make_layout_sm100(int S, int Hq, int Hkv, int D, int page, int max_q_len, int v_format, int scale_mode,
                             int num_ctas, bool q_lens_given, Layout& L) {
  if (S < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hkv % 2 || D != 128 || page != 16) return CUDA_LLM_EINVAL;
  const int group = Hq / Hkv;
  if (max_q_len < 1) max_q_len = 1;
  if (group * max_q_len > 16) return CUDA_LLM_EINVAL;
  memset(&L, 0, sizeof(L));
  L.NT = (group * max_q_len <= 8) ? 1 : 2;
  L.rows_max = (group * max_q_len <= 4 && !q_lens_given) ? 4 : 8 * L.NT;  // the kernel's padded row counts: 4, 8, 16
  L.HG = 2;
  L.SUBS = 1;
  L.tok_stage = 128;
  L.n_hg = Hkv / 2;
  L.PPS = 128 / page;
  const int DV = (v_format == CUDA_LLM_KV_FP4_E2M1) ? D / 2 : D;
  L.k_chunk = 2u * D * page;   // both heads of a pair are contiguous in a page
  L.v_chunk = 2u * DV * page;
  L.ks_chunk = L.vs_chunk = 2u * ((scale_mode == CUDA_LLM_SCALE_PER_TOKEN) ? (uint32_t)page * 4 : (uint32_t)(D / 32) * page);
  if (num_ctas <= 0) num_ctas = sm_count_cached();
  if (num_ctas <= 0) return fail(CUDA_LLM_ECUDA, "cannot query the SM count");
  L.grid = num_ctas;
  const size_t n_slots = (size_t)S * L.n_hg + L.grid;
  const size_t rows = n_slots * L.SUBS * L.HG * L.rows_max;
  L.ws_table = 256;
  L.ws_lse = align_up(L.ws_table + (size_t)S * L.n_hg * 16, 256);
  L.ws_o = align_up(L.ws_lse + rows * 4, 256);
  L.ws_total = align_up(L.ws_o + rows * D * 4, 256);
  return CUDA_LLM_OK;
}

cudaError_t launch_paged_decode_sm100(const DecodeArgs& a, int mode, int rp, int grid, cudaStream_t st);
unsigned int decode100_wait_timeouts();
static std::atomic<uint64_t> g_sm100_launches{0};
static std::atomic<uint64_t> g_f32_launches{0};

// The tcgen05 kernel serves head_dim 128, an even number of KV heads, pages of 16 tokens, E4M3 K and V with
// per-token fp32 or E8M0 block scales and 16-bit queries, when the call (CUDA_LLM_FLAG_TCGEN05) or the process
// (CUDA_LLM_DECODE_KERNEL=tcgen05) asks for it.
static bool decode_sm100_wanted(const CudaLlmPagedDecodeParams* p) {
  const bool kv16 = (p->k_format == CUDA_LLM_KV_F16 || p->k_format == CUDA_LLM_KV_BF16);
  if (kv16 || p->head_dim != 128 || p->page_size != 16 || (p->num_kv_heads & 1)) return false;
  if (p->k_format != CUDA_LLM_KV_FP8_E4M3 || p->v_format != CUDA_LLM_KV_FP8_E4M3) return false;
  if (p->scale_mode != CUDA_LLM_SCALE_PER_TOKEN && p->scale_mode != CUDA_LLM_SCALE_MX_E8M0) return false;
  if (p->q_dtype == CUDA_LLM_F32 || p->rope_cos || p->rope_sin) return false;
  if (((uintptr_t)p->query & 7) != 0) return false;
  if (p->flags & CUDA_LLM_FLAG_TCGEN05) return true;
  const char* v = getenv("CUDA_LLM_DECODE_KERNEL");
  return v != nullptr && strcmp(v, "tcgen05") == 0;
}

using LaunchFn = cudaError_t (*)(const DecodeArgs&, const KvTensorMaps&, int, size_t, cudaStream_t);

template <int D, int MODE>
static LaunchFn pick_page_nt(int page, int NT, bool precise) {
#define B200_PICK(P)                                                             \
  if (page == P) {                                                               \
    if (NT == 2) return launch_paged_decode<D, P, MODE, 2, false>;               \
    return precise ? launch_paged_decode<D, P, MODE, 1, true>                    \
                   : launch_paged_decode<D, P, MODE, 1, false>;                  \
  }
  B200_PICK(16)
  B200_PICK(32)
  B200_PICK(64)
#undef B200_PICK
  return nullptr;
}
template <int MODE>
static LaunchFn pick_d(int D, int page, int NT, bool precise) {
  return D == 64 ? pick_page_nt<64, MODE>(page, NT, precise) : pick_page_nt<128, MODE>(page, NT, precise);
}
template <int D, int MODE>
static LaunchFn pick_kv16_page(int page, int NT) {
  if (page == 16) return NT == 2 ? launch_paged_decode<D, 16, MODE, 2, false> : launch_paged_decode<D, 16, MODE, 1, false>;
  if (page == 32) return NT == 2 ? launch_paged_decode<D, 32, MODE, 2, false> : launch_paged_decode<D, 32, MODE, 1, false>;
  if (page == 64) return NT == 2 ? launch_paged_decode<D, 64, MODE, 2, false> : launch_paged_decode<D, 64, MODE, 1, false>;
  return nullptr;
}
static LaunchFn pick_kv16(bool bf16, int D, int page, int NT) {
  if (bf16) return D == 64 ? pick_kv16_page<64, MODE_KV_BF16>(page, NT) : pick_kv16_page<128, MODE_KV_BF16>(page, NT);
  return D == 64 ? pick_kv16_page<64, MODE_KV_F16>(page, NT) : pick_kv16_page<128, MODE_KV_F16>(page, NT);
}

}  // namespace b200

using namespace b200;

// Scratch for cuda_llm_paged_decode_static(): lives in the library image, one copy per GPU that
// loads it, for the life of the process.  Host code may not pass this name to a kernel (on the
// host it is only a handle for the symbol); its device address is looked up once per device.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

extern "C" {

const char* cuda_llm_last_cuda_error(void) { return g_err; }
const char* cuda_llm_version(void) { return "cuda_llm_b200 0.1 (sm_100a)"; }

size_t cuda_llm_paged_decode_workspace_bytes(int32_t num_seqs, int32_t num_q_heads,
                                             int32_t num_kv_heads, int32_t head_dim,
                                             int32_t page_size, int32_t max_q_len,
                                             int32_t num_ctas) {
  Layout L;
  // the workspace does not depend on the formats
  if (make_layout(num_seqs, num_q_heads, num_kv_heads, head_dim, page_size, max_q_len, CUDA_LLM_KV_FP8_E4M3,
                  CUDA_LLM_KV_FP8_E4M3, CUDA_LLM_SCALE_PER_TOKEN, num_ctas, L) != CUDA_LLM_OK)
    return 0;
  size_t need = L.ws_total;  // a 16-bit cache may group fewer heads per stage: cover it too
  if (make_layout(num_seqs, num_q_heads, num_kv_heads, head_dim, page_size, max_q_len, CUDA_LLM_KV_BF16,
                  CUDA_LLM_KV_BF16, CUDA_LLM_SCALE_PER_HEAD, num_ctas, L) == CUDA_LLM_OK && L.ws_total > need)
    need = L.ws_total;
  // and the tcgen05 kernel's one-head units
  if (make_layout_sm100(num_seqs, num_q_heads, num_kv_heads, head_dim, page_size, max_q_len, CUDA_LLM_KV_FP8_E4M3,
                        CUDA_LLM_SCALE_PER_TOKEN, num_ctas, true, L) == CUDA_LLM_OK && L.ws_total > need)
    need = L.ws_total;
  return need;
}

int cuda_llm_paged_decode(const CudaLlmPagedDecodeParams* p, void* stream) {
  if (!p) return fail(CUDA_LLM_EINVAL, "params is null");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (p->num_seqs == 0) return CUDA_LLM_OK;
  if (!p->query || !p->key_cache || !p->value_cache || !p->block_tables || !p->context_lens || !p->out)
    return fail(CUDA_LLM_EINVAL, "a required tensor pointer is null");
  const bool kv16 = (p->k_format == CUDA_LLM_KV_F16 || p->k_format == CUDA_LLM_KV_BF16);
  if (kv16) {
    if (p->v_format != p->k_format) return fail(CUDA_LLM_EINVAL, "a 16-bit cache needs K and V of the same format");
  } else {
    if (!p->k_scale || !p->v_scale) return fail(CUDA_LLM_EINVAL, "scale tensors are required for a quantised cache");
    if (p->k_format != CUDA_LLM_KV_FP8_E4M3)
      return fail(CUDA_LLM_EINVAL, "K must be FP8-E4M3, fp16 or bf16 (the int8 reading of the reference kernel is not provided)");
    if (p->v_format != CUDA_LLM_KV_FP8_E4M3 && p->v_format != CUDA_LLM_KV_FP4_E2M1)
      return fail(CUDA_LLM_EINVAL, "V must be FP8-E4M3 or FP4-E2M1");
    if (p->v_format == CUDA_LLM_KV_FP4_E2M1 && p->scale_mode != CUDA_LLM_SCALE_MX_E8M0)
      return fail(CUDA_LLM_EINVAL, "FP4 V needs E8M0 block scales");
    if (p->scale_mode < 0 || p->scale_mode > CUDA_LLM_SCALE_MX_E8M0) return fail(CUDA_LLM_EINVAL, "unknown scale_mode");
  }
  if (p->q_dtype < 0 || p->q_dtype > CUDA_LLM_BF16 || p->out_dtype < 0 || p->out_dtype > CUDA_LLM_BF16)
    return fail(CUDA_LLM_EINVAL, "unknown dtype");
  if (p->max_blocks_per_seq <= 0 || p->num_blocks <= 0) return fail(CUDA_LLM_EINVAL, "max_blocks_per_seq and num_blocks must be positive");
  const uintptr_t al = (uintptr_t)p->key_cache | (uintptr_t)p->value_cache | (kv16 ? 0 : (uintptr_t)p->k_scale) |
                       (kv16 ? 0 : (uintptr_t)p->v_scale) | (uintptr_t)p->workspace;
  if (al & 15) return fail(CUDA_LLM_EALIGN, "caches, scales and workspace must be 16-byte aligned");

  Layout L;
  int rc = make_layout(p->num_seqs, p->num_q_heads, p->num_kv_heads, p->head_dim, p->page_size,
                       p->max_q_len, p->k_format, p->v_format, p->scale_mode, p->num_ctas, L, false,
                       p->q_dtype == CUDA_LLM_F32 ? 4 : 2);
  if (rc != CUDA_LLM_OK) return rc;
  const bool sm100 = decode_sm100_wanted(p);
  if (sm100) {
    rc = make_layout_sm100(p->num_seqs, p->num_q_heads, p->num_kv_heads, p->head_dim, p->page_size, p->max_q_len,
                           p->v_format, p->scale_mode, p->num_ctas, p->cu_q_lens != nullptr, L);
    if (rc != CUDA_LLM_OK) return rc;
  }
  if (!p->workspace || p->workspace_bytes < L.ws_total)
    return fail(CUDA_LLM_EWORKSPACE, "workspace missing or smaller than cuda_llm_paged_decode_workspace_bytes()");

  const int D = p->head_dim, page = p->page_size, Hkv = p->num_kv_heads;
  const int DV = (p->v_format == CUDA_LLM_KV_FP4_E2M1) ? D / 2 : D;
  DecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.q = p->query;
  a.kc = (const uint8_t*)p->key_cache;
  a.vc = (const uint8_t*)p->value_cache;
  a.ks = (const uint8_t*)p->k_scale;
  a.vs = (const uint8_t*)p->v_scale;
  a.bt = p->block_tables;
  a.ctx = p->context_lens;
  a.cuq = p->cu_q_lens;
  a.out = p->out;
  a.lse = p->lse;
  uint8_t* ws = (uint8_t*)p->workspace;
  a.status = (uint32_t*)ws;
  a.table = (int32_t*)(ws + L.ws_table);
  a.part_lse = (float*)(ws + L.ws_lse);
  a.part_o = (float*)(ws + L.ws_o);
  a.S = p->num_seqs;
  a.Hq = p->num_q_heads;
  a.Hkv = Hkv;
  a.group = p->num_q_heads / Hkv;
  a.max_blocks = p->max_blocks_per_seq;
  a.num_blocks = p->num_blocks;
  a.HG = L.HG;
  a.SUBS = L.SUBS;
  a.tok_stage = L.tok_stage;
  a.n_hg = L.n_hg;
  a.rows_max = L.rows_max;
  a.q_dtype = p->q_dtype;
  a.out_dtype = p->out_dtype;
  a.per_block = !kv16 && (p->scale_mode == CUDA_LLM_SCALE_PER_BLOCK);
  a.helper_pairs = (kv16 || sm100) ? 0 : 1;
  a.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  a.n_stages = L.n_stages;
  if (!sm100 && !((uintptr_t)p->query & 15)) {  // bulk copies need a 16-byte aligned source
    a.q_smem_off = L.q_smem_off;
    a.q_smem_bytes = L.q_smem_bytes;
    a.q_smem_tokens = L.q_smem_tokens;
  }
  if (p->rope_cos || p->rope_sin) {
    if (!p->rope_cos || !p->rope_sin || p->rope_num_positions <= 0)
      return fail(CUDA_LLM_EINVAL, "rotary embedding needs both tables and rope_num_positions > 0");
    if (((uintptr_t)p->rope_cos | (uintptr_t)p->rope_sin) & 7) return fail(CUDA_LLM_EALIGN, "rotary tables must be 8-byte aligned");
    a.rope_cos = p->rope_cos;
    a.rope_sin = p->rope_sin;
    a.rope_pos = p->rope_positions;
    a.rope_positions = p->rope_num_positions;
  }
  a.early_plan = (p->flags & CUDA_LLM_FLAG_STABLE_METADATA) ? 1 : 0;
  a.grid = L.grid;
  a.n_slots = p->num_seqs * L.n_hg + L.grid;
  a.stall_test = (p->flags & CUDA_LLM_FLAG_TEST_STALL) ? 1 : 0;
  a.short_waits = a.stall_test;
#ifdef CUDA_LLM_DIAGNOSTICS
  if (p->flags & CUDA_LLM_FLAG_DIAG_NO_MATH) a.debug |= 1;
  if (p->flags & CUDA_LLM_FLAG_DIAG_NO_COPY) a.debug |= 2;
  if (p->flags & CUDA_LLM_FLAG_DIAG_NO_SCALE_COPY) a.debug |= 16;
  if (p->flags & CUDA_LLM_FLAG_DIAG_REVERSED) a.debug |= 32;
  if (p->flags & CUDA_LLM_FLAG_DIAG_TRACE) {  // per-CTA timestamps go where the lse would go
    a.debug |= 4;
    a.trace = reinterpret_cast<unsigned long long*>(p->lse);
    a.lse = nullptr;
  }
  {
    const int ns_req = (p->flags >> 8) & 0xF;  // cap the ring depth
    if (ns_req >= 2 && ns_req < a.n_stages) a.n_stages = ns_req;
  }
#endif
  a.stage_bytes = L.stage_bytes;
  a.off_v = L.off_v;
  a.off_ks = L.off_ks;
  a.off_vs = L.off_vs;
  a.k_page_stride = L.k_page_stride;
  a.v_page_stride = L.v_page_stride;
  a.ks_page_stride = L.ks_page_stride;
  a.vs_page_stride = L.vs_page_stride;
  a.k_chunk = L.k_chunk;
  a.v_chunk = L.v_chunk;
  a.ks_chunk = L.ks_chunk;
  a.vs_chunk = L.vs_chunk;
  a.k_blk_stride = (uint64_t)Hkv * D * page * (kv16 ? 2 : 1);
  a.v_blk_stride = (uint64_t)Hkv * DV * page * (kv16 ? 2 : 1);
  if (kv16) a.ks_blk_stride = a.vs_blk_stride = 0;
  else if (p->scale_mode == CUDA_LLM_SCALE_PER_TOKEN) a.ks_blk_stride = a.vs_blk_stride = (uint64_t)Hkv * page * 4;
  else if (p->scale_mode == CUDA_LLM_SCALE_MX_E8M0) a.ks_blk_stride = a.vs_blk_stride = (uint64_t)Hkv * (D / 32) * page;

  const bool precise = (p->q_dtype == CUDA_LLM_F32) && L.NT == 1;
  if (sm100) {
    rc = check_device();
    if (rc != CUDA_LLM_OK) return rc;
    a.n_stages = 0;  // the kernel's own ring depth
#ifdef CUDA_LLM_DIAGNOSTICS
    a.n_stages = (p->flags >> 8) & 0xF;
#endif
    cudaError_t e = launch_paged_decode_sm100(a, p->scale_mode == CUDA_LLM_SCALE_PER_TOKEN ? MODE_TOKEN_SCALE : MODE_MX8,
                                              L.rows_max, L.grid, st);
    if (e != cudaSuccess) return fail_cuda(e, "paged_decode_sm100_kernel launch");
    g_sm100_launches.fetch_add(1, std::memory_order_relaxed);
    if (p->flags & CUDA_LLM_FLAG_SKIP_MERGE) return CUDA_LLM_OK;
    e = launch_merge_splits<128>(a, page, L.grid, st);
    if (e != cudaSuccess) return fail_cuda(e, "merge_splits_kernel launch");
    return CUDA_LLM_OK;
  }
  LaunchFn fn = nullptr;
  if (kv16)
    fn = pick_kv16(p->k_format == CUDA_LLM_KV_BF16, D, page, L.NT);
  else if (p->scale_mode == CUDA_LLM_SCALE_PER_HEAD || p->scale_mode == CUDA_LLM_SCALE_PER_BLOCK)
    fn = pick_d<MODE_PAGE_SCALE>(D, page, L.NT, precise);
  else if (p->scale_mode == CUDA_LLM_SCALE_PER_TOKEN)
    fn = pick_d<MODE_TOKEN_SCALE>(D, page, L.NT, precise);
  else if (p->v_format == CUDA_LLM_KV_FP4_E2M1)
    fn = pick_d<MODE_MX8K_MX4V>(D, page, L.NT, precise);
  else
    fn = pick_d<MODE_MX8>(D, page, L.NT, precise);
  if (!fn) return fail(CUDA_LLM_EINVAL, "no kernel for this shape");

  rc = check_device();
  if (rc != CUDA_LLM_OK) return rc;
  KvTensorMaps tm;
  memset(&tm, 0, sizeof(tm));
  const bool e4m3_page64 = !kv16 && p->v_format == CUDA_LLM_KV_FP8_E4M3 && page == 64;
  if ((kv16 && page >= 32) || e4m3_page64) {
    // 16-bit pages of 32 / 64 tokens and 8-bit pages of 64 tokens (rows of 64 / 128 bytes) travel as swizzled
    // TMA boxes (at most 256 head_dim lines each)
    const int eb = kv16 ? 2 : 1;
    a.tma_box_rows = L.HG * D < 256 ? L.HG * D : 256;
    a.tma_boxes = (L.HG * D) / a.tma_box_rows;
    rc = encode_cache_map(&tm.k, p->key_cache, p->num_blocks, Hkv, D, page, a.tma_box_rows, eb);
    if (rc == CUDA_LLM_OK) rc = encode_cache_map(&tm.v, p->value_cache, p->num_blocks, Hkv, D, page, a.tma_box_rows, eb);
    if (rc != CUDA_LLM_OK) return rc;
  }
  cudaError_t e = fn(a, tm, L.grid, L.smem_bytes, st);
  if (e != cudaSuccess) return fail_cuda(e, "paged_decode_kernel launch");
  if (p->flags & CUDA_LLM_FLAG_SKIP_MERGE) return CUDA_LLM_OK;
  e = (D == 64) ? launch_merge_splits<64>(a, page, L.grid, st) : launch_merge_splits<128>(a, page, L.grid, st);
  if (e != cudaSuccess) return fail_cuda(e, "merge_splits_kernel launch");
  return CUDA_LLM_OK;
}

size_t cuda_llm_static_scratch_bytes(void) { return kStaticScratchBytes; }

// Device address of g_static_scratch on the current device, resolved (and its status word
// zeroed) the first time a device asks.  No allocation: a symbol look-up and a 256-byte memset.
static int static_scratch_address(cudaStream_t st, void** out) {
  static std::mutex mu;
  static void* scratch_addr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(CUDA_LLM_EINVAL, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!scratch_addr[dev]) {  // first use on this device: resolve the symbol with this device current
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    // the status word starts at zero; after that it is sticky until cuda_llm_static_decode_status
    e = cudaMemsetAsync(ptr, 0, 256, st);
    if (e != cudaSuccess) return fail_cuda(e, "clearing the static scratch header");
    scratch_addr[dev] = ptr;
  }
  *out = scratch_addr[dev];
  return CUDA_LLM_OK;
}

int cuda_llm_paged_decode_static(const CudaLlmPagedDecodeParams* p, void* stream) {
  if (!p) return fail(CUDA_LLM_EINVAL, "params is null");
  const size_t need = cuda_llm_paged_decode_workspace_bytes(p->num_seqs, p->num_q_heads, p->num_kv_heads,
                                                            p->head_dim, p->page_size, p->max_q_len, p->num_ctas);
  if (p->num_seqs > 0 && need == 0) return CUDA_LLM_EINVAL;  // message set by the layout check
  if (need > kStaticScratchBytes)
    return fail(CUDA_LLM_EWORKSPACE, "problem needs more scratch than the 16 MiB built into the library; "
                                     "use cuda_llm_paged_decode with a caller-provided workspace");
  void* scratch = nullptr;
  const int rc = static_scratch_address(reinterpret_cast<cudaStream_t>(stream), &scratch);
  if (rc != CUDA_LLM_OK) return rc;
  CudaLlmPagedDecodeParams q = *p;
  q.workspace = scratch;
  q.workspace_bytes = kStaticScratchBytes;
  return cuda_llm_paged_decode(&q, stream);
}

int cuda_llm_static_decode_status(void* stream, uint32_t* status_out) {
  if (!status_out) return fail(CUDA_LLM_EINVAL, "null argument");
  void* scratch = nullptr;
  const int rc = static_scratch_address(reinterpret_cast<cudaStream_t>(stream), &scratch);
  if (rc != CUDA_LLM_OK) return rc;
  return cuda_llm_decode_status(scratch, stream, status_out);
}

int cuda_llm_decode_status(void* workspace, void* stream, uint32_t* status_out) {
  if (!workspace || !status_out) return fail(CUDA_LLM_EINVAL, "null argument");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status_out, workspace, 4, cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return fail_cuda(e, "status copy");
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail_cuda(e, "status sync");
  if (*status_out) {
    e = cudaMemsetAsync(workspace, 0, 4, st);
    if (e != cudaSuccess) return fail_cuda(e, "status clear");
  }
  return CUDA_LLM_OK;
}

int cuda_llm_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 256) return fail(CUDA_LLM_EWORKSPACE, "workspace missing or too small");
  cudaError_t e = cudaMemsetAsync(workspace, 0, 256, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "workspace init");
}

int cuda_llm_dequant_pages(const void* cache, const void* scale, const int32_t* pages,
                           int32_t n_pages, int32_t num_kv_heads, int32_t head_dim,
                           int32_t page_size, int32_t format, int32_t scale_mode, float* out,
                           void* stream) {
  if (!cache || !scale || !pages || !out) return fail(CUDA_LLM_EINVAL, "null argument");
  if (head_dim % 32 || page_size <= 0 || num_kv_heads <= 0 || n_pages < 0) return fail(CUDA_LLM_EINVAL, "bad dimensions");
  if (format != CUDA_LLM_KV_FP8_E4M3 && format != CUDA_LLM_KV_FP4_E2M1) return fail(CUDA_LLM_EINVAL, "unknown format");
  if (scale_mode < 0 || scale_mode > CUDA_LLM_SCALE_MX_E8M0) return fail(CUDA_LLM_EINVAL, "unknown scale_mode");
  cudaError_t e = launch_dequant_pages(cache, scale, pages, n_pages, num_kv_heads, head_dim, page_size,
                                       format, scale_mode, out, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "dequant_pages_kernel launch");
}

static int check_dense(int S, int Hq, int Hkv, int D, int dtype) {
  if (S < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return fail(CUDA_LLM_EINVAL, "num_heads must be a positive multiple of num_kv_heads");
  if (Hq / Hkv > 8) return fail(CUDA_LLM_EINVAL, "num_heads / num_kv_heads must be <= 8");
  if (D != 64 && D != 128) return fail(CUDA_LLM_EINVAL, "Only head_dim 64 and 128 supported");
  if (dtype < 0 || dtype > CUDA_LLM_BF16) return fail(CUDA_LLM_EINVAL, "unknown dtype");
  return CUDA_LLM_OK;
}

size_t cuda_llm_dense_decode_workspace_bytes(int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads,
                                             int32_t head_dim, int32_t max_tokens) {
  if (check_dense(num_seqs, num_heads, num_kv_heads, head_dim, CUDA_LLM_F32) != CUDA_LLM_OK || max_tokens < 0) return 0;
  size_t need = dense_decode_workspace_bytes(num_seqs, num_heads, num_kv_heads, head_dim, max_tokens);
  {  // an fp32 cache with pages of 16 tokens runs on the bulk-copy kernel, which cuts sequences into more chunks
    const size_t f32 = paged_f32_decode_workspace_bytes(num_seqs, num_heads, num_kv_heads, head_dim, max_tokens);
    if (f32 > need) need = f32;
  }
  // a 16-bit paged cache runs on the persistent kernel: cover its split partials for every page size
  for (int page = 16; page <= 64; page *= 2) {
    Layout L;
    if (make_layout(num_seqs, num_heads, num_kv_heads, head_dim, page, 1, CUDA_LLM_KV_BF16, CUDA_LLM_KV_BF16,
                    CUDA_LLM_SCALE_PER_HEAD, 0, L) == CUDA_LLM_OK && L.ws_total > need)
      need = L.ws_total;
  }
  {  // contiguous 16-bit K/V: one head per stage
    Layout L;
    if (make_layout(num_seqs, num_heads, num_kv_heads, head_dim, 16, 1, CUDA_LLM_KV_BF16, CUDA_LLM_KV_BF16,
                    CUDA_LLM_SCALE_PER_HEAD, 0, L, true) == CUDA_LLM_OK && L.ws_total > need)
      need = L.ws_total;
  }
  return need;
}

int cuda_llm_paged_attention(const void* query, const void* key_cache, const void* value_cache,
                             const int32_t* block_tables, const int32_t* context_lens, void* out,
                             int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                             int32_t page_size, int32_t max_blocks_per_seq, int32_t num_blocks,
                             float softmax_scale, int32_t dtype, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (num_seqs == 0) return CUDA_LLM_OK;
  if (!query || !key_cache || !value_cache || !block_tables || !context_lens || !out)
    return fail(CUDA_LLM_EINVAL, "a required tensor pointer is null");
  int rc = check_dense(num_seqs, num_heads, num_kv_heads, head_dim, dtype);
  if (rc != CUDA_LLM_OK) return rc;
  if (page_size != 16 && page_size != 32 && page_size != 64) return fail(CUDA_LLM_EINVAL, "Only page_size 16, 32 and 64 supported");
  if (max_blocks_per_seq <= 0 || num_blocks <= 0) return fail(CUDA_LLM_EINVAL, "max_blocks_per_seq and num_blocks must be positive");
  const size_t need = cuda_llm_dense_decode_workspace_bytes(num_seqs, num_heads, num_kv_heads, head_dim, max_blocks_per_seq * page_size);
  if (!workspace || workspace_bytes < need) return fail(CUDA_LLM_EWORKSPACE, "workspace missing or smaller than cuda_llm_dense_decode_workspace_bytes()");
  if (dtype != CUDA_LLM_F32 && !(((uintptr_t)key_cache | (uintptr_t)value_cache | (uintptr_t)workspace) & 15)) {
    // 16-bit cache: the persistent tensor-core kernel (an fp32 cache stays on the SIMT kernel)
    CudaLlmPagedDecodeParams p;
    memset(&p, 0, sizeof(p));
    p.query = query; p.key_cache = key_cache; p.value_cache = value_cache;
    p.block_tables = block_tables; p.context_lens = context_lens; p.out = out;
    p.workspace = workspace; p.workspace_bytes = workspace_bytes;
    p.num_seqs = num_seqs; p.num_q_heads = num_heads; p.num_kv_heads = num_kv_heads;
    p.head_dim = head_dim; p.page_size = page_size; p.max_blocks_per_seq = max_blocks_per_seq;
    p.num_blocks = num_blocks; p.max_q_len = 1;
    p.q_dtype = p.out_dtype = dtype;
    p.k_format = p.v_format = (dtype == CUDA_LLM_F16) ? CUDA_LLM_KV_F16 : CUDA_LLM_KV_BF16;
    p.softmax_scale = softmax_scale;
    return cuda_llm_paged_decode(&p, stream);
  }
  if (dtype == CUDA_LLM_F32 && paged_f32_decode_supported(head_dim, page_size, key_cache, value_cache) &&
      !((uintptr_t)workspace & 15) && (page_size == 16 || (num_blocks < INT_MAX && encode_tiled_fn()))) {
    // (the C++ dispatchers of the reference carry no pool size and pass INT_MAX: they use pages of 16 tokens only)
    F32TensorMaps maps;
    memset(&maps, 0, sizeof(maps));
    if (page_size > 16) {
      rc = encode_f32_cache_map(&maps.k, key_cache, num_blocks, num_kv_heads, head_dim, page_size);
      if (rc == CUDA_LLM_OK) rc = encode_f32_cache_map(&maps.v, value_cache, num_blocks, num_kv_heads, head_dim, page_size);
      if (rc != CUDA_LLM_OK) return rc;
    }
    cudaError_t e = run_paged_f32_decode(true, query, key_cache, value_cache, block_tables, context_lens, out, num_seqs,
                                         num_heads, num_kv_heads, head_dim, page_size, max_blocks_per_seq, num_blocks, 0,
                                         softmax_scale, workspace, sm_count_cached(), &maps,
                                         reinterpret_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) g_f32_launches.fetch_add(1, std::memory_order_relaxed);
    return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "paged_attention (fp32) launch");
  }
  cudaError_t e = run_dense_decode(true, query, key_cache, value_cache, block_tables, context_lens, out, num_seqs,
                                   num_heads, num_kv_heads, head_dim, page_size, max_blocks_per_seq, num_blocks, 0,
                                   softmax_scale, dtype, workspace, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "paged_attention launch");
}

int cuda_llm_flash_decode(const void* q, const void* k, const void* v, void* o, int32_t batch_size,
                          int32_t num_heads, int32_t num_kv_heads, int32_t seq_len, int32_t head_dim,
                          float softmax_scale, int32_t dtype, void* workspace, size_t workspace_bytes,
                          void* stream) {
  if (batch_size == 0) return CUDA_LLM_OK;
  if (!q || !k || !v || !o) return fail(CUDA_LLM_EINVAL, "a required tensor pointer is null");
  int rc = check_dense(batch_size, num_heads, num_kv_heads, head_dim, dtype);
  if (rc != CUDA_LLM_OK) return rc;
  if (seq_len < 0) return fail(CUDA_LLM_EINVAL, "seq_len must be >= 0");
  const size_t need = cuda_llm_dense_decode_workspace_bytes(batch_size, num_heads, num_kv_heads, head_dim, seq_len);
  if (!workspace || workspace_bytes < need) return fail(CUDA_LLM_EWORKSPACE, "workspace missing or smaller than cuda_llm_dense_decode_workspace_bytes()");
  if (dtype != CUDA_LLM_F32 && seq_len > 0 && !(((uintptr_t)k | (uintptr_t)v | (uintptr_t)workspace) & 15)) {
    // 16-bit K/V: the persistent tensor-core kernel reading token-major rows (fp32 stays on the SIMT kernel)
    Layout L;
    int lrc = make_layout(batch_size, num_heads, num_kv_heads, head_dim, 16, 1, CUDA_LLM_KV_BF16, CUDA_LLM_KV_BF16,
                          CUDA_LLM_SCALE_PER_HEAD, 0, L, true);
    if (lrc != CUDA_LLM_OK) return lrc;
    if (workspace_bytes < L.ws_total) return fail(CUDA_LLM_EWORKSPACE, "workspace missing or smaller than cuda_llm_dense_decode_workspace_bytes()");
    DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.q = q; a.kc = (const uint8_t*)k; a.vc = (const uint8_t*)v; a.out = o;
    uint8_t* ws = (uint8_t*)workspace;
    a.status = (uint32_t*)ws;
    a.table = (int32_t*)(ws + L.ws_table);
    a.part_lse = (float*)(ws + L.ws_lse);
    a.part_o = (float*)(ws + L.ws_o);
    a.S = batch_size; a.Hq = num_heads; a.Hkv = num_kv_heads; a.group = num_heads / num_kv_heads;
    a.max_blocks = 1; a.num_blocks = 1; a.fixed_ctx = seq_len;
    a.HG = L.HG; a.SUBS = L.SUBS; a.tok_stage = L.tok_stage; a.n_hg = L.n_hg; a.rows_max = L.rows_max;
    a.q_dtype = a.out_dtype = dtype;
    a.scale_log2 = softmax_scale * 1.4426950408889634f;
    a.n_stages = L.n_stages;
    a.grid = L.grid;
    a.n_slots = batch_size * L.n_hg + L.grid;
    if (!((uintptr_t)q & 15)) {
      a.q_smem_off = L.q_smem_off;
      a.q_smem_bytes = L.q_smem_bytes;
      a.q_smem_tokens = 1;
    }
    a.stage_bytes = L.stage_bytes; a.off_v = L.off_v; a.off_ks = L.off_ks; a.off_vs = L.off_vs;
    a.k_page_stride = L.k_page_stride; a.v_page_stride = L.v_page_stride;
    a.k_chunk = L.k_chunk; a.v_chunk = L.v_chunk;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    lrc = check_device();
    if (lrc != CUDA_LLM_OK) return lrc;
    LaunchFn fn;
    if (dtype == CUDA_LLM_BF16) fn = head_dim == 64 ? launch_paged_decode<64, 16, MODE_KV_BF16_TM, 1, false> : launch_paged_decode<128, 16, MODE_KV_BF16_TM, 1, false>;
    else fn = head_dim == 64 ? launch_paged_decode<64, 16, MODE_KV_F16_TM, 1, false> : launch_paged_decode<128, 16, MODE_KV_F16_TM, 1, false>;
    KvTensorMaps tm;
    memset(&tm, 0, sizeof(tm));
    cudaError_t e = fn(a, tm, L.grid, L.smem_bytes, st);
    if (e != cudaSuccess) return fail_cuda(e, "paged_decode_kernel launch");
    e = (head_dim == 64) ? launch_merge_splits<64>(a, 16, L.grid, st) : launch_merge_splits<128>(a, 16, L.grid, st);
    return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "merge_splits_kernel launch");
  }
  if (dtype == CUDA_LLM_F32 && seq_len > 0 && paged_f32_decode_supported(head_dim, 16, k, v) &&
      !((uintptr_t)workspace & 15)) {
    // fp32 K/V: the bulk-copy kernel in its token-major mode
    cudaError_t e = run_paged_f32_decode(false, q, k, v, nullptr, nullptr, o, batch_size, num_heads, num_kv_heads,
                                         head_dim, 16, (seq_len + 15) / 16, 1, seq_len, softmax_scale, workspace,
                                         sm_count_cached(), nullptr, reinterpret_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) g_f32_launches.fetch_add(1, std::memory_order_relaxed);
    return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "flash_decode (fp32) launch");
  }
  cudaError_t e = run_dense_decode(false, q, k, v, nullptr, nullptr, o, batch_size, num_heads, num_kv_heads, head_dim,
                                   1, 1, 1, seq_len, softmax_scale, dtype, workspace, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "flash_decode launch");
}

int cuda_llm_gqa_prefill(const void* q, const void* k, const void* v, void* out, int32_t batch_size,
                         int32_t num_q_heads, int32_t num_kv_heads, int32_t seq_len, int32_t head_dim,
                         float softmax_scale, int32_t is_causal, int32_t dtype,
                         const CudaLlmKvCacheTarget* cache, void* stream) {
  if (batch_size == 0 || seq_len == 0) return CUDA_LLM_OK;
  if (!q || !k || !v || !out) return fail(CUDA_LLM_EINVAL, "a required tensor pointer is null");
  if (batch_size < 0 || seq_len < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads)
    return fail(CUDA_LLM_EINVAL, "num_q_heads must be divisible by num_kv_heads");
  if (head_dim != 64 && head_dim != 128) return fail(CUDA_LLM_EINVAL, "Only head_dim 64 and 128 supported");
  if (dtype < 0 || dtype > CUDA_LLM_BF16) return fail(CUDA_LLM_EINVAL, "unknown dtype");
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
    return fail(CUDA_LLM_EALIGN, "q, k, v and out must be 16-byte aligned");
  if (cache) {
    if (!cache->key_cache || !cache->value_cache || !cache->k_scale || !cache->v_scale || !cache->slot_block ||
        !cache->slot_offset)
      return fail(CUDA_LLM_EINVAL, "cache target: a required pointer is null");
    if (cache->page_size <= 0 || cache->num_blocks <= 0 || cache->scale_mode < 0 ||
        cache->scale_mode > CUDA_LLM_SCALE_MX_E8M0 ||
        (cache->v_format != CUDA_LLM_KV_FP8_E4M3 && cache->v_format != CUDA_LLM_KV_FP4_E2M1) ||
        (cache->v_format == CUDA_LLM_KV_FP4_E2M1 && cache->scale_mode != CUDA_LLM_SCALE_MX_E8M0))
      return fail(CUDA_LLM_EINVAL, "cache target: unsupported page size, format or scale mode");
  }
  const int rc = check_device();
  if (rc != CUDA_LLM_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // 16-bit tensors run on tcgen05 / TMEM (every group size); the other kernels take fp32.
  // CUDA_LLM_PREFILL_KERNEL=warp_mma forces the warp-MMA kernel (A/B measurements).
  static const bool force_warp_mma = [] {
    const char* v = getenv("CUDA_LLM_PREFILL_KERNEL");
    return v && strcmp(v, "warp_mma") == 0;
  }();
  cudaError_t e;
  // (the tcgen05 kernel takes the row maximum before scaling, which needs a positive softmax scale)
  if (!force_warp_mma && softmax_scale > 0.f && gqa_prefill_sm100_supported(num_q_heads, num_kv_heads, head_dim, dtype) &&
      encode_tiled_fn())
    e = run_gqa_prefill_sm100(q, k, v, out, batch_size, num_q_heads, num_kv_heads, seq_len, head_dim, softmax_scale,
                              is_causal != 0, dtype, dtype, st);
  else
    e = run_gqa_prefill(q, k, v, out, batch_size, num_q_heads, num_kv_heads, seq_len, head_dim, softmax_scale,
                        is_causal != 0, dtype, st);
  if (e != cudaSuccess) return fail_cuda(e, "gqa_prefill_kernel launch");
  if (cache) {
    e = run_kv_append_prefill(k, v, *cache, batch_size, num_kv_heads, seq_len, head_dim, dtype, st);
    if (e != cudaSuccess) return fail_cuda(e, "kv_append_kernel launch");
  }
  return CUDA_LLM_OK;
}

int cuda_llm_paged_attention_f32_launches(uint64_t* launches) {
  if (!launches) return fail(CUDA_LLM_EINVAL, "null argument");
  *launches = g_f32_launches.load(std::memory_order_relaxed);
  return CUDA_LLM_OK;
}

int cuda_llm_decode_tcgen05_counters(uint64_t* launches, uint32_t* wait_timeouts) {
  if (launches) *launches = g_sm100_launches.load(std::memory_order_relaxed);
  if (wait_timeouts) {
    const int rc = check_device();
    if (rc != CUDA_LLM_OK) return rc;
    *wait_timeouts = decode100_wait_timeouts();
  }
  return CUDA_LLM_OK;
}

int cuda_llm_prefill_wait_timeouts(uint32_t* count) {
  if (!count) return fail(CUDA_LLM_EINVAL, "null argument");
  unsigned int c = 0;
  const cudaError_t e = prefill_wait_timeouts(&c);
  if (e != cudaSuccess) return fail_cuda(e, "reading the prefill time-out counter");
  *count = c;
  return CUDA_LLM_OK;
}

// The tcgen05 route of the microscaled attention: operands dequantised once into f16 tensors in the
// caller's workspace (codes times scale, one rounding: what the one-kernel route does on the way into shared
// memory), then the tcgen05 / TMEM prefill kernel on those.
static bool mx_attention_tcgen05_shape(int Hq, int Hkv, int D, float softmax_scale) {
  return softmax_scale > 0.f && gqa_prefill_sm100_supported(Hq, Hkv, D, CUDA_LLM_F16) && encode_tiled_fn() != nullptr;
}
static size_t mx_elems(int B, int H, int S, int D) { return (size_t)B * H * S * D; }
static std::atomic<uint64_t> g_mx_tcgen05_launches{0};

size_t cuda_llm_mx_attention_workspace_bytes(int32_t batch_size, int32_t num_q_heads, int32_t num_kv_heads,
                                             int32_t seq_len, int32_t head_dim) {
  if (batch_size <= 0 || seq_len <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return 0;
  if (!mx_attention_tcgen05_shape(num_q_heads, num_kv_heads, head_dim, 1.f)) return 0;
  const size_t a256 = 255;
  return ((mx_elems(batch_size, num_q_heads, seq_len, head_dim) * 2 + a256) & ~a256) +
         2 * ((mx_elems(batch_size, num_kv_heads, seq_len, head_dim) * 2 + a256) & ~a256);
}

int cuda_llm_mx_attention_ws(const void* q, const float* q_scale, const void* k, const float* k_scale, const void* v,
                             const float* v_scale, void* out, int32_t batch_size, int32_t num_q_heads,
                             int32_t num_kv_heads, int32_t seq_len, int32_t head_dim, float softmax_scale,
                             int32_t is_causal, int32_t out_dtype, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (batch_size == 0 || seq_len == 0) return CUDA_LLM_OK;
  if (!q || !k || !v || !q_scale || !k_scale || !v_scale || !out) return fail(CUDA_LLM_EINVAL, "a required tensor pointer is null");
  if (batch_size < 0 || seq_len < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads)
    return fail(CUDA_LLM_EINVAL, "num_q_heads must be divisible by num_kv_heads");
  if (head_dim != 64 && head_dim != 128) return fail(CUDA_LLM_EINVAL, "Only head_dim 64 and 128 supported");
  if (out_dtype < 0 || out_dtype > CUDA_LLM_BF16) return fail(CUDA_LLM_EINVAL, "unknown dtype");
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
    return fail(CUDA_LLM_EALIGN, "q, k, v and out must be 16-byte aligned");
  const int rc = check_device();
  if (rc != CUDA_LLM_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t need = cuda_llm_mx_attention_workspace_bytes(batch_size, num_q_heads, num_kv_heads, seq_len, head_dim);
  if (workspace && need > 0 && workspace_bytes >= need && !((uintptr_t)workspace & 255) &&
      mx_attention_tcgen05_shape(num_q_heads, num_kv_heads, head_dim, softmax_scale)) {
    const size_t nq = mx_elems(batch_size, num_q_heads, seq_len, head_dim), nk = mx_elems(batch_size, num_kv_heads, seq_len, head_dim);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    void* qh = ws;
    void* kh = ws + ((nq * 2 + 255) & ~(size_t)255);
    void* vh = reinterpret_cast<uint8_t*>(kh) + ((nk * 2 + 255) & ~(size_t)255);
    cudaError_t e = launch_mx_to_f16(q, q_scale, qh, nq, st);
    if (e == cudaSuccess) e = launch_mx_to_f16(k, k_scale, kh, nk, st);
    if (e == cudaSuccess) e = launch_mx_to_f16(v, v_scale, vh, nk, st);
    if (e == cudaSuccess)
      e = run_gqa_prefill_sm100(qh, kh, vh, out, batch_size, num_q_heads, num_kv_heads, seq_len, head_dim, softmax_scale,
                                is_causal != 0, CUDA_LLM_F16, out_dtype, st);
    if (e != cudaSuccess) return fail_cuda(e, "microscaled attention (tcgen05 route) launch");
    g_mx_tcgen05_launches.fetch_add(1, std::memory_order_relaxed);
    return CUDA_LLM_OK;
  }
  cudaError_t e = run_mx_attention(q, q_scale, k, k_scale, v, v_scale, out, batch_size, num_q_heads, num_kv_heads,
                                   seq_len, head_dim, softmax_scale, is_causal != 0, out_dtype, st);
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "gqa_prefill_kernel (microscaled) launch");
}

int cuda_llm_mx_attention(const void* q, const float* q_scale, const void* k, const float* k_scale, const void* v,
                          const float* v_scale, void* out, int32_t batch_size, int32_t num_q_heads,
                          int32_t num_kv_heads, int32_t seq_len, int32_t head_dim, float softmax_scale,
                          int32_t is_causal, int32_t out_dtype, void* stream) {
  return cuda_llm_mx_attention_ws(q, q_scale, k, k_scale, v, v_scale, out, batch_size, num_q_heads, num_kv_heads, seq_len,
                                  head_dim, softmax_scale, is_causal, out_dtype, nullptr, 0, stream);
}

int cuda_llm_mx_attention_tcgen05_launches(uint64_t* launches) {
  if (!launches) return fail(CUDA_LLM_EINVAL, "null argument");
  *launches = g_mx_tcgen05_launches.load(std::memory_order_relaxed);
  return CUDA_LLM_OK;
}

int cuda_llm_merge_partials(const float* parts_out, const float* parts_lse, int32_t num_parts,
                            int64_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                            float* lse, void* stream) {
  if (!parts_out || !parts_lse || !out) return fail(CUDA_LLM_EINVAL, "null argument");
  if (head_dim != 64 && head_dim != 128) return fail(CUDA_LLM_EINVAL, "Only head_dim 64 and 128 supported");
  if (num_parts < 1 || rows < 0) return fail(CUDA_LLM_EINVAL, "num_parts >= 1 and rows >= 0 required");
  if (out_dtype < 0 || out_dtype > CUDA_LLM_BF16) return fail(CUDA_LLM_EINVAL, "unknown dtype");
  cudaError_t e = launch_merge_partials(parts_out, parts_lse, num_parts, rows, head_dim, out,
                                        out_dtype, lse, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CUDA_LLM_OK : fail_cuda(e, "merge_partials_kernel launch");
}

}  // extern "C"
