// PyTorch extension `fused_online_softmax_cuda`: the decode path and the GQA prefill in front of it.
//
// Same module name, function names, argument names and defaults as the reference binding
// (fused_softmax_binding.cpp in the reference project: paged_attention_forward :109-173 / m.def
// :733-741, async_flash_decode :308-360 / :759-763, fp8_paged_attention_forward :634-718 /
// :800-807, fused_gqa_forward :246-302 / :751-756), same TORCH_CHECK messages.  Differences, all additive: a device guard taken from the
// query tensor (the reference has none), GQA inferred from the cache's head count, page sizes 32 and
// 64, per-token and E8M0 scales, packed FP4 V, and keyword-only extensions (cu_q_lens, max_q_len,
// return_lse, kv_format, rope_cos / rope_sin / rope_positions).  Every call goes straight to the C ABI of libcuda_llm_b200.so on the
// current stream; torch supplies tensors, the stream and the scratch buffer.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cmath>
#include <map>
#include <mutex>
#include <tuple>

#include "cuda_llm_b200.h"

namespace {

int dtype_code(const torch::Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::ScalarType::Float: return CUDA_LLM_F32;
    case at::ScalarType::Half: return CUDA_LLM_F16;
    case at::ScalarType::BFloat16: return CUDA_LLM_BF16;
    default: TORCH_CHECK(false, what);
  }
  return -1;
}

void check_rc(int rc, const char* where) {
  TORCH_CHECK(rc == CUDA_LLM_OK, where, " failed with code ", rc, ": ", cuda_llm_last_cuda_error());
}

// One grow-only scratch buffer per (device, stream); its status header is zeroed when it is made.
torch::Tensor workspace_for(const torch::Tensor& like, size_t bytes, cudaStream_t stream) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, torch::Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair((int)like.get_device(), stream);
  auto it = cache.find(key);
  if (it == cache.end() || (size_t)it->second.numel() < bytes) {
    const int64_t n = (int64_t)std::max<size_t>(bytes, (size_t)1 << 20);
    auto ws = torch::empty({n}, torch::TensorOptions().dtype(torch::kUInt8).device(like.device()));
    check_rc(cuda_llm_workspace_init(ws.data_ptr(), (size_t)n, stream), "cuda_llm_workspace_init");
    cache[key] = ws;
    return ws;
  }
  return it->second;
}

float scale_or_default(const c10::optional<double>& s, int head_dim) {
  return s.has_value() ? static_cast<float>(s.value()) : 1.0f / std::sqrt(static_cast<float>(head_dim));
}

}  // namespace

torch::Tensor paged_attention_forward(torch::Tensor query, torch::Tensor key_cache, torch::Tensor value_cache,
                                      torch::Tensor block_tables, torch::Tensor context_lens,
                                      c10::optional<double> softmax_scale_opt) {
  TORCH_CHECK(query.is_cuda() && key_cache.is_cuda() && value_cache.is_cuda(), "Inputs must be on CUDA");
  TORCH_CHECK(block_tables.is_cuda() && context_lens.is_cuda(), "Metadata tensors must be on CUDA");
  TORCH_CHECK(query.dim() == 3, "Query must be 3D [num_seqs, num_heads, head_dim]");
  TORCH_CHECK(key_cache.dim() == 4 && value_cache.dim() == 4,
              "KV caches must be 4D [num_blocks, num_heads, head_dim, page_size]");
  const int num_seqs = query.size(0), num_heads = query.size(1), head_dim = query.size(2);
  TORCH_CHECK(head_dim == 64 || head_dim == 128, "Only head_dim 64 and 128 supported");
  const int dt = dtype_code(query, "Unsupported scalar type for PagedAttention. Supported: Float32, Float16, BFloat16.");
  TORCH_CHECK(key_cache.scalar_type() == query.scalar_type() && value_cache.scalar_type() == query.scalar_type(),
              "query and KV caches must have the same dtype");
  TORCH_CHECK(key_cache.size(2) == head_dim && value_cache.sizes() == key_cache.sizes(),
              "KV caches must be [num_blocks, num_kv_heads, head_dim, page_size] with the query's head_dim");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && context_lens.scalar_type() == at::kInt,
              "block_tables and context_lens must be int32");
  TORCH_CHECK(query.is_contiguous() && key_cache.is_contiguous() && value_cache.is_contiguous() &&
                  block_tables.is_contiguous() && context_lens.is_contiguous(), "inputs must be contiguous");
  const int num_kv_heads = key_cache.size(1), page = key_cache.size(3);
  c10::cuda::CUDAGuard guard(query.device());
  auto output = torch::empty_like(query);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const size_t need = cuda_llm_dense_decode_workspace_bytes(num_seqs, num_heads, num_kv_heads, head_dim,
                                                            (int)block_tables.size(1) * page);
  TORCH_CHECK(need != 0 || num_seqs == 0, "cuda_llm_dense_decode_workspace_bytes: ", cuda_llm_last_cuda_error());
  auto ws = workspace_for(query, need, stream);
  check_rc(cuda_llm_paged_attention(query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                                    block_tables.data_ptr<int32_t>(), context_lens.data_ptr<int32_t>(),
                                    output.data_ptr(), num_seqs, num_heads, num_kv_heads, head_dim, page,
                                    (int)block_tables.size(1), (int)key_cache.size(0),
                                    scale_or_default(softmax_scale_opt, head_dim), dt, ws.data_ptr(),
                                    (size_t)ws.numel(), stream),
           "cuda_llm_paged_attention");
  return output;
}

torch::Tensor async_flash_decode_forward(torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                         c10::optional<double> softmax_scale_opt) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "Inputs must be on CUDA");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "Inputs must be 4D [batch, heads, seq, dim]");
  TORCH_CHECK(q.size(2) == 1, "Query sequence length must be 1 for Flash-Decoding");
  TORCH_CHECK(k.sizes() == v.sizes(), "K and V must have identical shapes");
  const int batch = q.size(0), num_heads = q.size(1), seq_len = k.size(2), head_dim = q.size(3);
  TORCH_CHECK(head_dim == 64 || head_dim == 128, "Only head_dim 64 and 128 supported");
  const int dt = dtype_code(q, "Unsupported scalar type for Async Flash-Decode. Supported: Float32, Float16, BFloat16.");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q, k and v must have one dtype");
  q = q.contiguous();
  k = k.contiguous();
  v = v.contiguous();
  c10::cuda::CUDAGuard guard(q.device());
  auto output = torch::empty_like(q);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int num_kv_heads = k.size(1);
  const size_t need = cuda_llm_dense_decode_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, seq_len);
  TORCH_CHECK(need != 0 || batch == 0, "cuda_llm_dense_decode_workspace_bytes: ", cuda_llm_last_cuda_error());
  auto ws = workspace_for(q, need, stream);
  check_rc(cuda_llm_flash_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(), batch, num_heads,
                                 num_kv_heads, seq_len, head_dim, scale_or_default(softmax_scale_opt, head_dim), dt,
                                 ws.data_ptr(), (size_t)ws.numel(), stream),
           "cuda_llm_flash_decode");
  return output;
}

torch::Tensor fused_gqa_forward(torch::Tensor q, torch::Tensor k, torch::Tensor v, bool is_causal,
                                c10::optional<double> softmax_scale_opt) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "Inputs must be on CUDA");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "Inputs must be 4D [batch, heads, seq, dim]");
  TORCH_CHECK(k.sizes() == v.sizes(), "K and V must have identical shapes");
  const int batch = q.size(0), num_q_heads = q.size(1), seq_len = q.size(2), head_dim = q.size(3);
  const int num_kv_heads = k.size(1);
  TORCH_CHECK(num_q_heads % num_kv_heads == 0, "num_q_heads must be divisible by num_kv_heads");
  TORCH_CHECK(head_dim == 64 || head_dim == 128, "Only head_dim 64 and 128 supported");
  const int dt = dtype_code(q, "Unsupported scalar type for GQA. Supported: Float32, Float16, BFloat16.");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() && k.size(0) == batch &&
                  k.size(2) == seq_len && k.size(3) == head_dim,
              "q, k and v must share dtype, batch, sequence length and head_dim");
  q = q.contiguous();
  k = k.contiguous();
  v = v.contiguous();
  c10::cuda::CUDAGuard guard(q.device());
  auto output = torch::empty_like(q);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  check_rc(cuda_llm_gqa_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(), batch, num_q_heads,
                                num_kv_heads, seq_len, head_dim, scale_or_default(softmax_scale_opt, head_dim),
                                is_causal ? 1 : 0, dt, nullptr, stream),
           "cuda_llm_gqa_prefill");
  return output;
}

pybind11::object fp8_paged_attention_forward(torch::Tensor query, torch::Tensor key_cache_fp8,
                                             torch::Tensor value_cache_fp8, torch::Tensor k_scale,
                                             torch::Tensor v_scale, torch::Tensor block_tables,
                                             torch::Tensor context_lens, c10::optional<double> softmax_scale_opt,
                                             c10::optional<torch::Tensor> cu_q_lens, int64_t max_q_len,
                                             bool return_lse, c10::optional<std::string> kv_format,
                                             c10::optional<torch::Tensor> rope_cos,
                                             c10::optional<torch::Tensor> rope_sin,
                                             c10::optional<torch::Tensor> rope_positions) {
  TORCH_CHECK(query.is_cuda() && key_cache_fp8.is_cuda() && value_cache_fp8.is_cuda(), "Inputs must be on CUDA");
  TORCH_CHECK(k_scale.is_cuda() && v_scale.is_cuda(), "Scale tensors must be on CUDA");
  TORCH_CHECK(block_tables.is_cuda() && context_lens.is_cuda(), "Metadata tensors must be on CUDA");
  TORCH_CHECK(query.dim() == 3, "Query must be 3D [num_seqs, num_heads, head_dim]");
  TORCH_CHECK(key_cache_fp8.dim() == 4 && value_cache_fp8.dim() == 4,
              "KV caches must be 4D [num_blocks, num_heads, head_dim, page_size]");
  auto is_byte = [](const torch::Tensor& t) {
    return t.scalar_type() == at::ScalarType::Char || t.scalar_type() == at::ScalarType::Byte ||
           t.scalar_type() == at::ScalarType::Float8_e4m3fn;
  };
  TORCH_CHECK(is_byte(key_cache_fp8) && is_byte(value_cache_fp8), "KV caches must be 8-bit quantized (int8 or uint8)");
  TORCH_CHECK(!kv_format.has_value() || kv_format.value() == "fp8_e4m3", "unknown kv_format: only 'fp8_e4m3' is provided");
  // The reference kernel reads an int8 cache as integers (fp8_paged_attention_kernel.cuh:102); this
  // library reads bytes as E4M3 codes and refuses to reinterpret an int8 tensor silently.
  const bool any_int8 = key_cache_fp8.scalar_type() == at::ScalarType::Char ||
                        value_cache_fp8.scalar_type() == at::ScalarType::Char;
  TORCH_CHECK(!any_int8 || kv_format.has_value(),
              "int8 KV caches are not accepted: this library reads cache bytes as FP8-E4M3 codes, the reference "
              "kernel reads them as integers (fp8_paged_attention_kernel.cuh:102). Pass uint8 / float8_e4m3fn "
              "tensors, or kv_format='fp8_e4m3' if the int8 tensor holds E4M3 codes.");
  const int total_q = query.size(0), num_heads = query.size(1), head_dim = query.size(2);
  const int num_kv_heads = key_cache_fp8.size(1), page_size = key_cache_fp8.size(3);
  TORCH_CHECK(head_dim == 64 || head_dim == 128, "Only head_dim 64 and 128 supported");
  TORCH_CHECK(page_size == 16 || page_size == 32 || page_size == 64, "Only page_size 16, 32 and 64 are supported");
  const int qdt = dtype_code(query, "Unsupported query scalar type for FP8 PagedAttention. Supported: Float32, Float16, BFloat16.");
  TORCH_CHECK(key_cache_fp8.size(2) == head_dim, "key cache head_dim does not match the query");
  int v_format = CUDA_LLM_KV_FP8_E4M3;
  if (value_cache_fp8.size(2) * 2 == head_dim) v_format = CUDA_LLM_KV_FP4_E2M1;
  else TORCH_CHECK(value_cache_fp8.size(2) == head_dim, "value cache head_dim does not match the query");
  TORCH_CHECK(num_heads % num_kv_heads == 0, "num_heads must be a multiple of the cache's num_kv_heads");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && context_lens.scalar_type() == at::kInt,
              "block_tables and context_lens must be int32");
  TORCH_CHECK(query.is_contiguous() && key_cache_fp8.is_contiguous() && value_cache_fp8.is_contiguous() &&
                  block_tables.is_contiguous() && context_lens.is_contiguous(), "inputs must be contiguous");
  const int num_seqs = context_lens.size(0);
  TORCH_CHECK(cu_q_lens.has_value() || total_q == num_seqs, "query has more rows than sequences: pass cu_q_lens");

  int scale_mode;
  const bool e8m0 = k_scale.scalar_type() == at::ScalarType::Byte || k_scale.scalar_type() == at::ScalarType::Float8_e8m0fnu;
  if (e8m0) {
    TORCH_CHECK(k_scale.dim() == 4, "E8M0 scales must be 4D [num_blocks, num_kv_heads, head_dim/32, page_size]");
    scale_mode = CUDA_LLM_SCALE_MX_E8M0;
  } else {
    TORCH_CHECK(k_scale.dim() >= 1 && k_scale.dim() <= 3,
                "Scale tensors must be 1D [heads], 2D [blocks, heads], 3D [blocks, heads, page] "
                "or 4D E8M0 [blocks, heads, head_dim/32, page]");
    // reference: per_block_scales = (k_scale.dim() == 2), fused_softmax_binding.cpp:671
    scale_mode = k_scale.dim() == 1 ? CUDA_LLM_SCALE_PER_HEAD
               : k_scale.dim() == 2 ? CUDA_LLM_SCALE_PER_BLOCK : CUDA_LLM_SCALE_PER_TOKEN;
  }
  c10::cuda::CUDAGuard guard(query.device());
  // the reference converts scales to fp32 contiguous temporaries (fused_softmax_binding.cpp:680-681)
  auto ks = e8m0 ? k_scale.contiguous() : k_scale.to(torch::kFloat32).contiguous();
  auto vs = e8m0 ? v_scale.contiguous() : v_scale.to(torch::kFloat32).contiguous();
  auto output = torch::empty_like(query);
  torch::Tensor lse;
  if (return_lse) lse = torch::empty({total_q, num_heads}, query.options().dtype(torch::kFloat32));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const size_t need = cuda_llm_paged_decode_workspace_bytes(num_seqs, num_heads, num_kv_heads, head_dim, page_size,
                                                            (int)max_q_len, 0);
  TORCH_CHECK(need != 0 || num_seqs == 0, "cuda_llm_paged_decode_workspace_bytes: ", cuda_llm_last_cuda_error());
  auto ws = workspace_for(query, need, stream);

  CudaLlmPagedDecodeParams p = {};
  p.query = query.data_ptr();
  p.key_cache = key_cache_fp8.data_ptr();
  p.value_cache = value_cache_fp8.data_ptr();
  p.k_scale = ks.data_ptr();
  p.v_scale = vs.data_ptr();
  p.block_tables = block_tables.data_ptr<int32_t>();
  p.context_lens = context_lens.data_ptr<int32_t>();
  if (cu_q_lens.has_value()) {
    TORCH_CHECK(cu_q_lens->is_cuda() && cu_q_lens->scalar_type() == at::kInt && cu_q_lens->is_contiguous() &&
                    cu_q_lens->numel() == num_seqs + 1, "cu_q_lens must be a contiguous int32 CUDA tensor [num_seqs + 1]");
    p.cu_q_lens = cu_q_lens->data_ptr<int32_t>();
  }
  p.out = output.data_ptr();
  p.lse = return_lse ? lse.data_ptr<float>() : nullptr;
  p.workspace = ws.data_ptr();
  p.workspace_bytes = (size_t)ws.numel();
  p.num_seqs = num_seqs;
  p.num_q_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.head_dim = head_dim;
  p.page_size = page_size;
  p.max_blocks_per_seq = block_tables.size(1);
  p.num_blocks = key_cache_fp8.size(0);
  p.max_q_len = (int)max_q_len;
  p.q_dtype = p.out_dtype = qdt;
  p.k_format = CUDA_LLM_KV_FP8_E4M3;
  p.v_format = v_format;
  p.scale_mode = scale_mode;
  p.softmax_scale = scale_or_default(softmax_scale_opt, head_dim);
  torch::Tensor rc_t, rs_t, rp_t;  // keep the converted rotary tensors alive until the launch is queued
  if (rope_cos.has_value()) {
    TORCH_CHECK(rope_sin.has_value() && rope_cos->dim() == 2 && rope_cos->sizes() == rope_sin->sizes() &&
                    rope_cos->size(1) == head_dim, "rope_cos / rope_sin must both be [positions, head_dim]");
    rc_t = rope_cos->to(query.device(), torch::kFloat32).contiguous();
    rs_t = rope_sin->to(query.device(), torch::kFloat32).contiguous();
    p.rope_cos = rc_t.data_ptr<float>();
    p.rope_sin = rs_t.data_ptr<float>();
    p.rope_num_positions = (int)rc_t.size(0);
    if (rope_positions.has_value()) {
      rp_t = rope_positions->to(query.device(), torch::kInt32).contiguous();
      TORCH_CHECK(rp_t.numel() == total_q, "rope_positions must have one entry per query token");
      p.rope_positions = rp_t.data_ptr<int32_t>();
    }
  }
  check_rc(cuda_llm_paged_decode(&p, stream), "cuda_llm_paged_decode");
  if (return_lse) return pybind11::cast(std::make_tuple(output, lse));
  return pybind11::cast(output);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "B200 (sm_100a) decode-attention path behind the reference's module name";
  m.def("paged_attention_forward", &paged_attention_forward,
        "PagedAttention forward over a paged fp32 / fp16 / bf16 KV cache",
        pybind11::arg("query"), pybind11::arg("key_cache"), pybind11::arg("value_cache"),
        pybind11::arg("block_tables"), pybind11::arg("context_lens"),
        pybind11::arg("softmax_scale") = pybind11::none());
  m.def("async_flash_decode", &async_flash_decode_forward, "Flash-Decoding over contiguous K/V",
        pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"),
        pybind11::arg("softmax_scale") = pybind11::none());
  m.def("fused_gqa_forward", &fused_gqa_forward, "Grouped-query attention forward over a whole prompt",
        pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("is_causal") = true,
        pybind11::arg("softmax_scale") = pybind11::none());
  m.def("fp8_paged_attention_forward", &fp8_paged_attention_forward,
        "PagedAttention forward over a paged FP8-E4M3 / MXFP8 / MXFP4 KV cache",
        pybind11::arg("query"), pybind11::arg("key_cache_fp8"), pybind11::arg("value_cache_fp8"),
        pybind11::arg("k_scale"), pybind11::arg("v_scale"), pybind11::arg("block_tables"),
        pybind11::arg("context_lens"), pybind11::arg("softmax_scale") = pybind11::none(),
        pybind11::kw_only(), pybind11::arg("cu_q_lens") = pybind11::none(), pybind11::arg("max_q_len") = 1,
        pybind11::arg("return_lse") = false, pybind11::arg("kv_format") = pybind11::none(),
        pybind11::arg("rope_cos") = pybind11::none(), pybind11::arg("rope_sin") = pybind11::none(),
        pybind11::arg("rope_positions") = pybind11::none());
}
