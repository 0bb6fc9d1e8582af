// Split-context decode from one host call: local partial -> NCCL all-gather -> merge.
//
// One long context is sharded by KV range over the ranks of a communicator (one process per GPU).
// Every rank runs the ordinary paged decode over ITS range into an fp32 (out | lse) block, the
// blocks are exchanged with ONE ncclAllGather on the caller's stream, and the partial merge
// (algebra of combine_softmax_state, fused_online_softmax_kernel.cuh:40-49 in the reference
// project) follows on the same stream, reading the gathered blocks from local HBM.  No host code
// runs between the three steps.  The reference has no distributed code; this replaces the
// Python sequence (two all-gathers, four temporaries, a separate merge call).
//
// NCCL is not linked: the communicator belongs to the caller (for example torch.distributed's),
// so the collective must come from the very libnccl that created it.  The symbol is looked up in
// the libnccl.so.2 already loaded into the process.
#include <dlfcn.h>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda_runtime.h>

#include "cuda_llm_b200.h"

namespace b200 {
cudaError_t launch_merge_partials_strided(const float* parts_out, const float* parts_lse, size_t part_stride,
                                          int num_parts, long long rows, int head_dim, void* out, int out_dtype,
                                          float* lse, cudaStream_t st);
void set_error_message(const char* msg);
}  // namespace b200

namespace {
using AllGatherFn = int (*)(const void*, void*, size_t, int, void*, cudaStream_t);
using ErrStrFn = const char* (*)(int);
constexpr int kNcclFloat32 = 7;  // ncclDataType_t value of ncclFloat32 in every NCCL 2.x release

struct Nccl {
  AllGatherFn all_gather = nullptr;
  ErrStrFn err_str = nullptr;
};
const Nccl* nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the process already uses
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    n.all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
    n.err_str = reinterpret_cast<ErrStrFn>(dlsym(h, "ncclGetErrorString"));
  });
  return n.all_gather ? &n : nullptr;
}
int fail(int code, const char* msg) {
  b200::set_error_message(msg);
  return code;
}
}  // namespace

extern "C" {

size_t cuda_llm_split_context_exchange_bytes(int64_t rows, int32_t head_dim, int32_t nranks) {
  if (rows < 0 || head_dim <= 0 || nranks < 1) return 0;
  return (size_t)nranks * (size_t)rows * (size_t)(head_dim + 1) * sizeof(float);
}

int cuda_llm_split_context_decode(const CudaLlmPagedDecodeParams* p, void* nccl_comm, int32_t nranks,
                                  int32_t rank, void* exchange, size_t exchange_bytes, void* stream) {
  if (!p) return fail(CUDA_LLM_EINVAL, "params is null");
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(CUDA_LLM_EINVAL, "rank must lie in [0, nranks)");
  if (p->cu_q_lens) return fail(CUDA_LLM_EINVAL, "split-context decode supports one query token per sequence");
  if (nranks > 1 && !nccl_comm) return fail(CUDA_LLM_EINVAL, "an NCCL communicator is required for nranks > 1");
  const long long rows = (long long)p->num_seqs * p->num_q_heads;
  const int D = p->head_dim;
  const size_t block = (size_t)rows * (size_t)(D + 1);  // floats per rank: out [rows, D] then lse [rows]
  if (!exchange || ((uintptr_t)exchange & 15) || exchange_bytes < (size_t)nranks * block * sizeof(float))
    return fail(CUDA_LLM_EWORKSPACE, "exchange buffer missing, misaligned or smaller than "
                                     "cuda_llm_split_context_exchange_bytes()");
  if (rows == 0) return CUDA_LLM_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* all = reinterpret_cast<float*>(exchange);
  float* mine = all + (size_t)rank * block;

  // 1. local partial over this rank's KV range, normalised inside the range, fp32, with its lse
  CudaLlmPagedDecodeParams q = *p;
  q.out = mine;
  q.out_dtype = CUDA_LLM_F32;
  q.lse = mine + (size_t)rows * D;
  int rc = cuda_llm_paged_decode(&q, stream);
  if (rc != CUDA_LLM_OK) return rc;

  // 2. one in-place all-gather of the (out | lse) blocks over NVLink
  if (nranks > 1) {
    const Nccl* n = nccl();
    if (!n) return fail(CUDA_LLM_ECUDA, "libnccl.so.2 (ncclAllGather) is not available in this process");
    const int nrc = n->all_gather(mine, all, block, kNcclFloat32, nccl_comm, st);
    if (nrc != 0) {
      char msg[200];
      snprintf(msg, sizeof(msg), "ncclAllGather: %s", n->err_str ? n->err_str(nrc) : "error");
      return fail(CUDA_LLM_ECUDA, msg);
    }
  }

  // 3. merge the nranks partials of every row
  cudaError_t e = b200::launch_merge_partials_strided(all, all + (size_t)rows * D, block, nranks, rows, D, p->out,
                                                      p->out_dtype, p->lse, st);
  if (e != cudaSuccess) {
    char msg[200];
    snprintf(msg, sizeof(msg), "merge_partials_kernel launch: %s", cudaGetErrorString(e));
    return fail(CUDA_LLM_ECUDA, msg);
  }
  return CUDA_LLM_OK;
}

}  // extern "C"
