/* C ABI of the B200 paged decode-attention library (libcuda_llm_b200.so).
 *
 * Every entry point takes plain device pointers and sizes, launches asynchronously on the
 * stream it is given, and returns 0 on success or a negative CUDA_LLM_E* code.  Nothing here
 * traps, asserts or aborts; faults a kernel detects at run time (a block-table entry out of
 * range, a wait that ran out) are recorded in a status word inside the workspace and read
 * with cuda_llm_decode_status().
 *
 * Reference interfaces these replace (paths in the reference project):
 *   kernels_api.h:35-41    dispatch_paged_attention<T>
 *   kernels_api.h:58-62    dispatch_async_flash_decode<T>
 *   kernels_api.h:94-101   dispatch_fp8_paged_attention<T_OUT,T_Q>
 * The reference dispatchers return void and silently launch nothing for an unsupported shape
 * (paged_attention_kernel.cuh:169-181); these return an error code instead.
 */
#ifndef CUDA_LLM_B200_H_
#define CUDA_LLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ---------------------------------------------------------------------- */
#define CUDA_LLM_OK 0
#define CUDA_LLM_EINVAL (-1)     /* bad argument (null pointer, unsupported shape/format)   */
#define CUDA_LLM_EALIGN (-2)     /* a pointer is not 16-byte aligned                         */
#define CUDA_LLM_EWORKSPACE (-3) /* workspace missing or too small                           */
#define CUDA_LLM_ECUDA (-4)      /* a CUDA runtime call failed; see cuda_llm_last_cuda_error */
#define CUDA_LLM_EDEVICE (-5)    /* not an sm_100 device                                     */

/* bits of the device status word */
#define CUDA_LLM_ST_BAD_BLOCK 1u   /* block-table entry outside [0, num_blocks)              */
#define CUDA_LLM_ST_BAD_CTX 2u     /* context length exceeds max_blocks_per_seq * page_size  */
#define CUDA_LLM_ST_TIMEOUT 4u     /* a bounded wait gave up                                 */
#define CUDA_LLM_ST_BAD_QLEN 8u    /* group * q_len exceeds the rows the launch was sized for */
#define CUDA_LLM_ST_SCALE_RANGE 16u /* an E8M0 V scale byte of a live token is outside [32, 223] */
#define CUDA_LLM_ST_BAD_POSITION 64u /* a rotary position outside [0, rope_num_positions)         */
#define CUDA_LLM_ST_INCOMPLETE 32u /* a (sequence, head group) was left without a result: its rows
                                      are zeros (follows CUDA_LLM_ST_TIMEOUT)                     */

/* bits of CudaLlmPagedDecodeParams.flags */
#define CUDA_LLM_FLAG_SKIP_MERGE 1 /* launch the attention kernel only (profiling: sequences
                                      that were split across CTAs are left unmerged)         */

#define CUDA_LLM_FLAG_STABLE_METADATA 64 /* promise: the kernel immediately in front of this call on the
                                            stream does not write context_lens, cu_q_lens or
                                            block_tables (they were prepared earlier, e.g. once per
                                            model step for all layers).  The decode kernel is launched
                                            as a programmatic dependent and then plans its ranges and
                                            prefetches its first table entries while that kernel is
                                            still finishing; query, K/V, the split partials and the
                                            outputs are not touched before it has finished either way
                                            (a finding of the plan, such as CUDA_LLM_ST_BAD_CTX, may be
                                            OR-ed into the status word early). */
#define CUDA_LLM_FLAG_TEST_STALL 128 /* failure-path test: the CTA that owns the first stage of the
                                        launch announces its bytes but never sends them, and every wait gives up after a few
                                        thousand polls instead of seconds.  The waits run out, all warps
                                        return, CUDA_LLM_ST_TIMEOUT (and CUDA_LLM_ST_INCOMPLETE for the rows
                                        left without a result) is set; nothing faults or hangs.          */
#define CUDA_LLM_FLAG_TCGEN05 4096 /* run the call on the tcgen05 / tensor-memory decode kernel where it
                                    * applies (head_dim 128, an even number of KV heads, pages of 16 tokens, E4M3 K and V with per-token
                                    * fp32 or E8M0 block scales, 16-bit queries, no rotary embedding);
                                    * other calls ignore the flag.  The environment variable
                                    * CUDA_LLM_DECODE_KERNEL=tcgen05 sets it for every call of the process.
                                    * Same results contract; measured slower than the default warp-MMA
                                    * kernel on a B200, which is why it is opt-in. */

#ifdef CUDA_LLM_DIAGNOSTICS /* honoured only by a library built with -DCUDA_LLM_DIAGNOSTICS */
#define CUDA_LLM_FLAG_DIAG_NO_MATH 2 /* diagnostics: stream the pages but skip the attention math
                                        (output is meaningless; measures the copy pipeline)   */
#define CUDA_LLM_FLAG_DIAG_NO_COPY 4 /* diagnostics: do the attention math on stale shared memory,
                                        no page copies (output is meaningless)                */
#define CUDA_LLM_FLAG_DIAG_TRACE 8   /* diagnostics: `lse` receives, per CTA, eight 64-bit nanosecond
                                        words (ns of entry, first stage landed, last stage consumed,
                                        exit; SM id; three prologue marks) instead of log-sum-exps;
                                        needs grid*64 bytes         */
#define CUDA_LLM_FLAG_DIAG_NO_SCALE_COPY 16 /* diagnostics: do not copy the per-token / block scales
                                              (output is meaningless)                          */
#define CUDA_LLM_FLAG_DIAG_REVERSED 32      /* diagnostics: CTA i takes the unit range of CTA grid-1-i
                                              (same result; separates SM effects from data effects) */
/* bits 8..11: diagnostics: cap the shared-memory ring at this many stages (0 = as many as fit) */
#endif

/* ---- enums ---------------------------------------------------------------------------- */
enum CudaLlmDType { CUDA_LLM_F32 = 0, CUDA_LLM_F16 = 1, CUDA_LLM_BF16 = 2 };

enum CudaLlmKvFormat {
  CUDA_LLM_KV_FP8_E4M3 = 0, /* uint8 [num_blocks, Hkv, D,   page]                            */
  CUDA_LLM_KV_FP4_E2M1 = 1, /* uint8 [num_blocks, Hkv, D/2, page], low nibble = even d (V only) */
  CUDA_LLM_KV_INT8 = 2,     /* reference's integer reading of the byte (fp8_paged_attention_kernel.cuh:102) */
  CUDA_LLM_KV_F16 = 3,      /* fp16 [num_blocks, Hkv, D, page], no scales (K and V alike)    */
  CUDA_LLM_KV_BF16 = 4      /* bf16 [num_blocks, Hkv, D, page], no scales (K and V alike)    */
};

enum CudaLlmScaleMode {
  CUDA_LLM_SCALE_PER_HEAD = 0,  /* fp32 [Hkv]                                                */
  CUDA_LLM_SCALE_PER_BLOCK = 1, /* fp32 [num_blocks, Hkv]   (reference per_block_scales)     */
  CUDA_LLM_SCALE_PER_TOKEN = 2, /* fp32 [num_blocks, Hkv, page]                              */
  CUDA_LLM_SCALE_MX_E8M0 = 3    /* uint8 [num_blocks, Hkv, D/32, page]                       */
};

/* ---- paged decode --------------------------------------------------------------------- */
typedef struct CudaLlmPagedDecodeParams {
  /* device tensors, all borrowed */
  const void* query;           /* [total_q, Hq, D] of q_dtype                                */
  const void* key_cache;       /* see CudaLlmKvFormat                                        */
  const void* value_cache;
  const void* k_scale;         /* see CudaLlmScaleMode                                       */
  const void* v_scale;
  const int32_t* block_tables; /* [num_seqs, max_blocks_per_seq]                             */
  const int32_t* context_lens; /* [num_seqs]                                                 */
  const int32_t* cu_q_lens;    /* [num_seqs+1] prefix of per-sequence query lengths, or NULL
                                  when every sequence has exactly one query token            */
  void* out;                   /* [total_q, Hq, D] of out_dtype                              */
  float* lse;                  /* optional [total_q, Hq] natural-log sum-exp, or NULL        */
  void* workspace;             /* cuda_llm_paged_decode_workspace_bytes() bytes, 256-aligned */
  size_t workspace_bytes;

  int32_t num_seqs;
  int32_t num_q_heads;
  int32_t num_kv_heads;        /* divides num_q_heads; kv_head = q_head / (Hq/Hkv)           */
  int32_t head_dim;            /* 64 or 128                                                  */
  int32_t page_size;           /* 16, 32 or 64                                               */
  int32_t max_blocks_per_seq;
  int32_t num_blocks;          /* pages in the pool (bounds check of block-table entries)    */
  int32_t max_q_len;           /* upper bound of per-sequence q_len; (Hq/Hkv)*max_q_len <= 16 */
  int32_t q_dtype;             /* CudaLlmDType                                               */
  int32_t out_dtype;           /* CudaLlmDType                                               */
  int32_t k_format;            /* CudaLlmKvFormat                                            */
  int32_t v_format;
  int32_t scale_mode;          /* CudaLlmScaleMode, same for K and V                         */
  float softmax_scale;
  int32_t num_ctas;            /* 0 = one per SM                                             */
  int32_t flags;               /* CUDA_LLM_FLAG_* bits, normally 0                          */

  /* Optional rotary embedding fused into the query load (math of the reference's
   * fused_rope_flash_attention_kernel.cuh:56-74, rotate-half convention, tables as its
   * tests/_utils.py:75-81 builds them): q' = q * cos[pos] + rot_half(q) * sin[pos], in fp32, before
   * the dot products.  K in the cache is expected to be rotated already (it was when it was
   * appended).  All NULL / 0: no rotation. */
  const float* rope_cos;          /* [rope_num_positions, head_dim] fp32, or NULL             */
  const float* rope_sin;          /* [rope_num_positions, head_dim] fp32                      */
  const int32_t* rope_positions;  /* [total_q] position of every query token, or NULL: query
                                     token j of a sequence sits at context_len - q_len + j    */
  int32_t rope_num_positions;     /* rows of the tables (a position outside them is clamped
                                     and reported as CUDA_LLM_ST_BAD_POSITION)                */
} CudaLlmPagedDecodeParams;

/* Bytes of workspace cuda_llm_paged_decode needs for these dimensions on the current device. */
size_t cuda_llm_paged_decode_workspace_bytes(int32_t num_seqs, int32_t num_q_heads,
                                             int32_t num_kv_heads, int32_t head_dim,
                                             int32_t page_size, int32_t max_q_len,
                                             int32_t num_ctas);

/* Zero the workspace header (the device status word).  Call once after allocating a
 * workspace, before its first use. */
int cuda_llm_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Decode attention over a paged, quantised KV cache (replaces dispatch_fp8_paged_attention,
 * kernels_api.h:94-101, extended with GQA, per-token and microscaling formats, q_len > 1 and
 * split-KV).  Launches the attention kernel and the split merge on `stream`. */
int cuda_llm_paged_decode(const CudaLlmPagedDecodeParams* params, void* stream);

/* No counterpart in the reference.  Same computation as cuda_llm_paged_decode, for callers that
 * must not allocate device memory: a plugin called from a host runtime that owns the memory pool,
 * or a serving thread where a cudaMalloc (which can synchronise the device or fail under memory
 * pressure) is not acceptable.  params->workspace / workspace_bytes are ignored; the split
 * partials go to a 16 MiB array built into the library (cuda_llm_static_scratch_bytes()), which
 * every GPU that loads the library holds until the process exits.  Nothing is allocated or freed,
 * here or in anything this calls.  Problems whose workspace exceeds the array (see
 * cuda_llm_paged_decode_workspace_bytes) are refused with CUDA_LLM_EWORKSPACE.  The first call on
 * a device looks up the array's device address and zeroes its status word; make that first call
 * outside any stream capture.  All calls on a device share the one array: two calls that overlap
 * on the GPU (different streams) race on it, so keep them on one stream or order them with events.
 * The array keeps the previous call's contents; the status word keeps its bits until
 * cuda_llm_static_decode_status reads (and clears) them. */
int cuda_llm_paged_decode_static(const CudaLlmPagedDecodeParams* params, void* stream);
size_t cuda_llm_static_scratch_bytes(void);
/* No counterpart in the reference.  Read (and clear) the device status word of the built-in
 * scratch of the current device; synchronises `stream`.  Allocates nothing. */
int cuda_llm_static_decode_status(void* stream, uint32_t* status_out);

/* Read (and clear) the device status word of a workspace; synchronises `stream`. */
int cuda_llm_decode_status(void* workspace, void* stream, uint32_t* status_out);

/* ---- unquantised KV ------------------------------------------------------------------- */
/* Workspace for the two entry points below; max_tokens = max_blocks_per_seq * page_size (paged)
 * or seq_len (contiguous).  The partial results start behind the 256-byte header; of the header the
 * calls use the status word (an out-of-range block index of an fp32 cache is replaced by block 0 and
 * reported as CUDA_LLM_ST_BAD_BLOCK) and, for fp32 tensors, a work counter at byte 128 that every
 * call resets itself, so the buffer may be the one cuda_llm_paged_decode uses on the same stream. */
size_t cuda_llm_dense_decode_workspace_bytes(int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads,
                                             int32_t head_dim, int32_t max_tokens);

/* Replaces dispatch_paged_attention<T> (kernels_api.h:35-41): decode attention over a paged
 * fp32 / fp16 / bf16 cache [num_blocks, num_kv_heads, head_dim, page_size]; query and out
 * [num_seqs, num_heads, head_dim] of the same dtype.  num_kv_heads < num_heads is GQA (the
 * reference is MHA only); num_blocks bounds the block-table entries. */
int cuda_llm_paged_attention(const void* query, const void* key_cache, const void* value_cache,
                             const int32_t* block_tables, const int32_t* context_lens, void* out,
                             int32_t num_seqs, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                             int32_t page_size, int32_t max_blocks_per_seq, int32_t num_blocks,
                             float softmax_scale, int32_t dtype, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Replaces dispatch_async_flash_decode<T> (kernels_api.h:58-62): q, o [batch, num_heads, 1, head_dim],
 * k, v [batch, num_kv_heads, seq_len, head_dim], one dtype. */
int cuda_llm_flash_decode(const void* q, const void* k, const void* v, void* o, int32_t batch_size,
                          int32_t num_heads, int32_t num_kv_heads, int32_t seq_len, int32_t head_dim,
                          float softmax_scale, int32_t dtype, void* workspace, size_t workspace_bytes,
                          void* stream);

/* Merge `num_parts` split-KV partials: parts_out [num_parts, rows, D] fp32 (each normalised
 * inside its own KV range), parts_lse [num_parts, rows] natural-log sum-exp (-inf = empty).
 * Writes out [rows, D] of out_dtype and, if not NULL, lse [rows].  Used after the all-gather
 * of the split-context mode; algebra of combine_softmax_state
 * (fused_online_softmax_kernel.cuh:40-49). */
int cuda_llm_merge_partials(const float* parts_out, const float* parts_lse, int32_t num_parts,
                            int64_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                            float* lse, void* stream);

/* ---- split-context decode over several GPUs -------------------------------------------- */
/* No counterpart in the reference (it has no distributed code).  One context sharded by KV range
 * over `nranks` processes, one per GPU: every rank passes the cache, block tables and context
 * lengths of ITS token range in `params` (q_len 1 only; params->out / params->lse receive the final,
 * merged result in out_dtype on every rank).  The call issues, on `stream` and with no host work in
 * between: the paged decode over the local range into this rank's block of `exchange` (fp32 out
 * [rows, D] followed by lse [rows], rows = num_seqs * num_q_heads), ONE in-place ncclAllGather of
 * those blocks over `nccl_comm` (an ncclComm_t created by the caller on this device, e.g. the one
 * torch.distributed uses; ncclAllGather is taken from the libnccl.so.2 already loaded in the
 * process), and the partial merge.  `exchange`: cuda_llm_split_context_exchange_bytes() bytes,
 * 16-byte aligned.  nranks == 1 needs no communicator. */
size_t cuda_llm_split_context_exchange_bytes(int64_t rows, int32_t head_dim, int32_t nranks);
int cuda_llm_split_context_decode(const CudaLlmPagedDecodeParams* params, void* nccl_comm, int32_t nranks,
                                  int32_t rank, void* exchange, size_t exchange_bytes, void* stream);

/* Write n_tokens new K/V vectors ([n_tokens, Hkv, D] of in_dtype) into the paged quantised cache
 * at (slot_block[i], slot_offset[i]), quantising on the fly with the reference test's recipe
 * (tests/test_kernels_misc.py:51-55 extended to per-token and E8M0 block scales): per-token and
 * E8M0 scales are computed and stored, per-head / per-block scales are read.  No counterpart kernel
 * in the reference (it quantises with torch on the host).  `status` may be NULL. */
int cuda_llm_kv_append(const void* k_new, const void* v_new, const int32_t* slot_block,
                       const int32_t* slot_offset, void* key_cache, void* value_cache, void* k_scale,
                       void* v_scale, int32_t n_tokens, int32_t num_kv_heads, int32_t head_dim,
                       int32_t page_size, int32_t num_blocks, int32_t in_dtype, int32_t v_format,
                       int32_t scale_mode, uint32_t* status, void* stream);

/* ---- prefill ------------------------------------------------------------------------- */
/* Where a prefill writes its K / V: the paged, quantised cache the decode entry points read.  Token
 * s of batch row b goes to page slot_block[b * seq_len + s], offset slot_offset[b * seq_len + s];
 * formats and scale modes as in cuda_llm_kv_append.  `status` may be NULL. */
typedef struct CudaLlmKvCacheTarget {
  void* key_cache;
  void* value_cache;
  void* k_scale;
  void* v_scale;
  const int32_t* slot_block;
  const int32_t* slot_offset;
  uint32_t* status;
  int32_t page_size;
  int32_t num_blocks;
  int32_t v_format;   /* CudaLlmKvFormat: CUDA_LLM_KV_FP8_E4M3 or CUDA_LLM_KV_FP4_E2M1 */
  int32_t scale_mode; /* CudaLlmScaleMode */
} CudaLlmKvCacheTarget;

/* Replaces dispatch_fused_gqa<T> (kernels_api.h:52-56; kernel fused_gqa_kernel.cuh:22-212):
 * grouped-query attention over a whole prompt.  q, out [batch, num_q_heads, seq_len, head_dim],
 * k, v [batch, num_kv_heads, seq_len, head_dim], one dtype (fp16 / bf16 run on the tensor cores:
 * tcgen05.mma with TMEM accumulators and TMA operand loads when num_q_heads / num_kv_heads is 1, 2, 4
 * or a multiple of 8, warp-level MMA otherwise; fp32 on a plain fp32 kernel), kv_head = q_head / (num_q_heads / num_kv_heads), causal mask
 * "key position <= query position".  With `cache` not
 * NULL the same call also quantises K and V into the paged cache (the prompt's KV is then ready
 * for the decode entry points); the reference has no such output. */
int cuda_llm_gqa_prefill(const void* q, const void* k, const void* v, void* out, int32_t batch_size,
                         int32_t num_q_heads, int32_t num_kv_heads, int32_t seq_len, int32_t head_dim,
                         float softmax_scale, int32_t is_causal, int32_t dtype,
                         const CudaLlmKvCacheTarget* cache, void* stream);

/* No counterpart in the reference.  Number of bounded waits of the tcgen05 prefill kernel that ran out
 * since the library was loaded on the current device (0 in a healthy process; a non-zero count means
 * some prefill outputs are invalid).  Synchronises the device. */
int cuda_llm_prefill_wait_timeouts(uint32_t* count);

/* No counterpart in the reference.  Calls of this process that ran on the tcgen05 decode kernel
 * (CUDA_LLM_FLAG_TCGEN05), and bounded waits of that kernel that ran out on the current device (the
 * second synchronises the device).  Either pointer may be NULL. */
int cuda_llm_decode_tcgen05_counters(uint64_t* launches, uint32_t* wait_timeouts);

/* No counterpart in the reference.  Calls of cuda_llm_paged_attention (fp32 cache) and
 * cuda_llm_flash_decode (fp32 K/V) by this process that ran on the bulk-copy fp32 kernel; calls with
 * pointers that are not 16-byte aligned run on the plain split-KV kernel.  Failure-path test of that kernel (its entry points
 * carry no flags word): with CUDA_LLM_TEST_STALL=1 in the environment the first copy of a launch is
 * announced and never sent and every wait gives up after a few thousand polls; the wait runs out, the
 * warp returns, CUDA_LLM_ST_TIMEOUT is set in the workspace's status word, nothing faults or hangs. */
int cuda_llm_paged_attention_f32_launches(uint64_t* launches);

/* Replaces dispatch_fused_microscaled_attention<T_OUT> (kernels_api.h:103-108; the reference declares
 * it and ships no definition, test or Python binding, so the semantics are fixed here): dense
 * attention over microscaled FP8 tensors.  q [batch, num_q_heads, seq_len, head_dim] and k, v
 * [batch, num_kv_heads, seq_len, head_dim] hold E4M3 codes, *_scale [batch, heads, seq_len,
 * head_dim/32] one fp32 scale per 32 consecutive elements of head_dim; out [batch, num_q_heads,
 * seq_len, head_dim] of out_dtype = softmax(Q K^T * softmax_scale [+ causal mask]) V over the
 * dequantised tensors. */
int cuda_llm_mx_attention(const void* q, const float* q_scale, const void* k, const float* k_scale, const void* v,
                          const float* v_scale, void* out, int32_t batch_size, int32_t num_q_heads,
                          int32_t num_kv_heads, int32_t seq_len, int32_t head_dim, float softmax_scale,
                          int32_t is_causal, int32_t out_dtype, void* stream);

/* The same operation with a caller-provided workspace of cuda_llm_mx_attention_workspace_bytes() bytes
 * (256-byte aligned; 0 = the shape has no tcgen05 route): q, k and v are first dequantised once into f16
 * tensors in the workspace (code times scale, one rounding: the same operand values the one-kernel route
 * builds on the way into shared memory) and the tcgen05 / tensor-memory prefill kernel runs on those,
 * several times faster on long sequences.  Without a sufficient workspace, or for group sizes that kernel
 * does not take, the call is cuda_llm_mx_attention.  cuda_llm_mx_attention_tcgen05_launches counts the
 * calls of this process that took the tcgen05 route. */
size_t cuda_llm_mx_attention_workspace_bytes(int32_t batch_size, int32_t num_q_heads, int32_t num_kv_heads,
                                             int32_t seq_len, int32_t head_dim);
int cuda_llm_mx_attention_ws(const void* q, const float* q_scale, const void* k, const float* k_scale, const void* v,
                             const float* v_scale, void* out, int32_t batch_size, int32_t num_q_heads,
                             int32_t num_kv_heads, int32_t seq_len, int32_t head_dim, float softmax_scale,
                             int32_t is_causal, int32_t out_dtype, void* workspace, size_t workspace_bytes,
                             void* stream);
int cuda_llm_mx_attention_tcgen05_launches(uint64_t* launches);

/* Bit-exact dequantisation of whole pages to fp32 (test and debugging aid):
 * out [n_pages, Hkv, D, page] fp32 for the pages listed in `pages`. */
int cuda_llm_dequant_pages(const void* cache, const void* scale, const int32_t* pages,
                           int32_t n_pages, int32_t num_kv_heads, int32_t head_dim,
                           int32_t page_size, int32_t format, int32_t scale_mode, float* out,
                           void* stream);

const char* cuda_llm_last_cuda_error(void);
const char* cuda_llm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CUDA_LLM_B200_H_ */
