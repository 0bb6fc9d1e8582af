"""ctypes binding of libcuda_llm_b200.so (the C ABI declared in include/cuda_llm_b200.h).

There is no fallback: if the library is missing the import of any op raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libcuda_llm_b200.so")

OK, EINVAL, EALIGN, EWORKSPACE, ECUDA, EDEVICE = 0, -1, -2, -3, -4, -5
ST_BAD_BLOCK, ST_BAD_CTX, ST_TIMEOUT, ST_BAD_QLEN, ST_SCALE_RANGE, ST_INCOMPLETE, ST_BAD_POSITION = 1, 2, 4, 8, 16, 32, 64
F32, F16, BF16 = 0, 1, 2
KV_FP8_E4M3, KV_FP4_E2M1, KV_INT8, KV_F16, KV_BF16 = 0, 1, 2, 3, 4
SCALE_PER_HEAD, SCALE_PER_BLOCK, SCALE_PER_TOKEN, SCALE_MX_E8M0 = 0, 1, 2, 3
FLAG_SKIP_MERGE = 1
FLAG_STABLE_METADATA = 64   # lengths / offsets / block tables are not written by the kernel in front of the call
FLAG_TEST_STALL = 128       # failure-path test: one stage is announced but never sent; waits give up quickly
FLAG_TCGEN05 = 4096         # run on the tcgen05 / tensor-memory decode kernel where it applies (opt-in, measured slower)


class PagedDecodeParams(C.Structure):
    _fields_ = [
        ("query", C.c_void_p), ("key_cache", C.c_void_p), ("value_cache", C.c_void_p),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("block_tables", C.c_void_p),
        ("context_lens", C.c_void_p), ("cu_q_lens", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("num_seqs", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("page_size", C.c_int32), ("max_blocks_per_seq", C.c_int32),
        ("num_blocks", C.c_int32), ("max_q_len", C.c_int32), ("q_dtype", C.c_int32),
        ("out_dtype", C.c_int32), ("k_format", C.c_int32), ("v_format", C.c_int32),
        ("scale_mode", C.c_int32), ("softmax_scale", C.c_float), ("num_ctas", C.c_int32),
        ("flags", C.c_int32),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("rope_positions", C.c_void_p),
        ("rope_num_positions", C.c_int32),
    ]


class KvCacheTarget(C.Structure):
    _fields_ = [
        ("key_cache", C.c_void_p), ("value_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("slot_block", C.c_void_p), ("slot_offset", C.c_void_p), ("status", C.c_void_p),
        ("page_size", C.c_int32), ("num_blocks", C.c_int32), ("v_format", C.c_int32), ("scale_mode", C.c_int32),
    ]


# name -> (restype, argtypes): every symbol include/cuda_llm_b200.h declares
SYMBOLS = {
    "cuda_llm_paged_decode_workspace_bytes": (C.c_size_t, [C.c_int32] * 7),
    "cuda_llm_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "cuda_llm_paged_decode": (C.c_int, [C.POINTER(PagedDecodeParams), C.c_void_p]),
    "cuda_llm_paged_decode_static": (C.c_int, [C.POINTER(PagedDecodeParams), C.c_void_p]),
    "cuda_llm_static_scratch_bytes": (C.c_size_t, []),
    "cuda_llm_static_decode_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "cuda_llm_dense_decode_workspace_bytes": (C.c_size_t, [C.c_int32] * 5),
    "cuda_llm_paged_attention": (C.c_int, [C.c_void_p] * 6 + [C.c_int32] * 7 + [C.c_float, C.c_int32, C.c_void_p,
                                                                            C.c_size_t, C.c_void_p]),
    "cuda_llm_flash_decode": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 5 + [C.c_float, C.c_int32, C.c_void_p,
                                                                         C.c_size_t, C.c_void_p]),
    "cuda_llm_kv_append": (C.c_int, [C.c_void_p] * 8 + [C.c_int32] * 8 + [C.c_void_p, C.c_void_p]),
    "cuda_llm_decode_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]),
    "cuda_llm_merge_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                          C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "cuda_llm_split_context_exchange_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "cuda_llm_split_context_decode": (C.c_int, [C.POINTER(PagedDecodeParams), C.c_void_p, C.c_int32, C.c_int32,
                                                C.c_void_p, C.c_size_t, C.c_void_p]),
    "cuda_llm_gqa_prefill": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 5 + [C.c_float, C.c_int32, C.c_int32,
                                                                    C.POINTER(KvCacheTarget), C.c_void_p]),
    "cuda_llm_prefill_wait_timeouts": (C.c_int, [C.POINTER(C.c_uint32)]),
    "cuda_llm_decode_tcgen05_counters": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "cuda_llm_paged_attention_f32_launches": (C.c_int, [C.POINTER(C.c_uint64)]),
    "cuda_llm_mx_attention": (C.c_int, [C.c_void_p] * 7 + [C.c_int32] * 5 + [C.c_float, C.c_int32, C.c_int32, C.c_void_p]),
    "cuda_llm_mx_attention_workspace_bytes": (C.c_size_t, [C.c_int32] * 5),
    "cuda_llm_mx_attention_ws": (C.c_int, [C.c_void_p] * 7 + [C.c_int32] * 5 + [C.c_float, C.c_int32, C.c_int32, C.c_void_p,
                                                                                 C.c_size_t, C.c_void_p]),
    "cuda_llm_mx_attention_tcgen05_launches": (C.c_int, [C.POINTER(C.c_uint64)]),
    "cuda_llm_dequant_pages": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                         C.c_void_p]),
    "cuda_llm_last_cuda_error": (C.c_char_p, []),
    "cuda_llm_version": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cuda_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class CudaLlmError(RuntimeError):
    """Raised for a non-zero return code, as the reference binding raises RuntimeError from
    TORCH_CHECK (fused_softmax_binding.cpp:645-669 in the reference project)."""

    def __init__(self, code: int, where: str):
        msg = load().cuda_llm_last_cuda_error().decode()
        super().__init__(f"{where} failed with code {code}: {msg}")
        self.code = code


def check(code: int, where: str) -> None:
    if code != OK:
        raise CudaLlmError(code, where)
