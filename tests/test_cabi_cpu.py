"""The C-ABI library loads, exports every declared symbol, and rejects bad arguments before
touching a device (no compute calls: these run without a GPU)."""
import ctypes as C
import os
import re

import pytest

from cuda_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(L.LIB_PATH):
        from cuda_b200 import build
        build.build()
    return L.load()


def test_exports_every_declared_symbol(lib):
    hdr = open(os.path.join(ROOT, "include", "cuda_llm_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(cuda_llm_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(L.SYMBOLS), (declared ^ set(L.SYMBOLS))
    assert b"sm_100a" in lib.cuda_llm_version()


def test_workspace_bytes_arithmetic(lib):
    f = lib.cuda_llm_paged_decode_workspace_bytes
    # S=64, Hq=32, Hkv=8, D=128, page=16, q_len 1, 148 CTAs: (64+148) slots, each 16 warp
    # partials of 8 rows, 128 + 1 floats per row
    n = f(64, 32, 8, 128, 16, 1, 148)
    rows = (64 + 148) * 16 * 8
    assert n >= rows * 129 * 4 and n < rows * 129 * 4 + 4096 + 64 * 16
    assert f(64, 32, 8, 128, 16, 4, 148) == n         # 8 warp partials of 16 rows
    assert f(128, 32, 8, 128, 16, 1, 148) > n
    assert f(64, 32, 8, 96, 16, 1, 148) == 0          # unsupported head_dim
    assert f(64, 32, 8, 128, 8, 1, 148) == 0          # unsupported page size
    assert f(64, 32, 5, 128, 16, 1, 148) == 0         # Hq not a multiple of Hkv
    assert f(64, 64, 2, 128, 16, 1, 148) == 0         # group 32 > 16 rows


def test_bad_arguments_return_codes(lib):
    assert lib.cuda_llm_paged_decode(None, None) == L.EINVAL
    p = L.PagedDecodeParams()
    p.num_seqs = 0
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.OK       # nothing to do
    p.num_seqs = 1
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.EINVAL   # null tensors
    assert b"null" in lib.cuda_llm_last_cuda_error()
    assert lib.cuda_llm_merge_partials(None, None, 1, 1, 128, None, 0, None, None) == L.EINVAL
    assert lib.cuda_llm_workspace_init(None, 0, None) == L.EWORKSPACE
    st = C.c_uint32(0)
    assert lib.cuda_llm_decode_status(None, None, C.byref(st)) == L.EINVAL
    assert lib.cuda_llm_dequant_pages(None, None, None, 0, 8, 128, 16, 0, 0, None, None) == L.EINVAL


def test_misaligned_and_unsupported(lib):
    p = L.PagedDecodeParams()
    for f in ("query", "key_cache", "value_cache", "k_scale", "v_scale", "block_tables",
              "context_lens", "out", "workspace"):
        setattr(p, f, 0x1000)
    p.workspace_bytes = 1 << 30
    p.num_seqs, p.num_q_heads, p.num_kv_heads, p.head_dim, p.page_size = 2, 8, 8, 64, 16
    p.max_blocks_per_seq, p.num_blocks, p.max_q_len, p.num_ctas = 4, 8, 1, 148
    p.k_format = L.KV_INT8
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.EINVAL   # int8 reading is rejected loudly
    p.k_format = L.KV_FP8_E4M3
    p.key_cache = 0x1008
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.EALIGN
    p.key_cache = 0x1000
    p.head_dim = 96
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.EINVAL
    assert b"head_dim" in lib.cuda_llm_last_cuda_error()
    p.head_dim = 64
    p.workspace_bytes = 16
    assert lib.cuda_llm_paged_decode(C.byref(p), None) == L.EWORKSPACE


def test_int8_caches_are_refused_not_reinterpreted():
    """The reference kernel reads an int8 cache as integers (fp8_paged_attention_kernel.cuh:102 in the
    reference project); this library reads bytes as E4M3 codes, so an int8 tensor is refused unless the
    caller says its bytes are E4M3 codes."""
    import torch
    from cuda_b200 import ops
    c8 = torch.zeros(2, 2, 64, 16, dtype=torch.int8)
    with pytest.raises(RuntimeError, match="int8 KV caches are not accepted"):
        ops._byte_cache_format(c8, c8, None)
    with pytest.raises(RuntimeError, match="int8 KV caches are not accepted"):
        ops._byte_cache_format(c8.view(torch.uint8), c8, None)
    assert ops._byte_cache_format(c8, c8, "fp8_e4m3") == L.KV_FP8_E4M3
    assert ops._byte_cache_format(c8.view(torch.uint8), c8.view(torch.float8_e4m3fn), None) == L.KV_FP8_E4M3
    with pytest.raises(RuntimeError, match="8-bit quantized"):
        ops._byte_cache_format(c8.half(), c8.half(), None)
    with pytest.raises(RuntimeError, match="unknown kv_format"):
        ops._byte_cache_format(c8, c8, "int8")


def test_ops_fail_loudly_without_library(monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", "/nonexistent/libcuda_llm_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        L.load()


CXX_SYMBOLS = {
    ("paged", "f32"): "_Z24dispatch_paged_attentionIfEvPKT_S2_S2_PKiS4_PS0_iiiifP11CUstream_st",
    ("paged", "f16"): "_Z24dispatch_paged_attentionI6__halfEvPKT_S3_S3_PKiS5_PS1_iiiifP11CUstream_st",
    ("paged", "bf16"): "_Z24dispatch_paged_attentionI13__nv_bfloat16EvPKT_S3_S3_PKiS5_PS1_iiiifP11CUstream_st",
    ("decode", "f32"): "_Z27dispatch_async_flash_decodeIfEvPKT_S2_S2_PS0_iiiifP11CUstream_st",
    ("decode", "f16"): "_Z27dispatch_async_flash_decodeI6__halfEvPKT_S3_S3_PS1_iiiifP11CUstream_st",
    ("decode", "bf16"): "_Z27dispatch_async_flash_decodeI13__nv_bfloat16EvPKT_S3_S3_PS1_iiiifP11CUstream_st",
    ("fp8", "f32"): "_Z28dispatch_fp8_paged_attentionIffEvPKT0_PKaS4_PKfS6_PKiS8_PT_iiiiifbP11CUstream_st",
    ("fp8", "f16"): "_Z28dispatch_fp8_paged_attentionI6__halfS0_EvPKT0_PKaS5_PKfS7_PKiS9_PT_iiiiifbP11CUstream_st",
    ("fp8", "bf16"): "_Z28dispatch_fp8_paged_attentionI13__nv_bfloat16S0_EvPKT0_PKaS5_PKfS7_PKiS9_PT_iiiiifbP11CUstream_st",
    ("gqa", "f32"): "_Z18dispatch_fused_gqaIfEvPKT_S2_S2_PS0_iiiiifbP11CUstream_st",
    ("gqa", "f16"): "_Z18dispatch_fused_gqaI6__halfEvPKT_S3_S3_PS1_iiiiifbP11CUstream_st",
    ("gqa", "bf16"): "_Z18dispatch_fused_gqaI13__nv_bfloat16EvPKT_S3_S3_PS1_iiiiifbP11CUstream_st",
}


def test_reference_cxx_dispatchers_are_exported(lib):
    """The three templates of the reference's kernels_api.h, instantiated for its three dtypes, under
    the names its binding's object file asks the linker for (Itanium mangling of those signatures)."""
    for name in CXX_SYMBOLS.values():
        assert hasattr(lib, name), name


def test_reference_module_names_import():
    """The compiled extension under the reference's module name loads without a GPU, exposes the three
    decode entry points with the reference's argument names and defaults (fused_softmax_binding.cpp
    :733-741, :759-763, :800-807 in the reference project), and the cuda_llm package re-exports them."""
    import importlib
    import sys
    import torch
    from cuda_b200 import build, compat
    if not os.path.exists(build.extension_path()):
        build.build_extension()
    sys.path.insert(0, compat.PATH)
    try:
        ext = importlib.import_module("fused_online_softmax_cuda")
        pkg = importlib.import_module("cuda_llm")
    finally:
        sys.path.remove(compat.PATH)
    assert ext.__file__.endswith(".so")                    # a compiled module, not a Python shim
    sig = ext.paged_attention_forward.__doc__
    for name in ("query", "key_cache", "value_cache", "block_tables", "context_lens", "softmax_scale"):
        assert name in sig
    sig = ext.fp8_paged_attention_forward.__doc__
    for name in ("query", "key_cache_fp8", "value_cache_fp8", "k_scale", "v_scale", "block_tables", "context_lens",
                 "softmax_scale", "cu_q_lens", "max_q_len", "return_lse", "kv_format"):
        assert name in sig
    for name in ("q:", "k:", "v:", "softmax_scale"):
        assert name in ext.async_flash_decode.__doc__
    assert pkg.flash_decode is ext.async_flash_decode
    assert pkg.paged_attention is ext.paged_attention_forward
    assert pkg.fp8_paged_attention is ext.fp8_paged_attention_forward
    # the reference's TORCH_CHECK messages, reached before any device work
    q = torch.zeros(2, 4, 64)
    c = torch.zeros(4, 4, 64, 16)
    bt = torch.zeros(2, 2, dtype=torch.int32)
    cl = torch.ones(2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="Inputs must be on CUDA"):
        ext.paged_attention_forward(q, c, c, bt, cl)
    with pytest.raises(RuntimeError, match="Inputs must be on CUDA"):
        ext.fp8_paged_attention_forward(q, c.to(torch.uint8), c.to(torch.uint8), cl.float(), cl.float(), bt, cl)
    with pytest.raises(RuntimeError, match="Inputs must be on CUDA"):
        ext.async_flash_decode(q[:, :, None], q[:, :, None], q[:, :, None])
    for mod in ("fused_online_softmax_cuda", "cuda_llm"):
        sys.modules.pop(mod, None)
