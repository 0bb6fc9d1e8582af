"""The allocation-free entry point gives the same answer as the ordinary one.

cuda_llm_paged_decode_static() exists for callers that are not allowed to allocate device memory
at call time (a plugin inside a runtime that owns the memory pool, a latency-critical serving
thread): its split partials live in an array compiled into the library instead of a
caller-provided workspace.  This file is collected last on purpose, so that a run that stops at the
first failure has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

from helpers import assert_parity

pytestmark = pytest.mark.gpu


def _params(L, wl, out, ws):
    return L.PagedDecodeParams(
        query=wl.query.data_ptr(), key_cache=wl.key_cache.data_ptr(), value_cache=wl.value_cache.data_ptr(),
        k_scale=wl.k_scale.data_ptr(), v_scale=wl.v_scale.data_ptr(), block_tables=wl.block_tables.data_ptr(),
        context_lens=wl.context_lens.data_ptr(), cu_q_lens=None, out=out.data_ptr(), lse=None,
        workspace=None if ws is None else ws.data_ptr(), workspace_bytes=0 if ws is None else ws.numel(),
        num_seqs=wl.num_seqs, num_q_heads=wl.num_q_heads, num_kv_heads=wl.num_kv_heads, head_dim=wl.head_dim,
        page_size=wl.page_size, max_blocks_per_seq=wl.block_tables.shape[1], num_blocks=wl.key_cache.shape[0],
        max_q_len=1, q_dtype=L.BF16, out_dtype=L.BF16, k_format=L.KV_FP8_E4M3, v_format=L.KV_FP8_E4M3,
        scale_mode=L.SCALE_PER_TOKEN, softmax_scale=wl.softmax_scale, num_ctas=0, flags=0)


def test_static_scratch_matches_workspace_entry_point():
    from cuda_b200 import _lib as L, workloads
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first call's leftovers
    for seed, batch in ((21, 6), (22, 3)):
        wl = workloads.make_config(2, "cuda", batch=batch, ctx_scale=1 / 8, seed=seed)
        need = lib.cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads,
                                                         wl.head_dim, wl.page_size, 1, 0)
        assert 0 < need <= lib.cuda_llm_static_scratch_bytes()
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        ref = torch.empty_like(wl.query)
        out = torch.full_like(wl.query, float("nan"))
        L.check(lib.cuda_llm_paged_decode(C.byref(_params(L, wl, ref, ws)), stream), "cuda_llm_paged_decode")
        L.check(lib.cuda_llm_paged_decode_static(C.byref(_params(L, wl, out, None)), stream),
                "cuda_llm_paged_decode_static")
        torch.cuda.synchronize()
        assert_parity(out, ref, torch.bfloat16, f"static scratch, batch {batch}")
        assert torch.equal(out, ref)          # same kernels, same split: bit-identical


def test_static_scratch_refuses_what_does_not_fit():
    from cuda_b200 import _lib as L, workloads
    lib = L.load()
    wl = workloads.make_config(2, "cuda", batch=2, ctx_scale=1 / 16, seed=5)
    out = torch.empty_like(wl.query)
    p = _params(L, wl, out, None)
    p.num_seqs = 4096                          # (4096 + SMs) slots of partials: far beyond 16 MiB
    rc = lib.cuda_llm_paged_decode_static(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == L.EWORKSPACE
    assert b"16 MiB" in lib.cuda_llm_last_cuda_error()


def test_static_scratch_status_is_readable():
    """A block-table entry outside the pool through the allocation-free entry point: the finding
    lands in the status word of the built-in scratch and cuda_llm_static_decode_status reads it."""
    from cuda_b200 import _lib as L, workloads
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    st = C.c_uint32(0xFFFFFFFF)
    L.check(lib.cuda_llm_static_decode_status(stream, C.byref(st)), "cuda_llm_static_decode_status")
    assert st.value == 0                       # the other tests of this file left nothing behind
    wl = workloads.make_config(2, "cpu", batch=2, ctx_scale=1 / 16, seed=6)
    wl.block_tables[1, 0] = 1_000_000
    wl = wl.to("cuda")
    out = torch.empty_like(wl.query)
    L.check(lib.cuda_llm_paged_decode_static(C.byref(_params(L, wl, out, None)), stream),
            "cuda_llm_paged_decode_static")
    L.check(lib.cuda_llm_static_decode_status(stream, C.byref(st)), "cuda_llm_static_decode_status")
    assert st.value & L.ST_BAD_BLOCK
    L.check(lib.cuda_llm_static_decode_status(stream, C.byref(st)), "cuda_llm_static_decode_status")
    assert st.value == 0                       # cleared by the read
