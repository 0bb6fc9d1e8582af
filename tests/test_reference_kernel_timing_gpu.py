"""Times the REFERENCE's own CUDA paged-decode kernels (compiled for sm_100a into
oracle/_ref/libref_paged.so by oracle/Makefile) next to this library's entry points on the same
inputs, on the shapes the reference supports (MHA, page 16, q_len 1), and prints one line per case:

    python -m pytest tests/test_reference_kernel_timing_gpu.py -m gpu -s

The reference's 8-bit kernel reads the cache bytes as int8, so its output differs from the E4M3
path by design; only its time is compared.  The fp16 kernel's output is also checked against
this library's paged_attention.  Skipped where oracle/_ref was not built.
"""
import ctypes as C
import os
import sys

import torch

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

REF = os.path.join(ROOT, "oracle", "_ref", "libref_paged.so")


def timeit(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


@pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref not built")
def test_reference_kernels_are_slower_than_this_library(capsys):
    from cuda_b200 import ops, workloads as W
    ref = C.CDLL(REF)
    lines, ratios = [], []
    st = lambda: torch.cuda.current_stream().cuda_stream
    cg = torch.Generator()
    cg.manual_seed(1002)
    for batch, heads in ((64, 8), (64, 32)):
        lens = torch.randint(1024, 8193, (batch,), generator=cg).tolist()
        # ---- fp16 paged cache, MHA
        wl = W.build_workload("ref_f16", context_lens=lens, q_lens=None, num_q_heads=heads, num_kv_heads=heads,
                              head_dim=128, page_size=16, q_dtype=torch.float16, scale_mode="none",
                              pool_factor=1.25, seed=1, device="cuda", cache_dtype=torch.float16)
        nbytes = sum(lens) * heads * 128 * 2 * 2
        out_ref = torch.empty_like(wl.query)

        def run_ref():
            ref.ref_paged_attention(C.c_void_p(wl.query.data_ptr()), C.c_void_p(wl.key_cache.data_ptr()),
                                    C.c_void_p(wl.value_cache.data_ptr()), C.c_void_p(wl.block_tables.data_ptr()),
                                    C.c_void_p(wl.context_lens.data_ptr()), C.c_void_p(out_ref.data_ptr()),
                                    batch, heads, 128, wl.block_tables.shape[1], C.c_float(wl.softmax_scale), 1,
                                    C.c_void_p(st()))
        t_ref = timeit(run_ref, iters=5, warm=1)
        ours = ops.paged_attention_forward(wl.query, wl.key_cache, wl.value_cache, wl.block_tables, wl.context_lens)
        err = (ours.float() - out_ref.float()).abs().max().item()
        t_ours = timeit(lambda: ops.paged_attention_forward(wl.query, wl.key_cache, wl.value_cache,
                                                            wl.block_tables, wl.context_lens))
        lines.append(f"fp16 paged  batch {batch} heads {heads}: {nbytes/1e6:8.1f} MB  reference kernel {t_ref*1e3:9.1f} us "
                     f"({nbytes/t_ref/1e9:6.3f} TB/s)  this library {t_ours*1e3:8.1f} us ({nbytes/t_ours/1e9:6.3f} TB/s)  "
                     f"max |diff| {err:.2e}")
        ratios.append(t_ref / t_ours)
        assert err <= 2e-2
        del wl, out_ref, ours
        # ---- 8-bit paged cache, per-head scales, MHA
        wl = W.build_workload("ref_8bit", context_lens=lens, q_lens=None, num_q_heads=heads, num_kv_heads=heads,
                              head_dim=128, page_size=16, q_dtype=torch.float16, scale_mode="per_head",
                              pool_factor=1.25, seed=2, device="cuda", poison=False)
        nbytes = sum(lens) * heads * 128 * 2
        out_ref = torch.empty_like(wl.query)

        def run_ref8():
            ref.ref_int8_paged_attention(C.c_void_p(wl.query.data_ptr()), C.c_void_p(wl.key_cache.data_ptr()),
                                         C.c_void_p(wl.value_cache.data_ptr()), C.c_void_p(wl.k_scale.data_ptr()),
                                         C.c_void_p(wl.v_scale.data_ptr()), C.c_void_p(wl.block_tables.data_ptr()),
                                         C.c_void_p(wl.context_lens.data_ptr()), C.c_void_p(out_ref.data_ptr()),
                                         batch, heads, 128, wl.block_tables.shape[1], C.c_float(wl.softmax_scale), 0,
                                         C.c_void_p(st()))
        t_ref = timeit(run_ref8, iters=5, warm=1)
        ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
        out = torch.empty_like(wl.query)
        t_ours = timeit(lambda: ops.run_workload(wl, out=out, workspace=ws))
        lines.append(f"8-bit paged batch {batch} heads {heads}: {nbytes/1e6:8.1f} MB  reference kernel {t_ref*1e3:9.1f} us "
                     f"({nbytes/t_ref/1e9:6.3f} TB/s, int8 reading)  this library {t_ours*1e3:8.1f} us "
                     f"({nbytes/t_ours/1e9:6.3f} TB/s, E4M3)")
        ratios.append(t_ref / t_ours)
        del wl, out_ref, out, ws
    with capsys.disabled():
        print()
        for line in lines:
            print(line, flush=True)
    assert min(ratios) > 1.0
