"""The compiled PyTorch extension, imported BY THE REFERENCE'S MODULE NAME, replays the reference's
own test cases (golden outputs of its tests/_utils.py) and the extensions; the ctypes layer is not
on the call path."""
import sys
import time

import pytest
import torch

import cases
from helpers import assert_parity, oracle_out
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu
REF_TOL = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2), torch.float32: (1e-4, 1e-4)}


@pytest.fixture(scope="module")
def ext():
    from cuda_b200 import compat
    sys.path.insert(0, compat.PATH)
    try:
        import fused_online_softmax_cuda as m
    finally:
        sys.path.remove(compat.PATH)
    assert m.__file__.endswith(".so")
    return m


@pytest.mark.parametrize("case", list(cases.paged_cases()), ids=lambda c: c[0])
def test_paged_attention_forward_golden(ext, golden, case):
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v, cases.PAGE, perm)
    out = ext.paged_attention_forward(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), lens_t.cuda())
    atol, rtol = REF_TOL[dtype]
    assert out.dtype == dtype and torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=atol, rtol=rtol)


@pytest.mark.parametrize("case", list(cases.fp8_cases()), ids=lambda c: c[0])
def test_fp8_paged_attention_forward_golden(ext, golden, case):
    """The reference's own E4M3 test (tests/test_kernels_misc.py:42-64 there, xfail against its
    kernel) passes against this module."""
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    k8, v8, ks, vs, _, _ = cases.fp8_quantise(k, v)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k8, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v8, cases.PAGE, perm)
    out = ext.fp8_paged_attention_forward(q.cuda(), kc.cuda(), vc.cuda(), ks.cuda(), vs.cuda(), bt.cuda(),
                                          lens_t.cuda(), softmax_scale=None)
    atol, rtol = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2)}[dtype]
    assert out.dtype == dtype
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=atol, rtol=rtol)


@pytest.mark.parametrize("case", list(cases.decode_cases()), ids=lambda c: c[0])
def test_async_flash_decode_golden(ext, golden, case):
    name, dtype, hd, kv_len = case
    q, k, v = cases.decode_inputs(dtype, hd, kv_len)
    out = ext.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
    atol, rtol = REF_TOL[dtype]
    assert out.shape == q.shape
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=atol, rtol=rtol)


def test_extensions_and_errors(ext):
    from cuda_b200 import workloads as W
    wl = W.make_config(5, batch=12, ctx_scale=1 / 8)                 # MXFP8 K, MXFP4 V, q_len 1/4, GQA
    ref, ref_lse = oracle_out(wl, return_lse=True)
    g = wl.to("cuda")
    out, lse = ext.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale,
                                               g.block_tables, g.context_lens, g.softmax_scale,
                                               cu_q_lens=g.cu_q_lens, max_q_len=g.max_q_len, return_lse=True)
    assert_parity(out, ref, torch.bfloat16, "extension, cfg5")
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2
    wl2 = W.make_config(2, batch=3, ctx_scale=1 / 16).to("cuda")
    i8 = wl2.key_cache.view(torch.int8)
    with pytest.raises(RuntimeError, match="int8 KV caches are not accepted"):
        ext.fp8_paged_attention_forward(wl2.query, i8, wl2.value_cache, wl2.k_scale, wl2.v_scale, wl2.block_tables,
                                        wl2.context_lens)
    a = ext.fp8_paged_attention_forward(wl2.query, i8, wl2.value_cache.view(torch.int8), wl2.k_scale, wl2.v_scale,
                                        wl2.block_tables, wl2.context_lens, kv_format="fp8_e4m3")
    b = ext.fp8_paged_attention_forward(wl2.query, wl2.key_cache, wl2.value_cache, wl2.k_scale, wl2.v_scale,
                                        wl2.block_tables, wl2.context_lens)
    assert torch.equal(a, b)
    with pytest.raises(RuntimeError, match="Query must be 3D"):
        ext.fp8_paged_attention_forward(wl2.query[0], wl2.key_cache, wl2.value_cache, wl2.k_scale, wl2.v_scale,
                                        wl2.block_tables, wl2.context_lens)
    with pytest.raises(RuntimeError, match="Only head_dim 64 and 128 supported"):
        ext.async_flash_decode(torch.zeros(1, 1, 1, 32, device="cuda"), torch.zeros(1, 1, 4, 32, device="cuda"),
                               torch.zeros(1, 1, 4, 32, device="cuda"))


def test_host_overhead_per_call(ext, capsys):
    """Host time of one call (launches queued, no synchronisation inside the loop) through the compiled
    module and through the ctypes layer, on a problem small enough that the host is the limit."""
    from cuda_b200 import ops, workloads as W
    wl = W.make_config(2, batch=2, ctx_scale=1 / 64).to("cuda")
    fns = {
        "extension": lambda: ext.fp8_paged_attention_forward(wl.query, wl.key_cache, wl.value_cache, wl.k_scale,
                                                             wl.v_scale, wl.block_tables, wl.context_lens),
        "ctypes": lambda: ops.fp8_paged_attention_forward(wl.query, wl.key_cache, wl.value_cache, wl.k_scale,
                                                          wl.v_scale, wl.block_tables, wl.context_lens),
    }
    us = {}
    for name, fn in fns.items():
        for _ in range(50):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(500):
            fn()
        us[name] = (time.perf_counter() - t0) / 500 * 1e6
        torch.cuda.synchronize()
    with capsys.disabled():
        print(f"\n[host overhead per call] extension {us['extension']:.1f} us, ctypes {us['ctypes']:.1f} us")
    assert us["extension"] < 200 and us["ctypes"] < 400
