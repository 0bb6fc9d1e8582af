"""GQA prefill (the reference's fused_gqa_forward) and its paged-KV output."""
import pytest
import torch

import cases
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu
REF_TOL = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2), torch.float32: (1e-4, 1e-4)}


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


@pytest.mark.parametrize("case", list(cases.gqa_cases()), ids=lambda c: c[0])
def test_reference_gqa_cases(ops, golden, case):
    """The reference's own test grid (tests/test_attention.py:43-54 there): sampled rows against the
    outputs of its ref_gqa, every row against the oracle (which reproduces ref_gqa bit for bit)."""
    name, dtype, hd, hq, hkv, causal = case
    q, k, v = cases.gqa_inputs(dtype, hd, hq, hkv)
    out = ops.fused_gqa_forward(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
    atol, rtol = REF_TOL[dtype]
    assert out.dtype == dtype and out.shape == q.shape and torch.isfinite(out).all()
    rows = torch.from_numpy(golden[f"{name}/rows"])
    assert torch.allclose(out[:, :, list(cases.GQA_ROWS), :].float().cpu(), rows, atol=atol, rtol=rtol)
    assert torch.allclose(out.float().cpu(), O.ref_gqa(q, k, v, causal), atol=atol, rtol=rtol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,hq,hkv,s,d,causal", [(2, 32, 8, 300, 128, True), (1, 12, 4, 129, 64, True),
                                                 (3, 16, 1, 64, 128, False), (1, 6, 2, 1, 64, True),
                                                 (2, 5, 5, 77, 128, True), (1, 24, 2, 200, 64, False),
                                                 (1, 10, 2, 700, 128, True), (1, 14, 2, 513, 128, True),
                                                 (2, 12, 2, 260, 64, True)])
def test_gqa_shapes(ops, dtype, b, hq, hkv, s, d, causal):
    """Group sizes 1..16 (the heads of a group share a CTA eight, four, two or one at a time, whichever divides
    the group), ragged lengths, all three dtypes of the reference's instantiations."""
    g = torch.Generator().manual_seed(b * 1000 + s)
    q = torch.randn(b, hq, s, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, s, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, s, d, generator=g).to(dtype)
    out = ops.fused_gqa_forward(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
    atol, rtol = REF_TOL[dtype]
    assert torch.allclose(out.float().cpu(), O.ref_gqa(q, k, v, causal), atol=atol, rtol=rtol)


@pytest.mark.parametrize("mode,vfmt", [("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"), ("mx_e8m0", "fp4_e2m1")])
def test_prefill_fills_the_paged_cache_for_decode(ops, mode, vfmt):
    """Prefill with a paged-KV target, then one decode step over the cache it wrote: the cache bytes and
    scales equal the host recipe bit for bit, and the decode output matches the oracle on that cache."""
    from cuda_b200 import workloads as W
    from helpers import assert_parity
    b, hq, hkv, s, d, page = 2, 16, 4, 150, 128, 16
    g = torch.Generator().manual_seed(7)
    q = torch.randn(b, hq, s, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    n_pages = (s + page - 1) // page
    pool = b * n_pages + 3
    perm = torch.randperm(pool, generator=g)[: b * n_pages]
    bt = perm.view(b, n_pages).to(torch.int32)
    pos = torch.arange(s)
    slot_block = bt[:, pos // page].reshape(-1)
    slot_offset = (pos % page).repeat(b).to(torch.int32)
    dv = d if vfmt == "fp8_e4m3" else d // 2
    kc = torch.zeros(pool, hkv, d, page, dtype=torch.uint8, device="cuda")
    vc = torch.zeros(pool, hkv, dv, page, dtype=torch.uint8, device="cuda")
    if mode == "per_token":
        ks = torch.ones(pool, hkv, page, device="cuda")
        vs = torch.ones(pool, hkv, page, device="cuda")
    else:
        ks = torch.full((pool, hkv, d // 32, page), 127, dtype=torch.uint8, device="cuda")
        vs = torch.full((pool, hkv, d // 32, page), 127, dtype=torch.uint8, device="cuda")
    out = ops.fused_gqa_forward(q.cuda(), k.cuda(), v.cuda(), is_causal=True,
                                paged_kv=(kc, vc, ks, vs, slot_block, slot_offset))
    assert torch.allclose(out.float().cpu(), O.ref_gqa(q, k, v, True), atol=4e-2, rtol=4e-2)
    # the cache against the host statement of the write recipe, token by token
    kt = k.permute(0, 2, 1, 3).reshape(b * s, hkv, d).float()
    vt = v.permute(0, 2, 1, 3).reshape(b * s, hkv, d).float()
    kq, ksc = O.quantize_tokens(kt, "fp8_e4m3", mode)
    vq, vsc = O.quantize_tokens(vt, vfmt, mode)
    sb, so = slot_block.long(), slot_offset.long()
    assert torch.equal(kc.cpu()[sb, :, :, so], kq)
    assert torch.equal(vc.cpu()[sb, :, :, so], vq)
    if mode == "per_token":
        assert torch.equal(ks.cpu()[sb, :, so], ksc) and torch.equal(vs.cpu()[sb, :, so], vsc)
    else:
        assert torch.equal(ks.cpu()[sb, :, :, so], ksc) and torch.equal(vs.cpu()[sb, :, :, so], vsc)
    # one decode step over what the prefill wrote
    ctx = torch.full((b,), s, dtype=torch.int32)
    qd = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
    kv = O.PagedKV(kc.cpu(), vc.cpu(), bt, ctx, page, d, "fp8_e4m3", vfmt, mode, mode, ks.cpu(), vs.cpu())
    ref = O.ref_paged_decode(qd, kv)
    dec = ops.fp8_paged_attention_forward(qd.cuda(), kc, vc, ks, vs, bt.cuda(), ctx.cuda(), check_status=True)
    assert_parity(dec, ref, torch.bfloat16, "decode after prefill")


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,hq,hkv,s,d,causal", [(2, 8, 8, 200, 128, True), (1, 16, 4, 77, 64, False),
                                                 (1, 4, 4, 1, 128, True)])
def test_microscaled_attention(ops, out_dtype, b, hq, hkv, s, d, causal):
    """Dense attention over E4M3 tensors with one fp32 scale per 32 elements of head_dim (the entry
    point the reference declares and never defines), against the oracle's dequantise-then-attend."""
    g = torch.Generator().manual_seed(s + d)

    def quant(h):
        x = torch.randn(b, h, s, d, generator=g) * torch.exp(0.3 * torch.randn(b, h, s, 1, generator=g))
        sc = (x.view(b, h, s, d // 32, 32).abs().amax(-1) / 448.0).clamp_min(1e-8)
        codes = (x.view(b, h, s, d // 32, 32) / sc.unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8)
        return codes.view(b, h, s, d), sc

    (q8, qs), (k8, ks), (v8, vs) = quant(hq), quant(hkv), quant(hkv)
    ref = O.ref_mx_attention(q8, qs, k8, ks, v8, vs, causal)
    out = ops.fused_microscaled_attention(q8.cuda(), qs.cuda(), k8.cuda(), ks.cuda(), v8.cuda(), vs.cuda(),
                                          is_causal=causal, out_dtype=out_dtype)
    assert out.dtype == out_dtype and torch.isfinite(out).all()
    scale = ref.abs().amax().clamp_min(1.0)
    err = (out.float().cpu() - ref).abs() / scale
    # the operands reach the tensor cores as f16 (codes times scale rounded once, P rounded to f16), so
    # every output dtype is held to the stated bf16 tolerance; fp32 / f16 outputs are well inside it
    assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())
    if out_dtype != torch.bfloat16:
        assert err.max().item() <= 8e-3


def _mx_launches(ops):
    import ctypes as C
    n = C.c_uint64(0)
    ops.L.check(ops.L.load().cuda_llm_mx_attention_tcgen05_launches(C.byref(n)), "counter")
    return n.value


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,hq,hkv,s,d,causal", [(1, 32, 8, 1000, 128, True), (2, 8, 8, 333, 128, False),
                                                 (1, 16, 2, 520, 64, True), (1, 4, 2, 129, 128, True)])
def test_microscaled_attention_tcgen05_route(ops, out_dtype, b, hq, hkv, s, d, causal):
    """The route through dequantised f16 operands and the tcgen05 / tensor-memory kernel (taken when the
    caller gives a workspace, as the Python op does) and the one-kernel route of the same call without a
    workspace, both against the oracle's dequantise-then-attend; fp32, f16 and bf16 outputs."""
    g = torch.Generator().manual_seed(s + d + hq)

    def quant(h):
        x = torch.randn(b, h, s, d, generator=g) * torch.exp(0.3 * torch.randn(b, h, s, 1, generator=g))
        sc = (x.view(b, h, s, d // 32, 32).abs().amax(-1) / 448.0).clamp_min(1e-8)
        codes = (x.view(b, h, s, d // 32, 32) / sc.unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8)
        return codes.view(b, h, s, d), sc

    (q8, qs), (k8, ks), (v8, vs) = quant(hq), quant(hkv), quant(hkv)
    ref = O.ref_mx_attention(q8, qs, k8, ks, v8, vs, causal)
    dev = [t.cuda() for t in (q8, qs, k8, ks, v8, vs)]
    before = _mx_launches(ops)
    out = ops.fused_microscaled_attention(*dev, is_causal=causal, out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert _mx_launches(ops) == before + 1, "the call did not take the tcgen05 route"
    # the same call without a workspace: the one-kernel route
    lib = ops.L.load()
    plain = torch.empty_like(out)
    ops.L.check(lib.cuda_llm_mx_attention(dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(),
                                          dev[4].data_ptr(), dev[5].data_ptr(), plain.data_ptr(), b, hq, hkv, s, d,
                                          1.0 / d ** 0.5, 1 if causal else 0, ops._DTYPE[out_dtype], None), "mx_attention")
    torch.cuda.synchronize()
    assert _mx_launches(ops) == before + 1
    scale = ref.abs().amax().clamp_min(1.0)
    for name, o in (("tcgen05", out), ("one kernel", plain)):
        assert o.dtype == out_dtype and torch.isfinite(o).all(), name
        err = (o.float().cpu() - ref).abs() / scale
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (name, err.max().item(), err.mean().item())
        if out_dtype != torch.bfloat16:
            assert err.max().item() <= 8e-3, (name, err.max().item())


def test_microscaled_dispatcher_symbol(ops):
    """dispatch_fused_microscaled_attention<T_OUT> exists under the reference's mangled names."""
    lib = ops.L.load()
    for sym in ("_Z36dispatch_fused_microscaled_attentionIfEvPKaPKfS1_S3_S1_S3_PT_iiiifbP11CUstream_st",
                "_Z36dispatch_fused_microscaled_attentionI6__halfEvPKaPKfS2_S4_S2_S4_PT_iiiifbP11CUstream_st",
                "_Z36dispatch_fused_microscaled_attentionI13__nv_bfloat16EvPKaPKfS2_S4_S2_S4_PT_iiiifbP11CUstream_st"):
        assert hasattr(lib, sym), sym


def test_no_prefill_wait_ran_out(ops):
    """Collected after the prefill tests of this file: none of the bounded waits of the tcgen05 kernel
    gave up."""
    import ctypes as C
    n = C.c_uint32(123)
    ops.L.check(ops.L.load().cuda_llm_prefill_wait_timeouts(C.byref(n)), "cuda_llm_prefill_wait_timeouts")
    assert n.value == 0
