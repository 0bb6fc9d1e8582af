"""The cache-append kernel writes exactly the bytes and scales of the oracle's statement of the write
recipe (torch / ml_dtypes casts), at the right place of the paged layout, and the decode kernel reads
them back."""
import pytest
import torch

from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,vfmt", [("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"),
                                       ("mx_e8m0", "fp4_e2m1"), ("per_head", "fp8_e4m3")])
@pytest.mark.parametrize("d,page,dtype", [(128, 16, torch.bfloat16), (64, 32, torch.float32), (128, 64, torch.float16)])
def test_append_is_bit_exact(mode, vfmt, d, page, dtype):
    from cuda_b200 import ops, workloads as W
    torch.manual_seed(3)
    n, h, nb = 37, 4, 11
    # magnitudes spread over many binades so that block exponents and subnormal codes are exercised
    mag = torch.exp2(torch.randint(-12, 6, (n, h, d // 32, 1)).float()).expand(n, h, d // 32, 32).reshape(n, h, d)
    k = (torch.randn(n, h, d) * mag).to(dtype)
    v = (torch.randn(n, h, d) * mag).to(dtype)
    k[3] = 0                                                   # an all-zero token
    slots = torch.randperm(nb * page)[:n]
    blk, off = (slots // page).to(torch.int32), (slots % page).to(torch.int32)
    # per-head scales by the reference recipe (tests/test_kernels_misc.py:51-52): amax / 448 per head
    k_head = (k.float().abs().amax(dim=(0, 2)) / 448.0).clamp_min(1e-8)
    v_head = (v.float().abs().amax(dim=(0, 2)) / 448.0).clamp_min(1e-8)
    kc_ref, ks_ref = O.quantize_tokens(k.float(), "fp8_e4m3", mode, k_head)
    vc_ref, vs_ref = O.quantize_tokens(v.float(), vfmt, mode, v_head)
    dv = d // 2 if vfmt == "fp4_e2m1" else d
    kc = torch.full((nb, h, d, page), 0xAA, dtype=torch.uint8, device="cuda")
    vc = torch.full((nb, h, dv, page), 0xAA, dtype=torch.uint8, device="cuda")
    if mode == "per_token":
        ks = torch.full((nb, h, page), -1.0, device="cuda"); vs = ks.clone()
    elif mode == "mx_e8m0":
        ks = torch.full((nb, h, d // 32, page), 0xAA, dtype=torch.uint8, device="cuda"); vs = ks.clone()
    else:
        ks = k_head.cuda(); vs = v_head.cuda()
    ops.kv_cache_append(k.cuda(), v.cuda(), blk.cuda(), off.cuda(), kc, vc, ks, vs)
    torch.cuda.synchronize()
    b, o = blk.long(), off.long()
    assert torch.equal(kc.cpu()[b, :, :, o], kc_ref)            # [n,h,d]
    assert torch.equal(vc.cpu()[b, :, :, o], vc_ref)
    if mode == "per_token":
        assert torch.equal(ks.cpu()[b, :, o], ks_ref) and torch.equal(vs.cpu()[b, :, o], vs_ref)
    elif mode == "mx_e8m0":
        assert torch.equal(ks.cpu()[b, :, :, o], ks_ref) and torch.equal(vs.cpu()[b, :, :, o], vs_ref)
    # untouched slots keep their fill
    untouched = torch.ones(nb, page, dtype=torch.bool)
    untouched[b, o] = False
    assert (kc.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all()


@pytest.mark.parametrize("mode,vfmt", [("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"),
                                       ("mx_e8m0", "fp4_e2m1"), ("per_head", "fp8_e4m3")])
@pytest.mark.parametrize("d,page,dtype", [(128, 16, torch.bfloat16), (64, 32, torch.float32), (128, 64, torch.float16),
                                          (64, 16, torch.bfloat16)])
def test_append_of_many_tokens_is_bit_exact(mode, vfmt, d, page, dtype):
    """A prefill's worth of tokens (the kernel that writes whole 16-token rows): a page-aligned sequence
    (full-width rows), a sequence that starts in the middle of a page (every group of 16 straddles the row
    grid: byte stores), scattered single tokens and a ragged last group, in one call."""
    from cuda_b200 import ops
    torch.manual_seed(5)
    h = 4
    n_a, n_b, n_c = 40 * page + 16, 517, 77        # aligned, misaligned by 5 slots, scattered
    n = n_a + n_b + n_c
    assert n >= 1024 and n % 16 != 0
    pages_a, pages_b = (n_a + page - 1) // page, (n_b + 5 + page - 1) // page
    nb = pages_a + pages_b + 12
    perm = torch.randperm(nb)
    blk = torch.empty(n, dtype=torch.int64)
    off = torch.empty(n, dtype=torch.int64)
    ta = torch.arange(n_a)
    blk[:n_a], off[:n_a] = perm[ta // page], ta % page
    tb = torch.arange(n_b) + 5
    blk[n_a:n_a + n_b], off[n_a:n_a + n_b] = perm[pages_a + tb // page], tb % page
    free = perm[pages_a + pages_b:]                                       # 12 pages for the scattered tokens
    slots = torch.randperm(12 * page)[:n_c]
    blk[n_a + n_b:], off[n_a + n_b:] = free[slots // page], slots % page
    mag = torch.exp2(torch.randint(-12, 6, (n, h, d // 32, 1)).float()).expand(n, h, d // 32, 32).reshape(n, h, d)
    k = (torch.randn(n, h, d) * mag).to(dtype)
    v = (torch.randn(n, h, d) * mag).to(dtype)
    k[3] = 0
    k[5, :, ::3] = -0.0                                         # negative zeros keep their sign bit
    k_head = (k.float().abs().amax(dim=(0, 2)) / 448.0).clamp_min(1e-8)
    v_head = (v.float().abs().amax(dim=(0, 2)) / 448.0).clamp_min(1e-8)
    kc_ref, ks_ref = O.quantize_tokens(k.float(), "fp8_e4m3", mode, k_head)
    vc_ref, vs_ref = O.quantize_tokens(v.float(), vfmt, mode, v_head)
    dv = d // 2 if vfmt == "fp4_e2m1" else d
    kc = torch.full((nb, h, d, page), 0xAA, dtype=torch.uint8, device="cuda")
    vc = torch.full((nb, h, dv, page), 0xAA, dtype=torch.uint8, device="cuda")
    if mode == "per_token":
        ks = torch.full((nb, h, page), -1.0, device="cuda"); vs = ks.clone()
    elif mode == "mx_e8m0":
        ks = torch.full((nb, h, d // 32, page), 0xAA, dtype=torch.uint8, device="cuda"); vs = ks.clone()
    else:
        ks = k_head.cuda(); vs = v_head.cuda()
    ops.kv_cache_append(k.cuda(), v.cuda(), blk.to(torch.int32).cuda(), off.to(torch.int32).cuda(), kc, vc, ks, vs)
    torch.cuda.synchronize()
    assert torch.equal(kc.cpu()[blk, :, :, off], kc_ref)
    assert torch.equal(vc.cpu()[blk, :, :, off], vc_ref)
    if mode == "per_token":
        assert torch.equal(ks.cpu()[blk, :, off], ks_ref) and torch.equal(vs.cpu()[blk, :, off], vs_ref)
    elif mode == "mx_e8m0":
        assert torch.equal(ks.cpu()[blk, :, :, off], ks_ref) and torch.equal(vs.cpu()[blk, :, :, off], vs_ref)
    untouched = torch.ones(nb, page, dtype=torch.bool)
    untouched[blk, off] = False
    assert (kc.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all()
    assert (vc.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all()
    if mode == "mx_e8m0":
        assert (ks.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all()
    elif mode == "per_token":
        assert (ks.cpu().permute(0, 2, 1)[untouched] == -1.0).all()


def test_append_quotients_are_ieee_on_fp32_inputs():
    """The kernel for many tokens divides by the per-token scale through a reciprocal and two fused
    multiply-adds, which must give the IEEE quotient the oracle's recipe (torch's fp32 division) gives:
    two million fp32 values with full-width significands, uniform over [-amax, amax] of their token, token maxima
    over 60 binades, scales whose significand is all ones among them."""
    from cuda_b200 import ops
    g = torch.Generator().manual_seed(11)
    n, h, d, page = 8192, 2, 128, 16
    amax = torch.exp2(torch.randint(-30, 30, (n, h, 1), generator=g).float()) * (1 + torch.rand(n, h, 1, generator=g))
    # a scale of 2^k (2 - 2^-23): amax = 448 * that, rounded; the quotient path must still be exact
    amax[::97] = 448.0 * torch.tensor(1.9999998807907104) * torch.exp2(torch.randint(-20, 10, (len(amax[::97]), h, 1), generator=g).float())
    k = (torch.rand(n, h, d, generator=g) * 2 - 1) * amax
    k[..., 0] = amax[..., 0]                                    # the maximum itself is present
    v = k.flip(0).contiguous()
    kc_ref, ks_ref = O.quantize_tokens(k, "fp8_e4m3", "per_token", None)
    vc_ref, vs_ref = O.quantize_tokens(v, "fp8_e4m3", "per_token", None)
    t = torch.arange(n)
    blk, off = (t // page).to(torch.int32).cuda(), (t % page).to(torch.int32).cuda()
    kc = torch.zeros(n // page, h, d, page, dtype=torch.uint8, device="cuda"); vc = torch.zeros_like(kc)
    ks = torch.zeros(n // page, h, page, device="cuda"); vs = torch.zeros_like(ks)
    ops.kv_cache_append(k.cuda(), v.cuda(), blk, off, kc, vc, ks, vs)
    torch.cuda.synchronize()
    b, o = (t // page), (t % page)
    assert torch.equal(ks.cpu()[b, :, o], ks_ref) and torch.equal(vs.cpu()[b, :, o], vs_ref)
    assert torch.equal(kc.cpu()[b, :, :, o], kc_ref)
    assert torch.equal(vc.cpu()[b, :, :, o], vc_ref)


def test_append_of_many_tokens_reports_a_bad_slot():
    from cuda_b200 import _lib as L
    n, h, d, page, nb = 2048, 2, 128, 16, 130
    k = torch.randn(n, h, d, device="cuda", dtype=torch.bfloat16)
    t = torch.arange(n)
    blk, off = (t // page).to(torch.int32), (t % page).to(torch.int32)
    blk[16 * 7 + 3] = nb + 5                                    # one token of one group points outside the pool
    kc = torch.zeros(nb, h, d, page, dtype=torch.uint8, device="cuda"); vc = torch.zeros_like(kc)
    ks = torch.zeros(nb, h, page, device="cuda"); vs = torch.zeros_like(ks)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    blk_d, off_d = blk.cuda(), off.cuda()
    L.check(L.load().cuda_llm_kv_append(k.data_ptr(), k.data_ptr(), blk_d.data_ptr(), off_d.data_ptr(), kc.data_ptr(),
                                        vc.data_ptr(), ks.data_ptr(), vs.data_ptr(), n, h, d, page, nb, L.BF16,
                                        L.KV_FP8_E4M3, L.SCALE_PER_TOKEN, status.data_ptr(), None), "kv_append")
    torch.cuda.synchronize()
    assert status.item() & L.ST_BAD_BLOCK
    # the other 15 tokens of that group and every other group were written
    written = (ks.cpu() != 0).permute(0, 2, 1)[..., 0]          # [nb, page]
    assert written[:n // page].sum().item() == n - 1


def test_append_then_decode_round_trip():
    """Fill a cache token by token with the append kernel, then attend over it: same result as the
    oracle on the host-quantised cache."""
    from cuda_b200 import ops, workloads as W
    from helpers import assert_parity, oracle_out
    wl = W.build_workload("rt", context_lens=[45, 130], q_lens=None, num_q_heads=8, num_kv_heads=2, head_dim=128,
                          page_size=16, q_dtype=torch.bfloat16, scale_mode="per_token", pool_factor=1.0, seed=8,
                          poison=False)
    torch.manual_seed(9)
    g = wl.to("cuda")
    kc, vc = torch.zeros_like(g.key_cache), torch.zeros_like(g.value_cache)
    ks, vs = torch.ones_like(g.k_scale), torch.ones_like(g.v_scale)
    import dataclasses
    ref_wl = dataclasses.replace(wl, key_cache=wl.key_cache.clone(), value_cache=wl.value_cache.clone(),
                                 k_scale=wl.k_scale.clone(), v_scale=wl.v_scale.clone())
    for s, ctx in enumerate([45, 130]):
        k = torch.randn(ctx, 2, 128)
        v = torch.randn(ctx, 2, 128)
        pos = torch.arange(ctx)
        blk = wl.block_tables[s, pos // 16]
        off = (pos % 16).to(torch.int32)
        ops.kv_cache_append(k.cuda(), v.cuda(), blk.cuda(), off.cuda(), kc, vc, ks, vs)
        kq, ksc = O.quantize_tokens(k, "fp8_e4m3", "per_token")
        vq, vsc = O.quantize_tokens(v, "fp8_e4m3", "per_token")
        ref_wl.key_cache[blk.long(), :, :, off.long()] = kq
        ref_wl.value_cache[blk.long(), :, :, off.long()] = vq
        ref_wl.k_scale[blk.long(), :, off.long()] = ksc
        ref_wl.v_scale[blk.long(), :, off.long()] = vsc
    out = ops.fp8_paged_attention_forward(g.query, kc, vc, ks, vs, g.block_tables, g.context_lens, check_status=True)
    assert_parity(out, oracle_out(ref_wl), torch.bfloat16, "append + decode")
