"""Seeded random shapes through every kernel family against the CPU oracle: sequence counts, head counts, GQA
groups, head sizes, page sizes, formats, query lengths, CTA counts and slot patterns that the hand-picked cases
of the other files do not combine.  Tolerances are those of the files that own each path."""
import random

import pytest
import torch

from helpers import TOL_MAX_ABS, TOL_MEAN_ABS, oracle_out
from oracle import paged_decode_oracle as O
import test_paged_f32_gpu as F32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_quantised_decode(ops, seed):
    """FP8 / MXFP8 / MXFP4 caches, both decode kernels, split merge with 1 to 148 CTAs, multi-token queries.
    (Seed 2 holds the launch that exposed a lost wake-up in the tcgen05 kernel: 36 sequences, most of them shorter
    than a tile, one head pair, E8M0 scales, 7 CTAs.)"""
    from cuda_b200 import workloads as W
    rnd = random.Random(seed)
    for it in range(16):
        S = rnd.randint(1, 40); hkv = rnd.choice([1, 2, 4, 8]); group = rnd.choice([1, 2, 4, 8]); d = rnd.choice([64, 128, 128])
        page = rnd.choice([16, 16, 32, 64])
        mode, vfmt = rnd.choice([("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"), ("mx_e8m0", "fp4_e2m1"), ("per_head", "fp8_e4m3")])
        lens = [rnd.choice([rnd.randint(1, 64), rnd.randint(1, 900), rnd.randint(1, 6000)]) for _ in range(S)]
        qls = [min(rnd.randint(1, min(max(1, 16 // group), 4)), l) for l in lens] if rnd.random() < 0.6 else None
        dt = rnd.choice([torch.bfloat16, torch.float16])
        wl = W.build_workload("rnd", context_lens=lens, q_lens=qls, num_q_heads=hkv * group, num_kv_heads=hkv, head_dim=d,
                              page_size=page, q_dtype=dt, v_format=vfmt, scale_mode=mode, pool_factor=1.2, seed=100 * seed + it)
        ref = oracle_out(wl)
        nc = rnd.choice([0, 0, 1, 7, 37, 148])
        flags = ops.L.FLAG_TCGEN05 if rnd.random() < 0.4 else 0
        what = (S, hkv, group, d, page, mode, vfmt, qls is not None, nc, flags)
        try:
            out = ops.run_workload(wl.to("cuda"), check_status=True, num_ctas=nc, flags=flags)
        except RuntimeError as e:
            raise AssertionError(f"case {it} {what} lens {lens[:8]} q_lens {None if qls is None else qls[:8]}: {e}")
        err = (out.float().cpu() - ref.float()).abs()
        assert torch.isfinite(out).all(), what
        assert err.max().item() <= TOL_MAX_ABS[dt] and err.mean().item() <= TOL_MEAN_ABS[dt], (what, err.max().item())


@pytest.mark.parametrize("seed", [1, 2])
def test_fp32_decode(ops, seed):
    """fp32 paged caches (pages of 16 / 32 / 64 tokens, NaN behind every sequence) and contiguous fp32 K/V."""
    rnd = random.Random(seed)
    for it in range(20):
        S = rnd.randint(1, 24); hkv = rnd.choice([1, 2, 3, 4, 8]); group = rnd.randint(1, 8); d = rnd.choice([64, 128])
        page = rnd.choice([16, 16, 32, 64])
        lens = [rnd.choice([0, 1, rnd.randint(1, 64), rnd.randint(1, 700), rnd.randint(1, 5000)]) for _ in range(S)]
        wl = F32._workload(lens, hkv, group, d, seed=100 * seed + it, page=page)
        g = wl.to("cuda")
        out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
        F32._check(out, F32._oracle(wl), f"paged {S} {hkv} {group} {d} {page}")
        s_len = rnd.choice([1, 15, 16, 17, rnd.randint(1, 3000)])
        q, k, v, ref = F32._flash_case(rnd.randint(1, 4), hkv, group, s_len, d, seed=it)
        F32._check(ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda()), ref, f"contiguous {hkv} {group} {s_len} {d}")


@pytest.mark.parametrize("seed", [1, 2])
def test_prefill(ops, seed):
    """GQA prefill on the tcgen05 kernel: every group size 1-16, ragged lengths, causal or not."""
    rnd = random.Random(seed)
    for it in range(12):
        b = rnd.randint(1, 3); hkv = rnd.choice([1, 2, 4]); group = rnd.choice([1, 2, 3, 4, 5, 6, 7, 8, 12, 16]); d = rnd.choice([64, 128])
        s = rnd.choice([1, 17, 128, 129, rnd.randint(1, 900)])
        causal = rnd.random() < 0.7
        dt = rnd.choice([torch.bfloat16, torch.float16])
        g = torch.Generator().manual_seed(100 * seed + it)
        q = torch.randn(b, hkv * group, s, d, generator=g).to(dt)
        k = torch.randn(b, hkv, s, d, generator=g).to(dt)
        v = torch.randn(b, hkv, s, d, generator=g).to(dt)
        out = ops.fused_gqa_forward(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
        tol = 2e-2 if dt == torch.float16 else 4e-2           # the reference's own table (tests/_utils.py:23-27)
        assert torch.allclose(out.float().cpu(), O.ref_gqa(q, k, v, causal), atol=tol, rtol=tol), (b, hkv, group, d, s, causal, dt)


@pytest.mark.parametrize("seed", [1, 2])
def test_cache_append(ops, seed):
    """The append kernel for many tokens on slot lists made of runs of 1 to 333 consecutive slots that start
    aligned or inside a page: full-width rows and byte stores mixed in one call, bit for bit."""
    rnd = random.Random(seed)
    for it in range(8):
        mode = rnd.choice(["per_token", "mx_e8m0", "per_head"])
        vfmt = "fp4_e2m1" if (mode == "mx_e8m0" and rnd.random() < 0.5) else "fp8_e4m3"
        d = rnd.choice([64, 128]); page = rnd.choice([16, 32, 64]); h = rnd.choice([1, 2, 4])
        dtype = rnd.choice([torch.float32, torch.float16, torch.bfloat16])
        n = rnd.randint(1024, 2600)
        nb = n // page + 40
        free = list(range(nb)); rnd.shuffle(free)
        blk, off = [], []
        while len(blk) < n:
            run = rnd.choice([1, 3, 16, 16, 32, 48, 100, 333])
            p_i, o = free.pop(), rnd.choice([0, 0, 0, rnd.randint(0, page - 1)])
            for _ in range(run):
                if len(blk) >= n:
                    break
                if o >= page:
                    p_i, o = free.pop(), 0
                blk.append(p_i); off.append(o); o += 1
        blk_t, off_t = torch.tensor(blk), torch.tensor(off)
        k = (torch.randn(n, h, d) * torch.exp2(torch.randint(-10, 5, (n, h, 1)).float())).to(dtype)
        v = torch.randn(n, h, d).to(dtype)
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
            ks, vs = k_head.cuda(), v_head.cuda()
        ops.kv_cache_append(k.cuda(), v.cuda(), blk_t.int().cuda(), off_t.int().cuda(), kc, vc, ks, vs)
        torch.cuda.synchronize()
        what = (mode, vfmt, d, page, dtype, h, n)
        assert torch.equal(kc.cpu()[blk_t, :, :, off_t], kc_ref) and torch.equal(vc.cpu()[blk_t, :, :, off_t], vc_ref), what
        if mode == "per_token":
            assert torch.equal(ks.cpu()[blk_t, :, off_t], ks_ref) and torch.equal(vs.cpu()[blk_t, :, off_t], vs_ref), what
        if mode == "mx_e8m0":
            assert torch.equal(ks.cpu()[blk_t, :, :, off_t], ks_ref) and torch.equal(vs.cpu()[blk_t, :, :, off_t], vs_ref), what
        untouched = torch.ones(nb, page, dtype=torch.bool)
        untouched[blk_t, off_t] = False
        assert (kc.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all() and (vc.cpu().permute(0, 3, 1, 2)[untouched] == 0xAA).all(), what
