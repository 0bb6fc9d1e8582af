"""The oracle is pinned against outputs of the reference's own specification functions
(fixtures made by ``tests/golden/make_golden.py``)."""
import zlib

import numpy as np
import pytest
import torch

import cases
from oracle import paged_decode_oracle as O


def crc(t):
    return zlib.crc32(t.contiguous().view(torch.uint8).numpy().tobytes())


def _paged_kv(kc, vc, bt, lens, head_dim, fmt, mode, ks=None, vs=None):
    return O.PagedKV(key_cache=kc, value_cache=vc, block_tables=bt, context_lens=lens,
                     page_size=cases.PAGE, head_dim=head_dim, k_format=fmt, v_format=fmt,
                     k_scale_mode=mode, v_scale_mode=mode, k_scale=ks, v_scale=vs)


@pytest.mark.parametrize("case", list(cases.paged_cases()), ids=lambda c: c[0])
def test_paged_matches_reference(golden, case):
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v, cases.PAGE, perm)
    # inputs and the page layout are bit-identical to what the reference built
    assert [crc(q), crc(kc), crc(vc)] == golden[f"{name}/crc"].tolist()
    kv = _paged_kv(kc, vc, bt, lens_t, hd, O.KV_F32, O.SCALE_NONE)
    ref = torch.from_numpy(golden[f"{name}/out"])
    out_sdpa = O.ref_paged_decode_sdpa(q, kv)
    assert torch.equal(out_sdpa, ref) or (out_sdpa - ref).abs().max() < 2e-6
    out = O.ref_paged_decode(q, kv)
    assert (out - ref).abs().max() < 1e-5


@pytest.mark.parametrize("case", list(cases.fp8_cases()), ids=lambda c: c[0])
def test_fp8_matches_reference(golden, case):
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    k8, v8, ks, vs, k_deq, v_deq = cases.fp8_quantise(k, v)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k8, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v8, cases.PAGE, perm)
    assert [crc(q), crc(kc), crc(vc), crc(ks), crc(vs)] == golden[f"{name}/crc"].tolist()
    # E4M3 table (built from the format definition) == torch's cast on every finite code
    kv = _paged_kv(kc, vc, bt, lens_t, hd, O.KV_FP8_E4M3, O.SCALE_PER_HEAD, ks, vs)
    for s, L in enumerate(lens):
        kk, vv = O.gather_sequence(kv, s)
        assert torch.equal(kk, k_deq[s, :, :L])       # dequant + block-table gather: bit-exact
        assert torch.equal(vv, v_deq[s, :, :L])
    ref = torch.from_numpy(golden[f"{name}/out"])
    out = O.ref_paged_decode(q, kv)
    assert (out - ref).abs().max() < 1e-5
    out_sdpa = O.ref_paged_decode_sdpa(q, kv)
    assert (out_sdpa - ref).abs().max() < 2e-6


@pytest.mark.parametrize("case", list(cases.decode_cases()), ids=lambda c: c[0])
def test_decode_matches_reference(golden, case):
    name, dtype, hd, kv_len = case
    q, k, v = cases.decode_inputs(dtype, hd, kv_len)
    assert [crc(q), crc(k), crc(v)] == golden[f"{name}/crc"].tolist()
    ref = torch.from_numpy(golden[f"{name}/out"])
    assert (O.ref_flash_decode(q, k, v) - ref).abs().max() < 2e-6


def test_gqa_convention(golden):
    torch.manual_seed(0)
    q = torch.randn(2, 8, 1, 64)
    k = torch.randn(2, 2, 77, 64)
    v = torch.randn(2, 2, 77, 64)
    assert [crc(q), crc(k), crc(v)] == golden["gqa_decode/crc"].tolist()
    ref = torch.from_numpy(golden["gqa_decode/out"])            # [2,8,1,64]
    # page the GQA case and run the oracle: kv_head = q_head // group
    perm = torch.randperm(2 * 5)
    kc = O.paged_layout_from_dense(k, 16, perm)
    vc = O.paged_layout_from_dense(v, 16, perm)
    kv = O.PagedKV(kc, vc, perm.view(2, 5).to(torch.int32), torch.tensor([77, 77], dtype=torch.int32),
                   16, 64, O.KV_F32, O.KV_F32, O.SCALE_NONE, O.SCALE_NONE)
    out = O.ref_paged_decode(q[:, :, 0], kv)
    assert (out - ref[:, :, 0]).abs().max() < 1e-5
    assert (O.ref_paged_decode_sdpa(q[:, :, 0], kv) - ref[:, :, 0]).abs().max() < 2e-6


def test_code_tables_match_torch():
    codes = torch.arange(256, dtype=torch.uint8)
    t = codes.view(torch.float8_e4m3fn).float()
    mine = torch.from_numpy(O.E4M3_TABLE)
    fin = torch.isfinite(t)
    assert torch.equal(mine[fin], t[fin]) and torch.isnan(mine[~fin]).all() and (~fin).sum() == 2
    e = codes.view(torch.float8_e8m0fnu).float()
    mine = torch.from_numpy(O.E8M0_TABLE)
    assert torch.equal(mine[:255], e[:255]) and torch.isnan(mine[255])
    import ml_dtypes
    f4 = np.arange(16, dtype=np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32)
    assert np.array_equal(O.E2M1_TABLE, f4)


def test_split_merge_equals_full():
    from cuda_b200 import workloads as W
    wl = W.build_workload("t", context_lens=[1, 37, 200, 0, 64], q_lens=[1, 4, 1, 1, 4],
                          num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=16,
                          q_dtype=torch.float32, scale_mode=W.SCALE_PER_TOKEN, pool_factor=1.5, seed=3)
    kv = to_oracle(wl)
    full, lse = O.ref_paged_decode(wl.query, kv, wl.softmax_scale, wl.cu_q_lens, return_lse=True)
    assert torch.isfinite(full).all()
    parts = [O.ref_paged_decode(wl.query, kv, wl.softmax_scale, wl.cu_q_lens, tok_range=r, return_lse=True)
             for r in ((0, 48), (48, 50), (50, 130), (130, 4096))]
    o, l = O.merge_partials(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert (o - full).abs().max() < 1e-5
    fin = torch.isfinite(lse)
    assert (l[fin] - lse[fin]).abs().max() < 1e-5 and torch.equal(torch.isfinite(l), fin)


def to_oracle(wl):
    return O.PagedKV(wl.key_cache, wl.value_cache, wl.block_tables, wl.context_lens, wl.page_size,
                     wl.head_dim, wl.k_format, wl.v_format, wl.k_scale_mode, wl.v_scale_mode,
                     wl.k_scale, wl.v_scale)


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_configs_small_are_finite_and_causal(cfg):
    from cuda_b200 import workloads as W
    wl = W.make_config(cfg, batch=3, ctx_scale=1 / 32)
    kv = to_oracle(wl)
    out = O.ref_paged_decode(wl.query, kv, wl.softmax_scale, wl.cu_q_lens)
    assert torch.isfinite(out).all()        # poisoned tails / unused pages are never read
    assert out.shape == wl.query.shape


@pytest.mark.parametrize("case", list(cases.rope_cases()), ids=lambda c: c[0])
def test_rope_oracle_matches_reference(golden, case):
    """rope_tables / apply_rope of the oracle reproduce the reference's (tests/_utils.py:75-88 there)
    bit for bit, and rotating only the last query row and attending over the rotated keys gives the
    last row of the reference's causal ref_rope_attention."""
    import zlib
    name, dtype, hd, seq = case
    q, k, v = cases.rope_inputs(dtype, hd, seq)
    cos, sin = O.rope_tables(seq, hd)
    crc = lambda t: zlib.crc32(t.contiguous().view(torch.uint8).numpy().tobytes())
    want = golden[f"{name}/crc"]
    k_rot = O.apply_rope(k, cos, sin).to(dtype)
    assert [crc(q), crc(k), crc(v), crc(cos), crc(sin), crc(k_rot)] == want.tolist()
    ctx = torch.full((2,), seq, dtype=torch.int32)
    q_last = q[:, :, -1, :]                                                     # [B, H, D]
    q_rot = O.rope_query(q_last, cos, sin, ctx)
    out = O.ref_flash_decode(q_rot[:, :, None, :], O.apply_rope(k, cos, sin), v)[:, :, 0]
    assert torch.allclose(out, torch.from_numpy(golden[f"{name}/out_last"]), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("case", list(cases.gqa_cases()), ids=lambda c: c[0])
def test_gqa_oracle_matches_reference(golden, case):
    """ref_gqa of the oracle reproduces the reference's ref_gqa on its own test grid: same inputs (CRC),
    the whole output tensor bit for bit (CRC) and the sampled rows the fixture keeps."""
    import zlib
    name, dtype, hd, hq, hkv, causal = case
    q, k, v = cases.gqa_inputs(dtype, hd, hq, hkv)
    o = O.ref_gqa(q, k, v, is_causal=causal)
    crc = lambda t: zlib.crc32(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert [crc(q), crc(k), crc(v), crc(o)] == golden[f"{name}/crc"].tolist()
    assert torch.equal(o[:, :, list(cases.GQA_ROWS), :], torch.from_numpy(golden[f"{name}/rows"]))


def test_quantisers_pinned_to_library_casts():
    """The workload generator's quantisers (the write side of the cache formats) agree bit for bit
    with the oracle's statement of the recipe, which uses torch's float8_e4m3fn cast and ml_dtypes'
    float4_e2m1fn cast: every rounding tie of E2M1, saturation, and random data in all scale modes."""
    import ml_dtypes
    from cuda_b200 import workloads as W
    ties = torch.tensor([0.0, 0.2, 0.25, 0.26, 0.74, 0.75, 0.76, 1.25, 1.26, 1.75, 2.5, 2.51, 3.5, 5.0, 5.01, 6.0,
                         7.0, 7.99, 100.0])
    x = torch.cat([ties, -ties, torch.randn(4096) * 2])
    want = torch.from_numpy(x.numpy().astype(ml_dtypes.float4_e2m1fn).view(np.uint8))
    assert torch.equal(W.quant_e2m1(x), want)
    g = torch.Generator().manual_seed(3)
    t = torch.randn(37, 3, 128, generator=g) * torch.exp(2 * torch.randn(37, 3, 1, generator=g))
    for fmt, mode in (("fp8_e4m3", "per_token"), ("fp8_e4m3", "mx_e8m0"), ("fp4_e2m1", "mx_e8m0")):
        a, sa = W.quantize_tokens(t, fmt, mode)
        b, sb = O.quantize_tokens(t, fmt, mode)
        assert torch.equal(a, b) and torch.equal(sa, sb), (fmt, mode)
    hs = torch.rand(3, generator=g) + 0.5
    a, _ = W.quantize_tokens(t, "fp8_e4m3", "per_head", hs)
    b, _ = O.quantize_tokens(t, "fp8_e4m3", "per_head", hs)
    assert torch.equal(a, b)
