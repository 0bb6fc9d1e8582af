"""Parity of the CUDA paged decode path (through the C ABI) against the CPU oracle."""
import pytest
import torch

import cases
from helpers import assert_parity, oracle_out, to_oracle
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _W():
    from cuda_b200 import workloads
    return workloads


# ------------------------------------------------------------------------------------------
# dequantisation and block-table gather: bit-exact
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode,vfmt", [("per_head", "fp8_e4m3"), ("per_block", "fp8_e4m3"),
                                       ("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"),
                                       ("mx_e8m0", "fp4_e2m1")])
def test_dequant_bit_exact(ops, mode, vfmt):
    W = _W()
    wl = W.build_workload("dq", context_lens=[70, 33, 128], q_lens=None, num_q_heads=8, num_kv_heads=4,
                          head_dim=128, page_size=16, q_dtype=torch.bfloat16, v_format=vfmt,
                          scale_mode=mode, pool_factor=1.5, seed=11, poison=False,
                          mx_exponent_range=(-20, 12) if vfmt == "fp8_e4m3" else None)
    kv = to_oracle(wl)
    g = wl.to("cuda")
    for s in range(3):
        n = (int(wl.context_lens[s]) + 15) // 16
        pages = wl.block_tables[s, :n]
        for cache, scale, fmt, smode, ocache in (
                (g.key_cache, g.k_scale, "fp8_e4m3", mode, kv.key_cache),
                (g.value_cache, g.v_scale, vfmt, mode, kv.value_cache)):
            got = ops.dequant_pages(cache, scale, pages.cuda(), 128, ops._FMT[fmt], ops._MODE[smode]).cpu()
            sc = kv.k_scale if cache is g.key_cache else kv.v_scale
            ref = O._dequant_pages(ocache, fmt, smode, sc, pages.long(), 128)   # [H, n*page, D]
            ref = ref.view(4, n, 16, 128).permute(1, 0, 3, 2)
            assert torch.equal(got, ref)


def test_dequant_all_codes(ops):
    """Every E4M3 byte and every E8M0 byte decodes exactly as the format tables say."""
    codes = torch.arange(256, dtype=torch.uint8).repeat(8).view(1, 1, 128, 16).cuda()
    one = torch.ones(1, dtype=torch.float32).cuda()
    got = ops.dequant_pages(codes, one, torch.zeros(1, dtype=torch.int32).cuda(), 128,
                            ops.L.KV_FP8_E4M3, ops.L.SCALE_PER_HEAD).cpu().view(-1)
    ref = torch.from_numpy(O.E4M3_TABLE)[codes.cpu().view(-1).long()]
    fin = torch.isfinite(ref)
    assert torch.equal(got[fin], ref[fin]) and torch.isnan(got[~fin]).all()
    # E8M0: payload 1.0 (0x38) times every scale byte
    payload = torch.full((1, 1, 128, 16), 0x38, dtype=torch.uint8).cuda()
    sc = torch.arange(256, dtype=torch.uint8)[:64].view(1, 1, 4, 16)
    for base in range(0, 256, 64):
        s = (sc + base).to(torch.uint8).cuda()
        got = ops.dequant_pages(payload, s, torch.zeros(1, dtype=torch.int32).cuda(), 128,
                                ops.L.KV_FP8_E4M3, ops.L.SCALE_MX_E8M0).cpu()
        ref = torch.from_numpy(O.E8M0_TABLE)[(sc + base).long()].repeat_interleave(32, dim=2)
        fin = torch.isfinite(ref)
        assert torch.equal(got[fin], ref[fin]) and torch.isnan(got[~fin]).all()


# ------------------------------------------------------------------------------------------
# the reference's own E4M3 cases, against the golden outputs of the reference's ref_decode
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", list(cases.fp8_cases()), ids=lambda c: c[0])
def test_reference_fp8_cases(ops, golden, case):
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    k8, v8, ks, vs, _, _ = cases.fp8_quantise(k, v)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k8, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v8, cases.PAGE, perm)
    out = ops.fp8_paged_attention_forward(q.cuda(), kc.cuda(), vc.cuda(), ks.cuda(), vs.cuda(),
                                          bt.cuda(), lens_t.cuda(), check_status=True)
    ref = torch.from_numpy(golden[f"{name}/out"])
    # the reference's tolerance table (tests/_utils.py:23-27)
    atol, rtol = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2)}[dtype]
    assert out.dtype == dtype and torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=atol, rtol=rtol)
    assert_parity(out, ref, dtype, name)


# ------------------------------------------------------------------------------------------
# the five configurations, shrunk
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg,batch,ctx_scale", [(1, 4, 1.0), (2, 6, 1 / 8), (3, 5, 1 / 16),
                                                 (4, 2, 1 / 64), (5, 24, 1 / 8)])
def test_configs_small(ops, cfg, batch, ctx_scale):
    W = _W()
    wl = W.make_config(cfg, batch=batch, ctx_scale=ctx_scale)
    ref, ref_lse = oracle_out(wl, return_lse=True)
    out, lse = ops.run_workload(wl.to("cuda"), return_lse=True, check_status=True)
    assert_parity(out, ref, wl.query.dtype, wl.name)
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("page", [16, 32, 64])
@pytest.mark.parametrize("hkv,group", [(1, 1), (1, 8), (2, 4), (4, 1), (8, 4), (16, 2), (3, 1)])
@pytest.mark.parametrize("mode,vfmt", [("per_token", "fp8_e4m3"), ("mx_e8m0", "fp8_e4m3"),
                                       ("mx_e8m0", "fp4_e2m1"), ("per_head", "fp8_e4m3")])
def test_head_and_page_shapes(ops, page, hkv, group, mode, vfmt):
    W = _W()
    d = 128 if hkv != 4 else 64
    wl = W.build_workload("shapes", context_lens=[1, page, page + 1, 5 * page + 3, 0, 300], q_lens=None,
                          num_q_heads=hkv * group, num_kv_heads=hkv, head_dim=d, page_size=page,
                          q_dtype=torch.bfloat16, v_format=vfmt, scale_mode=mode, pool_factor=1.3,
                          seed=page + hkv + group)
    ref = oracle_out(wl)
    out = ops.run_workload(wl.to("cuda"), check_status=True)
    assert_parity(out, ref, torch.bfloat16, f"p{page} hkv{hkv} g{group} {mode} {vfmt}")
    assert (out[4] == 0).all()          # empty context -> zeros


@pytest.mark.parametrize("page", [16, 32, 64])
def test_every_context_length(ops, page):
    """ctx = 1 .. 3*page+1: every page-tail length, GQA group 4."""
    W = _W()
    lens = list(range(1, 3 * page + 2))
    wl = W.build_workload("lens", context_lens=lens, q_lens=None, num_q_heads=8, num_kv_heads=2,
                          head_dim=64, page_size=page, q_dtype=torch.float16,
                          scale_mode="per_token", pool_factor=1.25, seed=5)
    ref = oracle_out(wl)
    out = ops.run_workload(wl.to("cuda"), check_status=True)
    assert_parity(out, ref, torch.float16, f"lens page {page}")


@pytest.mark.parametrize("mode,vfmt", [("per_token", "fp8_e4m3"), ("mx_e8m0", "fp4_e2m1")])
@pytest.mark.parametrize("group", [1, 4])
def test_q_len_causal(ops, mode, vfmt, group):
    """q_len in {1..4}: bottom-right aligned causal mask inside the verify window."""
    W = _W()
    lens = [4, 5, 16, 17, 35, 64, 100, 3, 250]
    qls = [4, 1, 2, 4, 3, 4, 1, 3, 4]
    wl = W.build_workload("qlen", context_lens=lens, q_lens=qls, num_q_heads=2 * group, num_kv_heads=2,
                          head_dim=128, page_size=16, q_dtype=torch.bfloat16, v_format=vfmt,
                          scale_mode=mode, pool_factor=1.5, seed=9)
    ref, ref_lse = oracle_out(wl, return_lse=True)
    out, lse = ops.run_workload(wl.to("cuda"), return_lse=True, check_status=True)
    assert_parity(out, ref, torch.bfloat16, "q_len causal")
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("num_ctas", [1, 2, 3, 7, 33, 148])
@pytest.mark.parametrize("seed", [21, 22])
def test_mixed_rows_partition(ops, num_ctas, seed):
    """A batch that mixes 4-row and 16-row queries: units of the 16-row sequences weigh twice in
    the partition, cuts fall inside them, and every CTA count must give the same answer."""
    W = _W()
    g = torch.Generator().manual_seed(seed)
    n = 14
    lens = torch.randint(1, 700, (n,), generator=g).tolist()
    qls = [4 if x else 1 for x in (torch.rand(n, generator=g) < 0.4).tolist()]
    wl = W.build_workload("mixed", context_lens=lens, q_lens=qls, num_q_heads=8, num_kv_heads=2,
                          head_dim=128, page_size=16, q_dtype=torch.bfloat16, v_format="fp4_e2m1",
                          scale_mode="mx_e8m0", pool_factor=1.4, seed=seed)
    ref = oracle_out(wl)
    out = ops.run_workload(wl.to("cuda"), num_ctas=num_ctas, check_status=True)
    assert_parity(out, ref, torch.bfloat16, f"mixed rows, {num_ctas} CTAs")


def test_query_longer_than_declared_still_fits_the_rows(ops):
    """max_q_len sizes the shared-memory query area; a sequence with more query tokens than declared
    that still fits the 8 rows of the kernel must take the global-memory path, not overrun the area."""
    W = _W()
    wl = W.build_workload("qlen2", context_lens=[300, 40, 1000, 17], q_lens=[2, 1, 2, 2], num_q_heads=8,
                          num_kv_heads=2, head_dim=128, page_size=16, q_dtype=torch.bfloat16,
                          scale_mode="per_token", pool_factor=1.3, seed=31)
    ref = oracle_out(wl)
    g = wl.to("cuda")
    out = ops.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale, g.block_tables,
                                          g.context_lens, g.softmax_scale, cu_q_lens=g.cu_q_lens, max_q_len=1,
                                          check_status=True)
    assert_parity(out, ref, torch.bfloat16, "q_len 2 with max_q_len 1")


def test_stable_metadata_flag_back_to_back(ops):
    """With CUDA_LLM_FLAG_STABLE_METADATA the kernel plans before the previous kernel on the stream
    has finished; calls issued back to back on two workloads must still be exact copies of the
    results without the flag."""
    W = _W()
    a = W.make_config(2, "cuda", batch=8, ctx_scale=1 / 8, seed=41)
    b = W.make_config(3, "cuda", batch=6, ctx_scale=1 / 16, seed=42)
    ref_a, ref_b = ops.run_workload(a), ops.run_workload(b)
    outs = []
    for i in range(12):
        wl = a if i % 2 == 0 else b
        outs.append(ops.run_workload(wl, flags=ops.L.FLAG_STABLE_METADATA, out=torch.empty_like(wl.query)))
    torch.cuda.synchronize()
    for i, o in enumerate(outs):
        assert torch.equal(o, ref_a if i % 2 == 0 else ref_b), f"call {i}"
    assert ops.decode_status(ops.get_workspace(torch.device("cuda", torch.cuda.current_device()), 1)) == 0


def test_fp32_query_is_tight(ops):
    """fp32 Q/out (the reference's <float,float> instantiation) uses split operands."""
    W = _W()
    wl = W.make_config(1)
    ref = oracle_out(wl)
    out = ops.run_workload(wl.to("cuda"), check_status=True)
    assert out.dtype == torch.float32
    assert (out.cpu() - ref).abs().max() < 2e-4


def test_split_invariance_and_merge(ops):
    """The result does not depend on how many CTAs the units are cut into."""
    W = _W()
    wl = W.make_config(2, batch=5, ctx_scale=1 / 4).to("cuda")
    ref = oracle_out(wl)
    outs = []
    for n in (1, 3, 37, 148, 500):
        ws = torch.zeros(ops.L.load().cuda_llm_paged_decode_workspace_bytes(5, 32, 8, 128, 16, 1, n),
                         dtype=torch.uint8, device="cuda")
        outs.append(ops.run_workload(wl, num_ctas=n, workspace=ws, check_status=True))
        assert_parity(outs[-1], ref, torch.bfloat16, f"{n} CTAs")
    for o in outs[1:]:
        assert (o.float() - outs[0].float()).abs().max() <= 2e-2


@pytest.mark.parametrize("P,rows,d", [(5, 37, 128), (64, 9, 64), (65, 9, 128), (300, 6, 64), (513, 3, 128)])
def test_merge_partials_matches_oracle(ops, P, rows, d):
    """Few parts (a warp per row) and many (a block of 16 warps per row, warp w taking parts w, w + 16, ...)."""
    torch.manual_seed(1)
    o = torch.randn(P, rows, d)
    l = torch.randn(P, rows) * 3
    l[2, :5] = float("-inf")
    l[:, rows - 1] = float("-inf")
    ro, rl = O.merge_partials(o, l)
    go, gl = ops.merge_partials(o.cuda(), l.cuda(), return_lse=True)
    assert (go.cpu() - ro).abs().max() < 1e-5
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(gl.cpu()), fin) and (gl.cpu()[fin] - rl[fin]).abs().max() < 1e-5
    assert (go.cpu()[rows - 1] == 0).all()


def test_bad_block_index_is_reported_not_faulted(ops):
    W = _W()
    wl = W.build_workload("bad", context_lens=[40, 40], q_lens=None, num_q_heads=8, num_kv_heads=8,
                          head_dim=64, page_size=16, q_dtype=torch.float16, scale_mode="per_token", seed=2)
    wl.block_tables[1, 1] = 10_000                 # outside the pool
    g = wl.to("cuda")
    ws = torch.zeros(16 << 20, dtype=torch.uint8, device="cuda")
    ops.run_workload(g, workspace=ws)
    st = ops.decode_status(ws)
    assert st & ops.L.ST_BAD_BLOCK
    assert ops.decode_status(ws) == 0              # cleared by the read


def test_reference_error_messages(ops):
    q = torch.zeros(2, 4, 64, device="cuda", dtype=torch.float16)
    c = torch.zeros(4, 4, 64, 16, device="cuda", dtype=torch.uint8)
    s = torch.ones(4, device="cuda")
    bt = torch.zeros(2, 2, device="cuda", dtype=torch.int32)
    cl = torch.ones(2, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError, match="Inputs must be on CUDA"):
        ops.fp8_paged_attention_forward(q.cpu(), c, c, s, s, bt, cl)
    with pytest.raises(RuntimeError, match="Query must be 3D"):
        ops.fp8_paged_attention_forward(q[0], c, c, s, s, bt, cl)
    with pytest.raises(RuntimeError, match="8-bit quantized"):
        ops.fp8_paged_attention_forward(q, c.half(), c.half(), s, s, bt, cl)
    with pytest.raises(RuntimeError, match="Only head_dim 64 and 128 supported"):
        ops.fp8_paged_attention_forward(torch.zeros(2, 4, 32, device="cuda", dtype=torch.float16),
                                        c[:, :, :32], c[:, :, :32], s, s, bt, cl)


# ------------------------------------------------------------------------------------------
# unquantised entry points: the reference's own cases against its golden outputs
# ------------------------------------------------------------------------------------------
REF_TOL = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2), torch.float32: (1e-4, 1e-4)}


@pytest.mark.parametrize("case", list(cases.paged_cases()), ids=lambda c: c[0])
def test_reference_paged_cases(ops, golden, case):
    name, dtype, hd, lens = case
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k, cases.PAGE, perm)
    vc = O.paged_layout_from_dense(v, cases.PAGE, perm)
    out = ops.paged_attention_forward(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), lens_t.cuda())
    ref = torch.from_numpy(golden[f"{name}/out"])
    atol, rtol = REF_TOL[dtype]
    assert out.dtype == dtype and torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=atol, rtol=rtol)


@pytest.mark.parametrize("case", list(cases.decode_cases()), ids=lambda c: c[0])
def test_reference_decode_cases(ops, golden, case):
    name, dtype, hd, kv_len = case
    q, k, v = cases.decode_inputs(dtype, hd, kv_len)
    out = ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
    ref = torch.from_numpy(golden[f"{name}/out"])
    atol, rtol = REF_TOL[dtype]
    assert out.shape == q.shape and torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=atol, rtol=rtol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("hkv,group,page", [(2, 4, 16), (8, 1, 32), (1, 8, 64)])
def test_paged_attention_gqa_long(ops, dtype, hkv, group, page):
    """GQA, page sizes 32/64, several splits, an empty sequence."""
    W = _W()
    wl = W.build_workload("pa", context_lens=[1000, 0, 37, 2049], q_lens=None, num_q_heads=hkv * group,
                          num_kv_heads=hkv, head_dim=128, page_size=page, q_dtype=dtype, scale_mode="none",
                          pool_factor=1.2, seed=3, cache_dtype=dtype)
    kv = O.PagedKV(wl.key_cache, wl.value_cache, wl.block_tables, wl.context_lens, page, 128,
                   O.KV_F32, O.KV_F32, O.SCALE_NONE, O.SCALE_NONE)
    ref = O.ref_paged_decode(wl.query, kv, wl.softmax_scale)
    g = wl.to("cuda")
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    atol, rtol = REF_TOL[dtype]
    assert torch.allclose(out.float().cpu(), ref, atol=atol, rtol=rtol)
    assert (out[1] == 0).all()


def test_flash_decode_gqa(ops):
    torch.manual_seed(4)
    q = torch.randn(3, 8, 1, 128, dtype=torch.bfloat16)
    k = torch.randn(3, 2, 777, 128, dtype=torch.bfloat16)
    v = torch.randn(3, 2, 777, 128, dtype=torch.bfloat16)
    ref = O.ref_flash_decode(q, k.repeat_interleave(4, dim=1), v.repeat_interleave(4, dim=1))
    out = ops.flash_decode(q.cuda(), k.cuda(), v.cuda())
    assert torch.allclose(out.float().cpu(), ref, atol=4e-2, rtol=4e-2)


def test_reference_cxx_dispatcher_fp8(ops, golden):
    """dispatch_fp8_paged_attention<__half,__half> called the way the reference binding calls it
    (raw pointers, current stream), through its C++ symbol."""
    import ctypes as C
    from test_cabi_cpu import CXX_SYMBOLS
    fn = getattr(ops.L.load(), CXX_SYMBOLS[("fp8", "f16")])
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 8 + [C.c_int] * 5 + [C.c_float, C.c_bool, C.c_void_p]
    name, dtype, hd, lens = "fp8_f16_d128", torch.float16, 128, [300, 129, 64]
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    k8, v8, ks, vs, _, _ = cases.fp8_quantise(k, v)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc = O.paged_layout_from_dense(k8, cases.PAGE, perm).cuda()
    vc = O.paged_layout_from_dense(v8, cases.PAGE, perm).cuda()
    qd, ksd, vsd, btd, ld = q.cuda(), ks.cuda(), vs.cuda(), bt.cuda(), lens_t.cuda()
    out = torch.empty_like(qd)
    fn(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), ksd.data_ptr(), vsd.data_ptr(), btd.data_ptr(), ld.data_ptr(),
       out.data_ptr(), 3, 4, hd, bt.shape[1], 16, 1.0 / hd ** 0.5, False, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ref = torch.from_numpy(golden[f"{name}/out"])
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)


def test_reference_cxx_dispatcher_paged_and_decode(ops, golden):
    import ctypes as C
    from test_cabi_cpu import CXX_SYMBOLS
    lib = ops.L.load()
    st = torch.cuda.current_stream().cuda_stream
    fn = getattr(lib, CXX_SYMBOLS[("paged", "bf16")])
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int] * 4 + [C.c_float, C.c_void_p]
    name, dtype, hd, lens = "paged_bf16_d64_l1", torch.bfloat16, 64, [300, 129, 64]
    q, k, v, lens_t = cases.paged_inputs(dtype, hd, lens)
    bt = torch.from_numpy(golden[f"{name}/bt"])
    perm = bt.reshape(-1).to(torch.int64)
    kc, vc = O.paged_layout_from_dense(k, 16, perm).cuda(), O.paged_layout_from_dense(v, 16, perm).cuda()
    qd, btd, ld = q.cuda(), bt.cuda(), lens_t.cuda()
    out = torch.empty_like(qd)
    fn(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), btd.data_ptr(), ld.data_ptr(), out.data_ptr(), 3, 4, hd,
       bt.shape[1], 1.0 / hd ** 0.5, st)
    torch.cuda.synchronize()
    assert torch.allclose(out.float().cpu(), torch.from_numpy(golden[f"{name}/out"]), atol=4e-2, rtol=4e-2)
    fn = getattr(lib, CXX_SYMBOLS[("decode", "f32")])
    fn.restype = None
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float, C.c_void_p]
    q = torch.randn(2, 4, 1, 128, device="cuda")
    k = torch.randn(2, 4, 500, 128, device="cuda")
    v = torch.randn(2, 4, 500, 128, device="cuda")
    out = torch.empty_like(q)
    fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 2, 4, 500, 128, 1.0 / 128 ** 0.5, st)
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu(), O.ref_flash_decode(q.cpu(), k.cpu(), v.cpu()), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("hkv,q4,num_ctas", [(8, False, 148), (16, False, 37), (8, True, 148), (16, True, 5)])
def test_segment_table_matches_host_plan(ops, hkv, q4, num_ctas):
    """The (first CTA, number of CTAs) the kernel records per (sequence, head group) is exactly what
    the host restatement of the plan predicts: integer parity of the range partition."""
    import os
    if os.environ.get("CUDA_LLM_DECODE_KERNEL") == "tcgen05":
        pytest.skip("the host restatement describes the default kernel's stage layout")
    import partition_plan as P
    W = _W()
    g = torch.Generator().manual_seed(51)
    n = 24
    lens = torch.randint(1, 3000, (n,), generator=g).tolist()
    qls = [4 if (q4 and x) else 1 for x in (torch.rand(n, generator=g) < 0.4).tolist()]
    wl = W.build_workload("plan", context_lens=lens, q_lens=qls, num_q_heads=hkv * 4, num_kv_heads=hkv,
                          head_dim=128, page_size=16, q_dtype=torch.bfloat16, scale_mode="per_token",
                          pool_factor=1.1, seed=52).to("cuda")
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(n, hkv * 4, hkv, 128, 16, wl.max_q_len, num_ctas)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    ops.run_workload(wl, workspace=ws, num_ctas=num_ctas, check_status=True)
    n_hg = hkv // 8
    table = ws[256:256 + n * n_hg * 16].view(torch.int32).view(n * n_hg, 4).cpu()
    _, _, _, segs = P.plan(lens, qls, group=4, n_head_groups=n_hg, tok_stage=32, num_ctas=num_ctas,
                           weighted=(wl.max_q_len * 4 > 8))
    for (s, hg), (first, cnt) in segs.items():
        row = table[s * n_hg + hg]
        assert (int(row[0]), int(row[1])) == (first, cnt), (s, hg, row.tolist(), first, cnt)
