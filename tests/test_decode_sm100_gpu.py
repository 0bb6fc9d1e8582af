"""The tcgen05 / tensor-memory decode kernel (``CUDA_LLM_FLAG_TCGEN05``) against the CPU oracle, through
the C ABI: same contract as the default kernel for the calls it serves (head_dim 128, pages of 16
tokens, E4M3 K and V with per-token fp32 or E8M0 block scales, 16-bit queries).

Spec: ``oracle/paged_decode_oracle.py``; the reference's own recipe for E4M3 caches is
``tests/test_kernels_misc.py:42-64`` in the reference project, the microscaling formats are extensions
(parity unpinned by the reference)."""
import ctypes

import pytest
import torch

from helpers import assert_parity, oracle_out, to_oracle
from oracle import paged_decode_oracle as O
from test_mx_exactness_gpu import _single_token_workload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _launches(ops):
    n = ctypes.c_uint64(0)
    ops.L.check(ops.L.load().cuda_llm_decode_tcgen05_counters(ctypes.byref(n), None), "counters")
    return n.value


def _run(ops, wl, **kw):
    """Run on the tcgen05 kernel and prove that it was the kernel that ran."""
    before = _launches(ops)
    out = ops.run_workload(wl, flags=ops.L.FLAG_TCGEN05 | kw.pop("flags", 0), check_status=kw.pop("check_status", True), **kw)
    assert _launches(ops) == before + 1, "the call did not reach the tcgen05 kernel"
    return out


def _workload(lens, q_lens=None, hq=32, hkv=8, scale_mode="per_token", seed=0, q_dtype=torch.bfloat16, **kw):
    from cuda_b200 import workloads as W
    return W.build_workload("sm100", context_lens=lens, q_lens=q_lens, num_q_heads=hq, num_kv_heads=hkv, head_dim=128,
                            page_size=16, q_dtype=q_dtype, scale_mode=scale_mode, pool_factor=1.3, seed=seed, **kw)


@pytest.mark.parametrize("batch,ctx_scale", [(2, 1 / 16), (8, 1 / 8), (16, 1 / 4)])
def test_config2_shapes(ops, batch, ctx_scale):
    from cuda_b200 import workloads as W
    wl = W.make_config(2, "cpu", batch=batch, ctx_scale=ctx_scale, seed=40 + batch)
    out = _run(ops, wl.to("cuda"))
    assert_parity(out, oracle_out(wl), torch.bfloat16, "cfg2")


@pytest.mark.parametrize("hq,hkv", [(8, 8), (16, 8), (64, 8), (32, 2), (12, 4), (24, 4)])
@pytest.mark.parametrize("q_dtype", [torch.bfloat16, torch.float16])
def test_group_sizes(ops, hq, hkv, q_dtype):
    """GQA groups of 1, 2, 8, 16, 3 and 6 query heads per KV head (4, 8 or 16 padded accumulator rows)."""
    wl = _workload([1, 15, 16, 17, 127, 128, 129, 300, 1025], hq=hq, hkv=hkv, seed=hq + hkv, q_dtype=q_dtype)
    out = _run(ops, wl.to("cuda"))
    assert_parity(out, oracle_out(wl), q_dtype, f"group {hq // hkv}")


def test_every_tail_length(ops):
    """Context lengths 1..272 in one launch: every position of the tile tail, poisoned slots behind it."""
    wl = _workload(list(range(1, 273)), hq=8, hkv=2, seed=5)
    out = _run(ops, wl.to("cuda"))
    assert_parity(out, oracle_out(wl), torch.bfloat16, "tails")


@pytest.mark.parametrize("scale_mode", ["per_token", "mx_e8m0"])
def test_multi_token_queries_causal(ops, scale_mode):
    """q_len 1 / 2 / 4 mixed (speculative verify): up to 16 rows per KV head, causal inside the query."""
    lens = [5, 64, 130, 257, 999, 33, 128, 4]
    q_lens = [1, 4, 2, 4, 4, 1, 4, 4]
    wl = _workload(lens, q_lens=q_lens, hq=32, hkv=8, scale_mode=scale_mode, seed=9)
    out = _run(ops, wl.to("cuda"))
    assert_parity(out, oracle_out(wl), torch.bfloat16, "q_len mix")


def test_query_longer_than_declared_still_fits_the_rows(ops):
    """A call with query lengths whose max_q_len under-declares them: a query of two tokens and a group of four
    fits the 8 rows the launch has (the four-row variant is for calls without query lengths only)."""
    wl = _workload([300, 40, 1000, 17], q_lens=[2, 1, 2, 2], hq=8, hkv=2, seed=31)
    ref = oracle_out(wl)
    g = wl.to("cuda")
    before = _launches(ops)
    out = ops.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale, g.block_tables,
                                          g.context_lens, g.softmax_scale, cu_q_lens=g.cu_q_lens, max_q_len=1,
                                          check_status=True, flags=ops.L.FLAG_TCGEN05)
    assert _launches(ops) == before + 1
    assert_parity(out, ref, torch.bfloat16, "q_len 2 with max_q_len 1")


@pytest.mark.parametrize("hq,hkv", [(64, 8), (16, 4)])
def test_mx_block_scales(ops, hq, hkv):
    wl = _workload([1, 31, 200, 1500, 77, 640], hq=hq, hkv=hkv, scale_mode="mx_e8m0", seed=21, mx_exponent_range=(-4, 4))
    out, lse = _run(ops, wl.to("cuda"), return_lse=True)
    ref, ref_lse = oracle_out(wl, return_lse=True)
    assert_parity(out, ref, torch.bfloat16, "mx")
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("spread", [6, 50])
def test_mx_wide_exponent_range(ops, spread):
    """V block exponents over [-30, +20], blocks of one token up to 2^50 apart: every block has its own
    running maximum in this kernel, so none of them is flushed."""
    from cuda_b200 import workloads as W
    wl = _workload([1, 17, 300, 64, 1000, 33], hq=16, hkv=4, scale_mode="mx_e8m0", seed=13)
    g = torch.Generator().manual_seed(14)
    pool = wl.v_scale.shape[0]
    base = torch.randint(-30 + spread if spread < 50 else 20, 21, (pool, 4, 1, 16), generator=g)
    e = base - torch.randint(0, spread + 1, (pool, 4, 4, 16), generator=g)
    live = wl.v_scale != W.POISON_E8M0
    wl.v_scale = torch.where(live, (e.clamp(-30, 20) + 127).to(torch.uint8), wl.v_scale)
    ref = O.ref_paged_decode(wl.query, to_oracle(wl), wl.softmax_scale)
    out = _run(ops, wl.to("cuda")).float().cpu()
    assert torch.isfinite(out).all()
    scale = ref.abs().amax(dim=-1, keepdim=True).clamp_min(1.0)
    err = (out - ref).abs() / scale
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())


@pytest.mark.parametrize("e_lo,e_hi", [(-30, 20), (-90, 90)])
def test_v_dequant_bit_exact(ops, e_lo, e_hi):
    """Context length 1: the softmax weight is exactly 1 (E4M3 high part 1, residual 0), so the output
    must be the dequantised V row bit for bit, for every E4M3 code and every block exponent."""
    wl = _single_token_workload("fp8_e4m3", 128, hkv=8, n_seq=64, e_lo=e_lo, e_hi=e_hi, spread=14, seed=3,
                                q_dtype=torch.bfloat16)
    kv = to_oracle(wl)
    out = _run(ops, wl.to("cuda")).cpu()
    group = wl.num_q_heads // wl.num_kv_heads
    for s in range(wl.num_seqs):
        _, v = O.gather_sequence(kv, s)
        want = v[:, 0].repeat_interleave(group, dim=0).to(torch.bfloat16)
        assert torch.equal(out[s], want), (s, (out[s].float() - want.float()).abs().max())


@pytest.mark.parametrize("scale_mode", ["per_token", "mx_e8m0"])
@pytest.mark.parametrize("with_q_lens", [False, True])
def test_many_one_stage_segments_on_few_ctas(ops, scale_mode, with_q_lens):
    """Dozens of sequences shorter than one 128-token tile on 3 and 7 CTAs: every stage starts and ends a segment,
    so the query warp runs two segments ahead of the softmax groups all the time.  (A group that lagged two such
    segments behind used to miss a phase of the query barrier and give up; the buffer is now released by the
    groups as well.)  Repeated, with the status word checked every time."""
    lens = [40, 44, 874, 14, 29, 35, 360, 7, 99, 120, 5, 61, 33, 127, 128, 1, 90, 17, 64, 12] * 2
    q_lens = [1] * len(lens) if with_q_lens else None
    wl = _workload(lens, q_lens=q_lens, hq=2, hkv=2, scale_mode=scale_mode, seed=210)
    ref = oracle_out(wl)
    dev = wl.to("cuda")
    for num_ctas in (7, 3):
        for _ in range(15):
            out = _run(ops, dev, num_ctas=num_ctas)            # check_status=True: a wait that ran out raises
        assert_parity(out, ref, torch.bfloat16, f"{num_ctas} CTAs")


def test_split_across_many_ctas_and_few(ops):
    """Two long sequences over all SMs (every segment straddles many CTAs) and the same on 3 CTAs."""
    wl = _workload([20000, 9000], hq=32, hkv=8, seed=31)
    ref = oracle_out(wl)
    dev = wl.to("cuda")
    assert_parity(_run(ops, dev), ref, torch.bfloat16, "all SMs")
    assert_parity(_run(ops, dev, num_ctas=3), ref, torch.bfloat16, "3 CTAs")


def test_bad_block_index_sets_the_status_bit(ops):
    wl = _workload([100, 200], hq=8, hkv=8, seed=2).to("cuda")
    wl.block_tables[1, 3] = 10 ** 6
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(2, 8, 8, 128, 16, 1, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    _run(ops, wl, workspace=ws, check_status=False)
    torch.cuda.synchronize()
    assert ops.decode_status(ws) & ops.L.ST_BAD_BLOCK


def test_bounded_waits_run_out_and_the_context_survives(ops):
    """CUDA_LLM_FLAG_TEST_STALL on this kernel: the bytes of the first unit are announced and never sent.
    Every warp must return (the tensor memory is released at the common exit), the host must read
    CUDA_LLM_ST_TIMEOUT and the time-out counter must move; the next call must be bit-identical to the
    call before."""
    from cuda_b200 import workloads as W
    wl = W.make_config(2, "cuda", batch=8, ctx_scale=1 / 8, seed=77)
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads, 128, 16, 1, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    ref = _run(ops, wl, workspace=ws).clone()
    t0 = ctypes.c_uint32(0)
    ops.L.check(ops.L.load().cuda_llm_decode_tcgen05_counters(None, ctypes.byref(t0)), "counters")
    _run(ops, wl, workspace=ws, flags=ops.L.FLAG_TEST_STALL, out=torch.empty_like(wl.query), check_status=False)
    torch.cuda.synchronize()                               # returns: nothing hangs
    st = ops.decode_status(ws)
    assert st & ops.L.ST_TIMEOUT, hex(st)
    t1 = ctypes.c_uint32(0)
    ops.L.check(ops.L.load().cuda_llm_decode_tcgen05_counters(None, ctypes.byref(t1)), "counters")
    assert t1.value > t0.value
    again = _run(ops, wl, workspace=ws)
    assert torch.equal(again, ref)


def test_calls_outside_its_shapes_keep_the_default_kernel(ops):
    """The flag is a request, not a requirement: pages of 32 tokens, head_dim 64 or an fp32 query run on the
    default kernel and still give the right answer."""
    from cuda_b200 import workloads as W
    before = _launches(ops)
    for cfg in (1, 3):
        wl = W.make_config(cfg, "cpu", batch=4, ctx_scale=1 / 16, seed=3)
        out = ops.run_workload(wl.to("cuda"), flags=ops.L.FLAG_TCGEN05, check_status=True)
        assert_parity(out, oracle_out(wl), wl.query.dtype, f"cfg{cfg}")
    assert _launches(ops) == before
