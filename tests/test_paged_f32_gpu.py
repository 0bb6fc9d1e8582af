"""Paged decode over an fp32 cache with pages of 16 tokens (the float instantiation of the reference's
``paged_attention``, ``paged_attention_kernel.cuh:20-145`` in the reference project) on the bulk-copy
kernel, against the CPU oracle on the same seeded inputs, through the C ABI.

Tolerance: the reference's own for this dtype (``tests/test_paged_attention.py``: 1e-4)."""
import ctypes

import pytest
import torch

from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu

TOL_MAX, TOL_MEAN = 1e-4, 1e-5


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _launches(ops):
    n = ctypes.c_uint64(0)
    ops.L.check(ops.L.load().cuda_llm_paged_attention_f32_launches(ctypes.byref(n)), "counter")
    return n.value


def _workload(ctx, hkv, group, d, seed, page=16, pool_factor=1.3):
    """Seeded fp32 workload; token slots behind a sequence's end and unused pages hold NaN."""
    from cuda_b200 import workloads as W
    wl = W.build_workload("pa32", context_lens=ctx, q_lens=None, num_q_heads=hkv * group, num_kv_heads=hkv,
                          head_dim=d, page_size=page, q_dtype=torch.float32, scale_mode="none",
                          pool_factor=pool_factor, seed=seed, cache_dtype=torch.float32)
    pool = wl.key_cache.shape[0]
    live = torch.zeros(pool, page, dtype=torch.bool)
    for s, c in enumerate(wl.context_lens.tolist()):
        n = (c + page - 1) // page
        if n == 0:
            continue
        rows = wl.block_tables[s, :n].long()
        live[rows] = True
        if c % page:
            live[rows[-1], c % page:] = False
    dead = ~live.view(pool, 1, 1, page)
    nan = torch.tensor(float("nan"))
    wl.key_cache = torch.where(dead, nan, wl.key_cache).contiguous()
    wl.value_cache = torch.where(dead, nan, wl.value_cache).contiguous()
    return wl


def _oracle(wl):
    kv = O.PagedKV(wl.key_cache, wl.value_cache, wl.block_tables, wl.context_lens, wl.page_size, wl.head_dim,
                   O.KV_F32, O.KV_F32, O.SCALE_NONE, O.SCALE_NONE)
    return O.ref_paged_decode(wl.query, kv, wl.softmax_scale)


def _run(ops, wl, expect_kernel=True):
    g = wl.to("cuda")
    before = _launches(ops)
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    torch.cuda.synchronize()
    assert _launches(ops) == before + (1 if expect_kernel else 0)
    return out


def _check(out, ref, name=""):
    assert out.dtype == torch.float32
    assert torch.isfinite(out).all(), name
    err = (out.cpu() - ref.float()).abs()
    assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN, \
        f"{name}: max-abs {err.max().item():.3e}, mean-abs {err.mean().item():.3e}"


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("hkv,group", [(1, 1), (4, 1), (2, 2), (2, 3), (8, 4), (2, 5), (2, 8), (3, 1), (32, 1)])
def test_head_shapes(ops, d, hkv, group):
    """GQA groups of 1-8 rows (one or two row groups of four), odd head counts, both head sizes; an empty
    sequence gives zeros."""
    wl = _workload([777, 0, 1, 15, 16, 17, 130, 2049], hkv, group, d, seed=3 + hkv + group)
    out = _run(ops, wl)
    _check(out, _oracle(wl), f"d {d} hkv {hkv} group {group}")
    assert (out[1] == 0).all()


def test_every_tail_length(ops):
    """Context lengths 1..200 in one launch: every position of the last page, NaN in the slots behind it."""
    wl = _workload(list(range(1, 201)), 2, 4, 128, seed=5)
    _check(_run(ops, wl), _oracle(wl), "tails")


def test_long_sequences_many_chunks(ops):
    """Sequences cut into up to 80 chunks (more than 32 pages of block table per item reload), next to
    short ones whose later chunks are empty."""
    wl = _workload([20000, 40, 9000, 5, 1300], 2, 4, 128, seed=7)
    _check(_run(ops, wl), _oracle(wl), "long")


def test_large_chunks(ops):
    """A block table so wide that an item covers more than 32 pages: the per-item block list is reloaded."""
    wl = _workload([140000, 300], 1, 1, 64, seed=8, pool_factor=1.05)
    _check(_run(ops, wl), _oracle(wl), "wide")


def test_batch_of_llama_shape(ops):
    wl = _workload(torch.randint(200, 1200, (48,), generator=torch.Generator().manual_seed(1)).tolist(), 8, 4, 128, seed=9)
    _check(_run(ops, wl), _oracle(wl), "batch")


def test_out_of_range_block_is_reported_not_read(ops):
    from cuda_b200 import _lib as L
    wl = _workload([100, 200], 2, 2, 128, seed=2).to("cuda")
    wl.block_tables[1, 3] = 10 ** 6
    n, hq, d = wl.query.shape
    lib = L.load()
    need = lib.cuda_llm_dense_decode_workspace_bytes(n, hq, 2, d, wl.block_tables.shape[1] * 16)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = torch.empty_like(wl.query)
    L.check(lib.cuda_llm_paged_attention(wl.query.data_ptr(), wl.key_cache.data_ptr(), wl.value_cache.data_ptr(),
                                         wl.block_tables.data_ptr(), wl.context_lens.data_ptr(), out.data_ptr(),
                                         n, hq, 2, d, 16, wl.block_tables.shape[1], wl.key_cache.shape[0],
                                         wl.softmax_scale, L.F32, ws.data_ptr(), ws.numel(), None), "paged_attention")
    torch.cuda.synchronize()
    assert ops.decode_status(ws) & L.ST_BAD_BLOCK


@pytest.mark.parametrize("page", [32, 64])
@pytest.mark.parametrize("hkv,group,d", [(2, 4, 128), (3, 1, 64), (2, 8, 128), (8, 4, 128)])
def test_pages_of_32_and_64_tokens(ops, page, hkv, group, d):
    """Pages of 32 / 64 tokens (an extension of the reference's 16): 16-token tiles fetched as TMA boxes.  Tails at
    every position of a page, an empty sequence, sequences of several chunks."""
    wl = _workload([777, 0, 1, 15, 16, 17, 31, 33, 63, 64, 65, 130, 2049, 5000], hkv, group, d, seed=4 + page + hkv, page=page)
    out = _run(ops, wl)
    _check(out, _oracle(wl), f"page {page} hkv {hkv} group {group} d {d}")
    assert (out[1] == 0).all()


def test_pages_of_64_tokens_long(ops):
    """More than 32 pages per item and a wide block table: the block list of an item is reloaded."""
    wl = _workload([150000, 300, 70000], 1, 2, 64, seed=12, page=64, pool_factor=1.05)
    _check(_run(ops, wl), _oracle(wl), "page 64 long")


def test_repeatable(ops):
    """Items are handed out dynamically, but every partial result has a fixed place and the merge a fixed
    order: two runs are bit-identical."""
    wl = _workload([3000, 700, 2222, 64], 4, 4, 128, seed=6)
    assert torch.equal(_run(ops, wl), _run(ops, wl))


# ------------------------------------------------------------------------------------------------
# contiguous fp32 K/V (the reference's async_flash_decode, tensors [B, H, S, D]): the token-major mode
# ------------------------------------------------------------------------------------------------
def _flash_case(b, hkv, group, s, d, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hkv * group, 1, d, generator=g)
    k = torch.randn(b, hkv, s, d, generator=g)
    v = torch.randn(b, hkv, s, d, generator=g)
    ref = O.ref_flash_decode(q, k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1))
    return q, k, v, ref


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("hkv,group", [(1, 1), (2, 2), (2, 3), (8, 4), (2, 8), (3, 1)])
@pytest.mark.parametrize("s", [1, 15, 16, 17, 130, 777, 2049])
def test_flash_decode_fp32(ops, d, hkv, group, s):
    q, k, v, ref = _flash_case(2, hkv, group, s, d, seed=s + hkv + group)
    before = _launches(ops)
    out = ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    assert _launches(ops) == before + 1
    _check(out, ref, f"flash d {d} hkv {hkv} group {group} s {s}")


def test_flash_decode_fp32_long(ops):
    """One long sequence (many chunks per head, a short last tile) and a batch of short ones."""
    for b, s in ((1, 50003), (24, 301)):
        q, k, v, ref = _flash_case(b, 2, 4, s, 128, seed=s)
        out = ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
        _check(out, ref, f"flash long {b}x{s}")


def test_bounded_wait_runs_out_and_the_context_survives(ops, monkeypatch):
    """CUDA_LLM_TEST_STALL=1: the first copy of the launch is announced and never sent.  The wait must run
    out, the call must return, the status word must say CUDA_LLM_ST_TIMEOUT, and the next call on the same
    workspace must be bit-identical to the call before."""
    from cuda_b200 import _lib as L
    wl = _workload([3000, 700, 2222, 64], 4, 4, 128, seed=6).to("cuda")
    n, hq, d = wl.query.shape
    lib = L.load()
    need = lib.cuda_llm_dense_decode_workspace_bytes(n, hq, 4, d, wl.block_tables.shape[1] * 16)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")

    def call():
        out = torch.empty_like(wl.query)
        L.check(lib.cuda_llm_paged_attention(wl.query.data_ptr(), wl.key_cache.data_ptr(), wl.value_cache.data_ptr(),
                                             wl.block_tables.data_ptr(), wl.context_lens.data_ptr(), out.data_ptr(),
                                             n, hq, 4, d, 16, wl.block_tables.shape[1], wl.key_cache.shape[0],
                                             wl.softmax_scale, L.F32, ws.data_ptr(), ws.numel(), None), "paged_attention")
        torch.cuda.synchronize()                            # returns: nothing hangs
        return out

    ref = call()
    assert ops.decode_status(ws) == 0
    monkeypatch.setenv("CUDA_LLM_TEST_STALL", "1")
    call()
    assert ops.decode_status(ws) & L.ST_TIMEOUT
    monkeypatch.delenv("CUDA_LLM_TEST_STALL")
    ws[:4] = 0
    again = call()
    assert ops.decode_status(ws) == 0
    assert torch.equal(again, ref)
