"""Paged decode over an unquantised fp16 / bf16 cache (the reference's paged_attention, layout
cache[num_blocks, heads, head_dim, page]) on the persistent tensor-core kernel, against the CPU
oracle on the same seeded inputs."""
import pytest
import torch

from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu

# Q and P are rounded to the cache's 16-bit type before the tensor-core products
TOL = {torch.float16: (2e-2, 2e-3), torch.bfloat16: (2e-2, 2e-3)}


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    return _ops


def _workload(dtype, ctx, q_lens, hkv, group, d, page, seed):
    from cuda_b200 import workloads as W
    return W.build_workload("kv16", context_lens=ctx, q_lens=q_lens, num_q_heads=hkv * group,
                            num_kv_heads=hkv, head_dim=d, page_size=page, q_dtype=dtype, scale_mode="none",
                            pool_factor=1.3, seed=seed, cache_dtype=dtype)


def _oracle(wl, return_lse=False):
    kv = O.PagedKV(wl.key_cache, wl.value_cache, wl.block_tables, wl.context_lens, wl.page_size, wl.head_dim,
                   O.KV_F32, O.KV_F32, O.SCALE_NONE, O.SCALE_NONE)
    return O.ref_paged_decode(wl.query, kv, wl.softmax_scale, wl.cu_q_lens, return_lse=return_lse)


def _check(out, ref, dtype, name=""):
    err = (out.float().cpu() - ref.float()).abs()
    mx, mean = TOL[dtype]
    assert torch.isfinite(out).all(), name
    assert err.max().item() <= mx and err.mean().item() <= mean, \
        f"{name}: max-abs {err.max().item():.3e}, mean-abs {err.mean().item():.3e}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("page", [16, 32, 64])
@pytest.mark.parametrize("hkv,group", [(1, 1), (1, 8), (2, 4), (4, 1), (8, 4), (16, 2), (3, 1), (32, 1)])
def test_head_and_page_shapes(ops, dtype, page, hkv, group):
    wl = _workload(dtype, [777, 0, 1, 15, 16, 17, 130, 2049], None, hkv, group, 128, page, seed=11)
    g = wl.to("cuda")
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    _check(out, _oracle(wl), dtype, f"{dtype} page {page} hkv {hkv} group {group}")
    assert (out[1] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_64(ops, dtype):
    wl = _workload(dtype, [300, 64, 5, 1025], None, 4, 2, 64, 16, seed=12)
    g = wl.to("cuda")
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    _check(out, _oracle(wl), dtype)


@pytest.mark.parametrize("page", [16, 32, 64])
def test_every_context_length(ops, page):
    ctx = list(range(0, 2 * page + 18))
    wl = _workload(torch.bfloat16, ctx, None, 2, 4, 128, page, seed=13)
    g = wl.to("cuda")
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    _check(out, _oracle(wl), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group,q_lens,max_q", [(1, [4, 1, 8, 3], 8), (4, [2, 1, 2, 1], 2), (4, [4, 3, 1, 4], 4),
                                                (2, [8, 5, 1, 7], 8), (1, [16, 9, 1, 12], 16)])
def test_q_len_causal_and_lse(ops, dtype, group, q_lens, max_q):
    """Several query rows per sequence (bottom-right causal), up to 16 rows per KV head, with the
    log-sum-exp output; the status word must stay clean."""
    wl = _workload(dtype, [500, 33, 16, 1200], q_lens, 2, group, 128, 16, seed=14)
    g = wl.to("cuda")
    out, lse = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens,
                                           cu_q_lens=g.cu_q_lens, max_q_len=max_q, return_lse=True,
                                           check_status=True)
    ref, ref_lse = _oracle(wl, return_lse=True)
    _check(out, ref, dtype)
    assert torch.allclose(lse.cpu(), ref_lse.float(), atol=2e-2, rtol=1e-3)


def test_split_invariance(ops):
    """The result must not depend on how many CTAs the unit range is cut into."""
    wl = _workload(torch.bfloat16, [4000, 900, 77], None, 8, 4, 128, 16, seed=15)
    g = wl.to("cuda")
    outs = [ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens,
                                        num_ctas=n, check_status=True).float() for n in (1, 7, 148)]
    ref = _oracle(wl)
    for o in outs:
        _check(o, ref, torch.bfloat16)
    assert (outs[0] - outs[2]).abs().max().item() < 1e-2


def test_llama_shape_batch(ops):
    """The headline shape with a bf16 cache: 32 query heads over 8 KV heads, page 16."""
    torch.manual_seed(0)
    ctx = torch.randint(200, 1500, (24,)).tolist()
    wl = _workload(torch.bfloat16, ctx, None, 8, 4, 128, 16, seed=16)
    g = wl.to("cuda")
    out = ops.paged_attention_forward(g.query, g.key_cache, g.value_cache, g.block_tables, g.context_lens)
    _check(out, _oracle(wl), torch.bfloat16)


# ------------------------------------------------------------------------------------------
# contiguous K/V [batch, kv_heads, seq, head_dim] (the reference's async_flash_decode)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("seq_len", [1, 15, 16, 17, 127, 128, 129, 1000, 4100])
@pytest.mark.parametrize("hkv,group,d", [(4, 1, 128), (2, 4, 128), (1, 8, 128), (3, 2, 64)])
def test_flash_decode_shapes(ops, dtype, seq_len, hkv, group, d):
    g = torch.Generator().manual_seed(seq_len * 31 + hkv)
    b = 3
    q = torch.randn(b, hkv * group, 1, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, seq_len, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, seq_len, d, generator=g).to(dtype)
    ref = O.ref_flash_decode(q, k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1))
    out = ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
    assert out.shape == q.shape and out.dtype == dtype
    _check(out, ref, dtype, f"seq {seq_len} hkv {hkv} group {group} d {d}")


def test_flash_decode_many_heads_few_ctas_worth_of_work(ops):
    """More (batch, head) segments than CTAs and fewer: both partitions of the unit range."""
    g = torch.Generator().manual_seed(77)
    for b, h, s in ((40, 8, 300), (1, 2, 9000)):
        q = torch.randn(b, h, 1, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(b, h, s, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(b, h, s, 128, generator=g).to(torch.bfloat16)
        out = ops.async_flash_decode(q.cuda(), k.cuda(), v.cuda())
        _check(out, O.ref_flash_decode(q, k, v), torch.bfloat16, f"b {b} h {h} s {s}")
