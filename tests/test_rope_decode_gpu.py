"""Rotary embedding fused into the decode kernel's query load, against the reference's own
ref_rope_attention (golden last rows) and against the oracle on the quantised formats."""
import pytest
import torch

import cases
from helpers import assert_parity, to_oracle
from oracle import paged_decode_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _params_16bit(ops, q, kc, vc, bt, lens, out, ws, cos, sin, dtype):
    L = ops.L
    fmt = L.KV_F16 if dtype == torch.float16 else L.KV_BF16
    dt = L.F16 if dtype == torch.float16 else L.BF16
    return L.PagedDecodeParams(
        query=q.data_ptr(), key_cache=kc.data_ptr(), value_cache=vc.data_ptr(), k_scale=None, v_scale=None,
        block_tables=bt.data_ptr(), context_lens=lens.data_ptr(), cu_q_lens=None, out=out.data_ptr(), lse=None,
        workspace=ws.data_ptr(), workspace_bytes=ws.numel(), num_seqs=q.shape[0], num_q_heads=q.shape[1],
        num_kv_heads=kc.shape[1], head_dim=q.shape[2], page_size=16, max_blocks_per_seq=bt.shape[1],
        num_blocks=kc.shape[0], max_q_len=1, q_dtype=dt, out_dtype=dt, k_format=fmt, v_format=fmt, scale_mode=0,
        softmax_scale=1.0 / q.shape[2] ** 0.5, num_ctas=0, flags=0, rope_cos=cos.data_ptr(), rope_sin=sin.data_ptr(),
        rope_positions=None, rope_num_positions=cos.shape[0])


@pytest.mark.parametrize("case", list(cases.rope_cases()), ids=lambda c: c[0])
def test_rope_decode_against_reference_golden(ops, golden, case):
    """The last row of the reference's causal RoPE attention is a decode step: the cache holds the
    rotated keys (rounded to the cache dtype), the query arrives unrotated and is rotated by the kernel
    at position context_len - 1."""
    import ctypes as C
    name, dtype, hd, seq = case
    q, k, v = cases.rope_inputs(dtype, hd, seq)
    cos, sin = O.rope_tables(seq, hd)
    k_rot = O.apply_rope(k, cos, sin).to(dtype)
    n_blocks = (seq + 15) // 16
    perm = torch.randperm(2 * n_blocks, generator=torch.Generator().manual_seed(1))
    kc = O.paged_layout_from_dense(k_rot, 16, perm).cuda()
    vc = O.paged_layout_from_dense(v, 16, perm).cuda()
    bt = perm.view(2, n_blocks).to(torch.int32).cuda()
    lens = torch.full((2,), seq, dtype=torch.int32).cuda()
    qd = q[:, :, -1, :].contiguous().cuda()
    out = torch.empty_like(qd)
    lib = ops.L.load()
    ws = torch.zeros(lib.cuda_llm_paged_decode_workspace_bytes(2, 4, 4, hd, 16, 1, 0), dtype=torch.uint8, device="cuda")
    p = _params_16bit(ops, qd, kc, vc, bt, lens, out, ws, cos.cuda(), sin.cuda(), dtype)
    ops.L.check(lib.cuda_llm_paged_decode(C.byref(p), torch.cuda.current_stream().cuda_stream), "cuda_llm_paged_decode")
    torch.cuda.synchronize()
    assert ops.decode_status(ws) == 0
    ref = torch.from_numpy(golden[f"{name}/out_last"])
    atol, rtol = {torch.float16: (2e-2, 2e-2), torch.bfloat16: (4e-2, 4e-2)}[dtype]
    assert torch.allclose(out.float().cpu(), ref, atol=atol, rtol=rtol)
    assert_parity(out, ref, dtype, name)


@pytest.mark.parametrize("cfg,batch,ctx_scale,q_dtype", [(2, 6, 1 / 8, None), (5, 16, 1 / 8, None), (1, 4, 1.0, None),
                                                          (3, 4, 1 / 16, torch.float16)])
def test_rope_decode_quantised_formats(ops, cfg, batch, ctx_scale, q_dtype):
    """FP8 per-token, MXFP8 + MXFP4 with q_len 1/4 (positions ctx - q_len + j), fp32 queries (split
    operands), against the oracle with the query rotated on the host."""
    from cuda_b200 import workloads as W
    wl = W.make_config(cfg, batch=batch, ctx_scale=ctx_scale)
    if q_dtype is not None:
        wl.query = wl.query.to(q_dtype)
    n_pos = int(wl.context_lens.max()) + 1
    cos, sin = O.rope_tables(n_pos, wl.head_dim)
    q_rot = O.rope_query(wl.query, cos, sin, wl.context_lens, wl.cu_q_lens)
    ref = O.ref_paged_decode(q_rot, to_oracle(wl), wl.softmax_scale, wl.cu_q_lens)
    g = wl.to("cuda")
    out = ops.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale, g.block_tables,
                                          g.context_lens, g.softmax_scale, cu_q_lens=g.cu_q_lens,
                                          max_q_len=g.max_q_len, check_status=True, rope_cos=cos, rope_sin=sin)
    assert_parity(out, ref, wl.query.dtype, f"rope cfg{cfg}")
    # explicit positions: the same answer when they spell out the default, another one otherwise
    pos = torch.zeros(wl.query.shape[0], dtype=torch.int32)
    cu = list(range(wl.num_seqs + 1)) if wl.cu_q_lens is None else wl.cu_q_lens.tolist()
    for s in range(wl.num_seqs):
        for j in range(cu[s + 1] - cu[s]):
            pos[cu[s] + j] = int(wl.context_lens[s]) - (cu[s + 1] - cu[s]) + j
    out2 = ops.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale, g.block_tables,
                                           g.context_lens, g.softmax_scale, cu_q_lens=g.cu_q_lens,
                                           max_q_len=g.max_q_len, rope_cos=cos, rope_sin=sin, rope_positions=pos)
    assert torch.equal(out, out2)
    pos3 = (pos // 2).to(torch.int32)
    ref3 = O.ref_paged_decode(O.rope_query(wl.query, cos, sin, wl.context_lens, wl.cu_q_lens, positions=pos3),
                              to_oracle(wl), wl.softmax_scale, wl.cu_q_lens)
    out3 = ops.fp8_paged_attention_forward(g.query, g.key_cache, g.value_cache, g.k_scale, g.v_scale, g.block_tables,
                                           g.context_lens, g.softmax_scale, cu_q_lens=g.cu_q_lens,
                                           max_q_len=g.max_q_len, rope_cos=cos, rope_sin=sin, rope_positions=pos3)
    assert_parity(out3, ref3, wl.query.dtype, f"rope cfg{cfg}, explicit positions")


def test_rope_position_outside_the_tables_is_reported(ops):
    from cuda_b200 import workloads as W
    wl = W.make_config(2, "cuda", batch=3, ctx_scale=1 / 16)
    cos, sin = O.rope_tables(8, wl.head_dim)                  # far fewer rows than the contexts need
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads,
                                                              wl.head_dim, wl.page_size, 1, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = ops.fp8_paged_attention_forward(wl.query, wl.key_cache, wl.value_cache, wl.k_scale, wl.v_scale,
                                          wl.block_tables, wl.context_lens, wl.softmax_scale, workspace=ws,
                                          rope_cos=cos, rope_sin=sin)
    assert ops.decode_status(ws) & ops.L.ST_BAD_POSITION
    assert torch.isfinite(out.float()).all()
