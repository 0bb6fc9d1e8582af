"""Failure paths of the decode kernel, exercised without faulting or hanging anything: a wait
that runs out by construction, status words, workspace sharing between entry points."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from cuda_b200 import ops as _ops
    _ops.L.load()
    return _ops


def _ws(ops, wl, num_ctas=0):
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads,
                                                              wl.head_dim, wl.page_size, wl.max_q_len, num_ctas)
    return torch.zeros(need, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("cfg,batch,ctx_scale", [(2, 8, 1 / 8), (5, 12, 1 / 8)])
def test_bounded_wait_runs_out_and_the_context_survives(ops, cfg, batch, ctx_scale):
    """CUDA_LLM_FLAG_TEST_STALL: the first CTA announces the bytes of its first stage and never sends
    them, waits give up after a few thousand polls.  Every warp must return, the host must read
    CUDA_LLM_ST_TIMEOUT, and the next ordinary call on the same workspace must be bit-identical to
    the call before."""
    from cuda_b200 import workloads as W
    wl = W.make_config(cfg, "cuda", batch=batch, ctx_scale=ctx_scale, seed=77)
    ws = _ws(ops, wl)
    ref = ops.run_workload(wl, workspace=ws, check_status=True).clone()
    ops.run_workload(wl, workspace=ws, flags=ops.L.FLAG_TEST_STALL, out=torch.empty_like(wl.query))
    torch.cuda.synchronize()                               # returns: nothing hangs
    st = ops.decode_status(ws)
    assert st & ops.L.ST_TIMEOUT, hex(st)
    assert ops.decode_status(ws) == 0                      # cleared by the read
    again = ops.run_workload(wl, workspace=ws, check_status=True)
    assert torch.equal(again, ref)


def test_unwritten_table_entries_are_not_followed(ops):
    """One CTA owns four sequences and stalls on its first stage: the table entries of the later
    sequences are never written.  The workspace was filled with 0x7F bytes beforehand, so those
    entries are garbage; the merge must refuse them (CUDA_LLM_ST_INCOMPLETE, rows of zeros) instead
    of indexing the partials with them, and the next ordinary call must be correct."""
    from cuda_b200 import workloads as W
    wl = W.make_config(2, "cuda", batch=4, ctx_scale=1 / 16, seed=78)
    ws = torch.full((_ws(ops, wl, 1).numel(),), 0x7F, dtype=torch.uint8, device="cuda")
    ops.L.check(ops.L.load().cuda_llm_workspace_init(ws.data_ptr(), ws.numel(),
                                                     torch.cuda.current_stream().cuda_stream), "init")
    out = ops.run_workload(wl, workspace=ws, num_ctas=1, flags=ops.L.FLAG_TEST_STALL)
    torch.cuda.synchronize()
    st = ops.decode_status(ws)
    assert st & ops.L.ST_TIMEOUT and st & ops.L.ST_INCOMPLETE, hex(st)
    assert (out[-1] == 0).all()                           # the last sequence was never reached
    ref = ops.run_workload(wl, workspace=_ws(ops, wl, 1), num_ctas=1, check_status=True)
    assert torch.equal(ops.run_workload(wl, workspace=ws, num_ctas=1, check_status=True), ref)


def test_dense_fp32_path_leaves_the_status_word_alone(ops):
    """One workspace serves every entry point: after an fp32 paged_attention (SIMT split-KV kernel,
    partials in the workspace) a quantised decode with check_status must not read float bits as a status."""
    from cuda_b200 import workloads as W
    wl32 = W.build_workload("pa32", context_lens=[300, 77], q_lens=None, num_q_heads=8, num_kv_heads=8, head_dim=64,
                            page_size=16, q_dtype=torch.float32, scale_mode="none", seed=4,
                            cache_dtype=torch.float32).to("cuda")
    ops.paged_attention_forward(wl32.query, wl32.key_cache, wl32.value_cache, wl32.block_tables, wl32.context_lens)
    q = torch.randn(2, 8, 1, 64, device="cuda")
    k = torch.randn(2, 8, 200, 64, device="cuda")
    ops.async_flash_decode(q, k, k)
    wl = W.make_config(2, "cuda", batch=3, ctx_scale=1 / 16, seed=80)
    ops.run_workload(wl, check_status=True)               # shares the per-stream workspace


def test_all_sequences_empty_with_stable_metadata(ops):
    """No CTA has work: the grid must still order itself behind the kernel in front of it; outputs are
    zeros, log-sum-exps -inf."""
    from cuda_b200 import workloads as W
    wl = W.make_config(2, "cuda", batch=4, ctx_scale=1 / 16, seed=81)
    wl.context_lens.zero_()
    big = W.make_config(2, "cuda", batch=8, ctx_scale=1 / 8, seed=82)
    for _ in range(3):
        ops.run_workload(big)                              # a kernel in front that is still running
        out, lse = ops.run_workload(wl, return_lse=True, flags=ops.L.FLAG_STABLE_METADATA)
    torch.cuda.synchronize()
    assert (out == 0).all() and torch.isinf(lse).all() and (lse < 0).all()


def test_wrong_device_generation_code_exists(ops):
    """CUDA_LLM_EDEVICE is what a non-sm_100 device gets; on the B200 the check passes."""
    assert ops.L.EDEVICE == -5
    assert torch.cuda.get_device_capability()[0] == 10
