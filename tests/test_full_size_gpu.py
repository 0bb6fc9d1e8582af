"""The benchmark configurations at their full sizes, through properties that do not need the
oracle on every byte: a sample of sequences against the oracle, invariance under the number of
CTAs the units are cut into, and the append -> decode round trip of the cache formats."""
import dataclasses

import pytest
import torch

from helpers import assert_parity, oracle_out

pytestmark = pytest.mark.gpu


def _sample(wl, ids):
    """The sub-workload of sequences `ids` (page pool shared)."""
    from cuda_b200 import sharding
    return sharding.slice_sequences(wl, ids)


@pytest.mark.parametrize("cfg,ids", [(2, [0, 17, 63]), (3, [1, 64, 127]), (5, [0, 100, 255])])
def test_full_config_sample_vs_oracle_and_split_invariance(cfg, ids):
    from cuda_b200 import ops, workloads as W
    wl = W.make_config(cfg, "cuda", poison=True)
    L = ops.L.load()
    outs = []
    for n_ctas in (0, 97):
        need = L.cuda_llm_paged_decode_workspace_bytes(wl.num_seqs, wl.num_q_heads, wl.num_kv_heads, wl.head_dim,
                                                       wl.page_size, wl.max_q_len, n_ctas)
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        outs.append(ops.run_workload(wl, workspace=ws, num_ctas=n_ctas, check_status=True))
    assert torch.isfinite(outs[0]).all()            # poisoned tails and unused pages never leak
    assert (outs[0].float() - outs[1].float()).abs().max() <= 2e-2
    # a few whole sequences against the oracle (the oracle needs ~25 ms per sequence)
    sub = _sample(wl, ids)
    ref = oracle_out(sub)
    cu = list(range(wl.num_seqs + 1)) if wl.cu_q_lens is None else wl.cu_q_lens.tolist()
    rows = [r for s in ids for r in range(cu[s], cu[s + 1])]
    assert_parity(outs[0][rows], ref, wl.query.dtype, f"config {cfg} sample")


def test_full_long_context_vs_oracle():
    """Config 4 in full (2 x 131072 tokens): every CTA holds a piece of each sequence."""
    from cuda_b200 import ops, workloads as W
    wl = W.make_config(4, "cuda")
    out, lse = ops.run_workload(wl, return_lse=True, check_status=True)
    ref, ref_lse = oracle_out(wl, return_lse=True)
    assert_parity(out, ref, torch.bfloat16, "config 4")
    assert (lse.cpu() - ref_lse).abs().max() < 2e-2
