"""Glue between workloads, the CUDA ops and the CPU oracle (tests only)."""
import torch

from oracle import paged_decode_oracle as O


def to_oracle(wl) -> O.PagedKV:
    w = wl.to("cpu")
    return O.PagedKV(w.key_cache, w.value_cache, w.block_tables, w.context_lens, w.page_size,
                     w.head_dim, w.k_format, w.v_format, w.k_scale_mode, w.v_scale_mode,
                     w.k_scale, w.v_scale)


def oracle_out(wl, return_lse=False, seqs=None):
    w = wl.to("cpu")
    kv = to_oracle(w)
    return O.ref_paged_decode(w.query, kv, w.softmax_scale, w.cu_q_lens, return_lse=return_lse)


# stated tolerance for bf16/f16 outputs (max-abs 2e-2, mean-abs 2e-3); fp32 outputs (hi/lo split operands) are held tighter
TOL_MAX_ABS = {torch.bfloat16: 2e-2, torch.float16: 2e-2, torch.float32: 2e-3}
TOL_MEAN_ABS = {torch.bfloat16: 2e-3, torch.float16: 2e-3, torch.float32: 2e-4}


def assert_parity(out, ref, dtype, name=""):
    o, r = out.float().cpu(), ref.float().cpu()
    assert o.shape == r.shape, f"{name}: shape {o.shape} != {r.shape}"
    assert torch.isfinite(o).all(), f"{name}: non-finite output"
    err = (o - r).abs()
    mx, mean = err.max().item(), err.mean().item()
    assert mx <= TOL_MAX_ABS[dtype] and mean <= TOL_MEAN_ABS[dtype], \
        f"{name}: max-abs {mx:.3e} (<= {TOL_MAX_ABS[dtype]}), mean-abs {mean:.3e} (<= {TOL_MEAN_ABS[dtype]})"
    return mx, mean
