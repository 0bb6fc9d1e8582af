"""Seeded synthetic decode workloads in the reference's paged-cache layout.

The cache layout is the reference's ``cache[num_blocks, heads, head_dim, page]`` with the
token index innermost (``tests/_utils.py:105-133``, read by ``paged_attention_kernel.cuh:24-25``);
quantisation follows the reference's E4M3 recipe (``tests/test_kernels_misc.py:51-55``:
``scale = amax/448`` clamped, ``(x/scale).to(float8_e4m3fn)``) and extends it to per-token
scales and to OCP microscaling (32-element blocks along head_dim, E8M0 scale per block).

Everything here is plain torch and runs on whichever device it is given: the tests build
small cases on the CPU, the benchmark builds the full-size ones directly in HBM.  These are
stand-ins shaped like Llama-3 decode steps; no dataset is involved.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Tuple, List, Optional, Sequence

import torch

KV_FP8_E4M3 = "fp8_e4m3"
KV_FP4_E2M1 = "fp4_e2m1"
KV_F32 = "f32"
SCALE_NONE = "none"
SCALE_PER_HEAD = "per_head"
SCALE_PER_BLOCK = "per_block"
SCALE_PER_TOKEN = "per_token"
SCALE_MX_E8M0 = "mx_e8m0"

E4M3_MAX = 448.0
POISON_E4M3 = 0x7F          # NaN code: an out-of-range read shows up as NaN in the output
POISON_E8M0 = 0xFF          # NaN code


@dataclass
class DecodeWorkload:
    name: str
    query: torch.Tensor                  # [total_q, Hq, D]
    key_cache: torch.Tensor              # uint8 [NB, Hkv, D, page]
    value_cache: torch.Tensor            # uint8 [NB, Hkv, D or D/2, page]
    k_scale: Optional[torch.Tensor]
    v_scale: Optional[torch.Tensor]
    block_tables: torch.Tensor           # int32 [S, max_blocks]
    context_lens: torch.Tensor           # int32 [S]
    cu_q_lens: Optional[torch.Tensor]    # int32 [S+1] or None (q_len 1 everywhere)
    page_size: int
    head_dim: int
    num_q_heads: int
    num_kv_heads: int
    k_format: str = KV_FP8_E4M3
    v_format: str = KV_FP8_E4M3
    k_scale_mode: str = SCALE_PER_HEAD
    v_scale_mode: str = SCALE_PER_HEAD
    softmax_scale: float = 0.0
    max_q_len: int = 1
    meta: dict = field(default_factory=dict)

    @property
    def num_seqs(self) -> int:
        return int(self.context_lens.shape[0])

    def kv_bytes(self) -> int:
        """Algorithmic HBM bytes of K+V (payload + scales) over valid tokens only."""
        tokens = int(self.context_lens.clamp_min(0).sum().item())
        per = (bytes_per_token_head(self.head_dim, self.k_format, self.k_scale_mode)
               + bytes_per_token_head(self.head_dim, self.v_format, self.v_scale_mode))
        return tokens * self.num_kv_heads * per

    def to(self, device) -> "DecodeWorkload":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device) if isinstance(v, torch.Tensor) else v
        return DecodeWorkload(**kw)


def bytes_per_token_head(head_dim: int, fmt: str, scale_mode: str, elem_bytes: int = 1) -> int:
    payload = head_dim // 2 if fmt == KV_FP4_E2M1 else head_dim * elem_bytes
    if scale_mode == SCALE_PER_TOKEN:
        return payload + 4
    if scale_mode == SCALE_MX_E8M0:
        return payload + head_dim // 32
    return payload


# --------------------------------------------------------------------------------------
# Quantisers (write side of the cache formats)
# --------------------------------------------------------------------------------------
def quant_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> E4M3 codes (uint8), round-to-nearest-even, exactly torch's cast, as the
    reference test does (``tests/test_kernels_misc.py:54-55``)."""
    return x.to(torch.float8_e4m3fn).view(torch.uint8)


def quant_e2m1(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> E2M1 codes (uint8 in 0..15), round to nearest, ties to the even code,
    saturating at 6."""
    mag = x.abs()
    # midpoints between {0,.5,1,1.5,2,3,4,6}; tie -> even code
    code = torch.zeros_like(mag, dtype=torch.uint8)
    code = torch.where(mag > 0.25, torch.ones_like(code), code)        # 0.25 -> 0 (even)
    code = torch.where(mag >= 0.75, torch.full_like(code, 2), code)    # 0.75 -> 1.0 (code 2)
    code = torch.where(mag > 1.25, torch.full_like(code, 3), code)     # 1.25 -> 1.0 (code 2)
    code = torch.where(mag >= 1.75, torch.full_like(code, 4), code)    # 1.75 -> 2.0 (code 4)
    code = torch.where(mag > 2.5, torch.full_like(code, 5), code)      # 2.5  -> 2.0 (code 4)
    code = torch.where(mag >= 3.5, torch.full_like(code, 6), code)     # 3.5  -> 4.0 (code 6)
    code = torch.where(mag > 5.0, torch.full_like(code, 7), code)      # 5.0  -> 4.0 (code 6)
    sign = (torch.signbit(x)).to(torch.uint8) << 3
    return code | sign


def _mx_exponent(amax: torch.Tensor, emax_elem: int) -> torch.Tensor:
    """OCP MX shared exponent: floor(log2(amax)) - emax_elem, as an E8M0 byte (bias 127)."""
    amax = amax.clamp_min(2.0 ** -100)
    e = torch.floor(torch.log2(amax)) - emax_elem
    return (e + 127).clamp(0, 254).to(torch.uint8)


def _e8m0_to_float(b: torch.Tensor) -> torch.Tensor:
    return torch.exp2(b.float() - 127.0)


def quantize_tokens(x: torch.Tensor, fmt: str, mode: str, scale: Optional[torch.Tensor] = None):
    """Host statement of the cache write recipe for token-major input ``x [n, H, D]`` (fp32):
    returns (codes uint8 ``[n, H, D]`` or packed ``[n, H, D/2]``, scale).  Per token:
    ``scale = max(amax/448, 1e-8)``; E8M0: ``floor(log2(amax_block)) - emax`` per 32-element block;
    per head: the given ``scale [H]``."""
    n, h, d = x.shape
    x = x.float()
    if mode == SCALE_PER_TOKEN:
        sc = (x.abs().amax(dim=2) / E4M3_MAX).clamp_min(1e-8)               # [n,H]
        return quant_e4m3(x / sc.unsqueeze(-1)), sc
    if mode == SCALE_PER_HEAD:
        return quant_e4m3(x / scale.view(1, h, 1)), scale
    if mode == SCALE_MX_E8M0:
        xb = x.view(n, h, d // 32, 32)
        eb = _mx_exponent(xb.abs().amax(dim=3), 8 if fmt == KV_FP8_E4M3 else 2)   # [n,H,D/32]
        y = xb / _e8m0_to_float(eb).unsqueeze(-1)
        if fmt == KV_FP8_E4M3:
            return quant_e4m3(y.clamp(-E4M3_MAX, E4M3_MAX)).view(n, h, d), eb
        c = quant_e2m1(y).view(n, h, d // 2, 2)
        return (c[..., 0] | (c[..., 1] << 4)).contiguous(), eb
    raise ValueError(mode)


# --------------------------------------------------------------------------------------
# Workload builder
# --------------------------------------------------------------------------------------
def build_workload(name: str, *, context_lens: Sequence[int], q_lens: Optional[Sequence[int]],
                   num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                   q_dtype: torch.dtype, k_format: str = KV_FP8_E4M3, v_format: str = KV_FP8_E4M3,
                   scale_mode: str = SCALE_PER_TOKEN, pool_factor: float = 1.0,
                   mx_exponent_range: Optional[tuple] = None, seed: int = 0,
                   device="cpu", poison: bool = True, max_blocks: Optional[int] = None,
                   softmax_scale: Optional[float] = None, cache_dtype=None) -> DecodeWorkload:
    """Build caches directly in paged form.  The value of every (page, head, d, token) cell is
    drawn i.i.d. N(0,1) and quantised in place, so the cost is one pass over the pool."""
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    ctx = [int(c) for c in context_lens]
    S = len(ctx)
    pages_per_seq = [(max(c, 0) + page_size - 1) // page_size for c in ctx]
    needed = sum(pages_per_seq)
    pool = max(1, int(math.ceil(pool_factor * needed)))
    perm = torch.randperm(pool, generator=g, device=dev)[:needed]
    mb = max(1, max(pages_per_seq) if pages_per_seq else 1) if max_blocks is None else max_blocks
    bt = torch.zeros(S, mb, dtype=torch.int32, device=dev)
    valid = torch.zeros(pool, page_size, dtype=torch.bool, device=dev)   # token slots in use
    off = 0
    for s in range(S):
        n = pages_per_seq[s]
        if n:
            rows = perm[off:off + n]
            bt[s, :n] = rows.to(torch.int32)
            valid[rows] = True
            tail = n * page_size - ctx[s]
            if tail:
                valid[rows[-1], page_size - tail:] = False
        off += n

    D, P, H = head_dim, page_size, num_kv_heads

    def draw():
        return torch.randn(pool, H, D, P, generator=g, device=dev, dtype=torch.float32)

    def quantise(x, fmt, mode):
        """x: [pool,H,D,P] fp32 -> (payload uint8, scale tensor or None)"""
        if mode == SCALE_NONE:
            return x.to(cache_dtype or torch.float16), None
        if mode == SCALE_PER_HEAD:
            # reference recipe: amax over everything but the head (tests/test_kernels_misc.py:51)
            sc = (x.abs().amax(dim=(0, 2, 3)) / E4M3_MAX).clamp_min(1e-8)
            return quant_e4m3(x / sc.view(1, H, 1, 1)), sc
        if mode == SCALE_PER_BLOCK:
            sc = (x.abs().amax(dim=(2, 3)) / E4M3_MAX).clamp_min(1e-8)
            return quant_e4m3(x / sc.view(pool, H, 1, 1)), sc
        if mode == SCALE_PER_TOKEN:
            sc = (x.abs().amax(dim=2) / E4M3_MAX).clamp_min(1e-8)           # [pool,H,P]
            return quant_e4m3(x / sc.view(pool, H, 1, P)), sc
        if mode == SCALE_MX_E8M0:
            xb = x.view(pool, H, D // 32, 32, P)
            if mx_exponent_range is not None and fmt == KV_FP8_E4M3:
                lo, hi = mx_exponent_range
                eb = torch.randint(lo + 127, hi + 128, (pool, H, D // 32, P), generator=g,
                                   device=dev).to(torch.uint8)
            else:
                emax = 8 if fmt == KV_FP8_E4M3 else 2
                eb = _mx_exponent(xb.abs().amax(dim=3), emax)
            y = xb / _e8m0_to_float(eb).unsqueeze(3)
            if fmt == KV_FP8_E4M3:
                payload = quant_e4m3(y.clamp(-E4M3_MAX, E4M3_MAX)).view(pool, H, D, P)
            else:
                c = quant_e2m1(y).view(pool, H, D // 2, 2, P)
                payload = (c[:, :, :, 0] | (c[:, :, :, 1] << 4)).contiguous()
            return payload, eb
        raise ValueError(mode)

    k_mode = scale_mode
    v_mode = scale_mode
    kc, ks = quantise(draw(), k_format, k_mode)
    vc, vs = quantise(draw(), v_format, v_mode)

    if poison and scale_mode != SCALE_NONE:
        inval = ~valid                                                       # [pool,P]
        m = inval.view(pool, 1, 1, P)
        kc = torch.where(m, torch.full_like(kc, POISON_E4M3), kc)
        vc = torch.where(m, torch.full_like(vc, POISON_E4M3), vc)
        if scale_mode == SCALE_PER_TOKEN:
            nan = torch.full_like(ks, float("nan"))
            ks = torch.where(inval.view(pool, 1, P), nan, ks)
            vs = torch.where(inval.view(pool, 1, P), nan, vs)
        elif scale_mode == SCALE_MX_E8M0:
            ks = torch.where(m, torch.full_like(ks, POISON_E8M0), ks)
            vs = torch.where(m, torch.full_like(vs, POISON_E8M0), vs)

    if q_lens is None:
        total_q, cu, max_q = S, None, 1
    else:
        ql = [int(x) for x in q_lens]
        total_q, max_q = sum(ql), max(ql) if ql else 1
        cu = torch.tensor([0] + list(torch.tensor(ql).cumsum(0).tolist()), dtype=torch.int32,
                          device=dev)
    q = torch.randn(total_q, num_q_heads, D, generator=g, device=dev, dtype=torch.float32).to(q_dtype)
    return DecodeWorkload(
        name=name, query=q, key_cache=kc.contiguous(), value_cache=vc.contiguous(),
        k_scale=ks, v_scale=vs, block_tables=bt,
        context_lens=torch.tensor(ctx, dtype=torch.int32, device=dev), cu_q_lens=cu,
        page_size=P, head_dim=D, num_q_heads=num_q_heads, num_kv_heads=H,
        k_format=k_format, v_format=v_format, k_scale_mode=k_mode, v_scale_mode=v_mode,
        softmax_scale=(1.0 / math.sqrt(D)) if softmax_scale is None else softmax_scale,
        max_q_len=max_q, meta={"seed": seed, "pool_pages": pool, "needed_pages": needed})


# --------------------------------------------------------------------------------------
# The five named configurations (seed = 1000 + id)
# --------------------------------------------------------------------------------------
def _lognormal_lens(n, median, sigma, lo, hi, gen):
    z = torch.randn(n, generator=gen)
    return torch.exp(math.log(median) + sigma * z).round().clamp(lo, hi).to(torch.int64).tolist()


def make_config(config_id: int, device="cpu", *, batch: Optional[int] = None,
                ctx_scale: float = 1.0, seed: Optional[int] = None,
                poison: bool = True, head_shards: int = 1, len_seed: Optional[int] = None,
                deal: Optional[Tuple[int, int]] = None) -> DecodeWorkload:
    """The benchmark configurations.  ``batch`` / ``ctx_scale`` shrink a configuration for
    parity tests (same shapes and value distributions, fewer / shorter sequences);
    ``head_shards`` builds one KV-head shard (1/head_shards of the KV and query heads);
    ``len_seed`` fixes the length draw independently of the data seed (ranks of a sharded run
    share the lengths and differ in the data); ``deal = (world, rank)`` draws the lengths of the
    whole job (``batch`` sequences in total) and keeps the sequences that heaviest-first dealing
    (``sharding.shard_sequences``: by context length, for config 5 by context length times the row
    weight of the query length) gives to ``rank``."""
    seed = 1000 + config_id if seed is None else seed
    cg = torch.Generator()
    cg.manual_seed(seed if len_seed is None else len_seed)
    hs = head_shards
    sc = lambda x: max(1, int(round(x * ctx_scale)))

    def dealt(lens, *extras, weights=None):
        if deal is None:
            return (lens,) + extras
        from .sharding import shard_sequences
        ids = shard_sequences(lens, deal[0], weights)[deal[1]]
        return tuple([x[i] for i in ids] for x in (lens,) + extras)

    if config_id == 1:
        b = batch or 4
        return build_workload("cfg1_mha_perhead_d64", context_lens=[sc(512)] * b, q_lens=None,
                              num_q_heads=8, num_kv_heads=8, head_dim=64, page_size=16,
                              q_dtype=torch.float32, scale_mode=SCALE_PER_HEAD, pool_factor=1.0,
                              seed=seed, device=device, poison=poison)
    if config_id == 2:
        b = batch or 64
        lens = torch.randint(sc(1024), sc(8192) + 1, (b,), generator=cg).tolist()
        (lens,) = dealt(lens)
        return build_workload("cfg2_llama8b_fp8_pertoken", context_lens=lens, q_lens=None,
                              num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16,
                              q_dtype=torch.bfloat16, scale_mode=SCALE_PER_TOKEN, pool_factor=1.25,
                              seed=seed, device=device, poison=poison)
    if config_id == 3:
        b = batch or 128
        lens = _lognormal_lens(b, 4096 * ctx_scale, 1.0, sc(256), sc(32768), cg)
        return build_workload("cfg3_llama70b_mxfp8", context_lens=lens, q_lens=None,
                              num_q_heads=64 // hs, num_kv_heads=8 // hs, head_dim=128, page_size=32,
                              q_dtype=torch.bfloat16, scale_mode=SCALE_MX_E8M0, pool_factor=1.0,
                              mx_exponent_range=(-4, 4), seed=seed, device=device, poison=poison)
    if config_id == 4:
        b = batch or 2
        return build_workload("cfg4_long_context", context_lens=[sc(131072)] * b, q_lens=None,
                              num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=64,
                              q_dtype=torch.bfloat16, scale_mode=SCALE_PER_TOKEN, pool_factor=1.0,
                              seed=seed, device=device, poison=poison)
    if config_id == 5:
        b = batch or 256
        lens = _lognormal_lens(b, 2048 * ctx_scale, 1.0, max(4, sc(16)), sc(16384), cg)
        ql = torch.where(torch.rand(b, generator=cg) < 0.7, 1, 4).tolist()
        ql = [min(q, l) for q, l in zip(ql, lens)]
        from .sharding import decode_cost_weights
        lens, ql = dealt(lens, ql, weights=decode_cost_weights(lens, ql, 32 // 8))
        return build_workload("cfg5_continuous_batching_mx8k_mx4v", context_lens=lens, q_lens=ql,
                              num_q_heads=32, num_kv_heads=8, head_dim=128, page_size=16,
                              q_dtype=torch.bfloat16, k_format=KV_FP8_E4M3, v_format=KV_FP4_E2M1,
                              scale_mode=SCALE_MX_E8M0, pool_factor=1.5, seed=seed, device=device,
                              poison=poison)
    raise ValueError(f"unknown config {config_id}")
