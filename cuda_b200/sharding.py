"""Multi-GPU layer of the decode path: one process per GPU (torch.distributed).

The reference has no distributed code at all; this layer exists because decode attention shards
naturally in three ways:

* by sequence   (batched decode): independent, no collective;
* by KV head    (tensor-parallel style): every rank owns ``Hkv / world`` KV heads of every page and
  the matching query heads; independent, the per-rank outputs are the final rows of their heads;
* by KV range   (one long context): every rank owns a page-aligned token range, computes a
  partial ``(out, lse)`` over it, the partials are all-gathered (NCCL over NVLink when the group
  is an NCCL group) and merged with ``combine_softmax_state``'s algebra
  (``fused_online_softmax_kernel.cuh:40-49`` in the reference project).

The compute callables are parameters so that the host logic can be exercised on CPU ranks (gloo)
with a stand-in; their defaults are the CUDA ops, and there is no CPU fallback inside them.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .workloads import DecodeWorkload, SCALE_NONE, SCALE_PER_HEAD


# --------------------------------------------------------------------------------------
# partition plans (pure integer logic)
# --------------------------------------------------------------------------------------
def shard_sequences(context_lens: Sequence[int], world: int,
                    weights: Optional[Sequence[float]] = None) -> List[List[int]]:
    """Deal sequences to ``world`` ranks, heaviest first onto the least loaded rank (LPT), so that
    every rank has about the same work.  The work of a sequence is its context length (the KV bytes it
    streams), or ``weights[s]`` where the caller knows better: the 8-bit decode kernel computes every
    stage of a sequence with more than 8 query rows per KV head twice (one row half per warp of a pair),
    so a router that knows the query lengths passes ``context_len * (2 if group * q_len > 8 else 1)``.
    Returns the sequence ids per rank, each list in ascending order."""
    cost = [max(float(w), 0.0) for w in (context_lens if weights is None else weights)]
    if len(cost) != len(context_lens):
        raise ValueError("weights must have one entry per sequence")
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for s in sorted(range(len(cost)), key=lambda i: (-cost[i], i)):
        r = min(range(world), key=lambda i: (loads[i], i))
        out[r].append(s)
        loads[r] += cost[s]
    return [sorted(x) for x in out]


def decode_cost_weights(context_lens: Sequence[int], q_lens: Optional[Sequence[int]], group: int) -> List[float]:
    """Work of each sequence for ``shard_sequences``: its context length, doubled where ``group * q_len``
    exceeds the 8 rows one warp of the decode kernel handles."""
    if q_lens is None:
        return [float(max(int(c), 0)) for c in context_lens]
    return [float(max(int(c), 0)) * (2.0 if group * int(q) > 8 else 1.0) for c, q in zip(context_lens, q_lens)]


def shard_kv_heads(num_kv_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """KV heads ``[lo, hi)`` of ``rank``; ``num_kv_heads`` must be a multiple of ``world``."""
    if num_kv_heads % world:
        raise ValueError("num_kv_heads must be a multiple of the number of ranks")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def split_context(ctx: int, world: int, rank: int, page_size: int) -> Tuple[int, int]:
    """Token range ``[begin, end)`` of ``rank`` for a context of ``ctx`` tokens: whole pages,
    spread as evenly as pages allow; ranks past the end get an empty range."""
    pages = (max(ctx, 0) + page_size - 1) // page_size
    lo = (pages * rank) // world
    hi = (pages * (rank + 1)) // world
    return min(lo * page_size, ctx), min(hi * page_size, ctx)


# --------------------------------------------------------------------------------------
# slicing a workload (tests and the benchmark build per-rank inputs with these)
# --------------------------------------------------------------------------------------
def slice_sequences(wl: DecodeWorkload, seq_ids: Sequence[int]) -> DecodeWorkload:
    ids = torch.as_tensor(list(seq_ids), dtype=torch.long, device=wl.context_lens.device)
    if wl.cu_q_lens is None:
        q = wl.query[ids]
        cu = None
    else:
        cu_all = wl.cu_q_lens.tolist()
        rows = [r for s in seq_ids for r in range(cu_all[s], cu_all[s + 1])]
        q = wl.query[torch.as_tensor(rows, dtype=torch.long, device=wl.query.device)]
        lens = [cu_all[s + 1] - cu_all[s] for s in seq_ids]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32,
                          device=wl.context_lens.device)
    return dataclasses.replace(wl, query=q.contiguous(), block_tables=wl.block_tables[ids].contiguous(),
                               context_lens=wl.context_lens[ids].contiguous(), cu_q_lens=cu)


def slice_kv_heads(wl: DecodeWorkload, lo: int, hi: int) -> DecodeWorkload:
    g = wl.num_q_heads // wl.num_kv_heads

    def sl(scale, mode):
        if scale is None or mode == SCALE_NONE:
            return scale
        if mode == SCALE_PER_HEAD:
            return scale[lo:hi].contiguous()
        return scale[:, lo:hi].contiguous()

    return dataclasses.replace(
        wl, query=wl.query[:, lo * g:hi * g].contiguous(), key_cache=wl.key_cache[:, lo:hi].contiguous(),
        value_cache=wl.value_cache[:, lo:hi].contiguous(), k_scale=sl(wl.k_scale, wl.k_scale_mode),
        v_scale=sl(wl.v_scale, wl.v_scale_mode), num_q_heads=(hi - lo) * g, num_kv_heads=hi - lo)


def slice_context(wl: DecodeWorkload, world: int, rank: int) -> DecodeWorkload:
    """The page-aligned KV range of ``rank`` for every sequence (q_len 1 only: a verify window
    would need absolute positions).  The page pool is shared; only tables and lengths change."""
    if wl.cu_q_lens is not None:
        raise ValueError("split-context mode supports q_len == 1")
    ctx = wl.context_lens.tolist()
    rng = [split_context(c, world, rank, wl.page_size) for c in ctx]
    width = max(1, max((e - b + wl.page_size - 1) // wl.page_size for b, e in rng))
    bt = torch.zeros(len(ctx), width, dtype=torch.int32, device=wl.block_tables.device)
    for s, (b, e) in enumerate(rng):
        n = (e - b + wl.page_size - 1) // wl.page_size
        if n:
            p0 = b // wl.page_size
            bt[s, :n] = wl.block_tables[s, p0:p0 + n]
    lens = torch.tensor([e - b for b, e in rng], dtype=torch.int32, device=wl.context_lens.device)
    return dataclasses.replace(wl, block_tables=bt, context_lens=lens)


# --------------------------------------------------------------------------------------
# split-context decode: local partial -> all-gather -> merge
# --------------------------------------------------------------------------------------
def _cuda_partial(wl: DecodeWorkload):
    from . import ops
    out = torch.empty(wl.query.shape, dtype=torch.float32, device=wl.query.device)
    return ops.run_workload(wl, return_lse=True, out=out)


def _cuda_merge(parts_out, parts_lse, out_dtype):
    from . import ops
    return ops.merge_partials(parts_out, parts_lse, out_dtype=out_dtype)


def decode_split_context(local: DecodeWorkload, group: Optional[dist.ProcessGroup] = None,
                         partial_fn: Callable = _cuda_partial, merge_fn: Callable = _cuda_merge,
                         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Every rank calls this with the workload restricted to ITS KV range (``slice_context``).
    Returns the full attention output on every rank.

    The exchange is an all-gather of ``[total_q, Hq, D]`` fp32 plus ``[total_q, Hq]`` log-sum-exps
    per rank, issued on the current stream right after the local kernel; the merge kernel follows
    on the same stream and reads the gathered partials from local HBM."""
    world = dist.get_world_size(group)
    out, lse = partial_fn(local)                                   # [T,Hq,D] fp32, [T,Hq] natural log
    out, lse = out.float().contiguous(), lse.float().contiguous()
    g_out = torch.empty((world,) + tuple(out.shape), dtype=torch.float32, device=out.device)
    g_lse = torch.empty((world,) + tuple(lse.shape), dtype=torch.float32, device=out.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(g_out, out, group=group)
        dist.all_gather_into_tensor(g_lse, lse, group=group)
    else:                                                          # gloo (CPU ranks in the tests)
        dist.all_gather(list(g_out.unbind(0)), out, group=group)
        dist.all_gather(list(g_lse.unbind(0)), lse, group=group)
    return merge_fn(g_out, g_lse, out_dtype or local.query.dtype)


class SplitContextDecoder:
    """Split-context decode with everything issued from one C++ call per step
    (``cuda_llm_split_context_decode``): local partial, ONE NCCL all-gather of the fp32 (out | lse)
    blocks, merge.  The exchange buffer, the output and the workspace are allocated once here and
    reused by every call, so a step allocates nothing and runs no Python between the kernels."""

    def __init__(self, local: DecodeWorkload, group: Optional[dist.ProcessGroup] = None):
        from . import ops
        self.ops = ops
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = local.query.device
        if self.world > 1:
            if dist.get_backend(group) != "nccl":
                raise RuntimeError("SplitContextDecoder needs an NCCL group (CPU ranks use decode_split_context)")
            dist.barrier(group)                       # makes sure the communicator exists on this device
            self.comm = ops.nccl_comm_ptr(group, dev)
        else:
            self.comm = None
        rows = local.query.shape[0] * local.num_q_heads
        self.exchange = ops.split_context_exchange(rows, local.head_dim, self.world, dev)
        self.out = torch.empty_like(local.query)
        need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(
            local.num_seqs, local.num_q_heads, local.num_kv_heads, local.head_dim, local.page_size, 1, 0)
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)

    def __call__(self, local: DecodeWorkload, flags: int = 0, check_status: bool = False) -> torch.Tensor:
        return self.ops.run_workload(local, out=self.out, workspace=self.workspace, flags=flags,
                                     check_status=check_status,
                                     split_context=(self.comm, self.world, self.rank, self.exchange))


def gather_head_shards(local_out: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """KV-head sharding produces final rows for a slice of the query heads; this concatenates the
    slices (checking / a consumer that needs the full tensor).  Not on the attention data path."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)
