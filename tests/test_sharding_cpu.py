"""Host logic of the multi-GPU layer on CPU ranks (gloo, world size 2): partition plans, workload
slicing, the all-gather + merge of the split-context mode.  The compute callables are replaced by
the oracle; nothing here touches a GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cuda_b200 import sharding as S, workloads as W
from helpers import to_oracle
from oracle import paged_decode_oracle as O


def test_shard_sequences_by_cost_weights():
    """With query lengths known, the work of a sequence is its context length times 2 where group * q_len exceeds
    8 rows: dealing by that weight balances the ranks' cost, dealing by length alone does not."""
    import random
    rnd = random.Random(3)
    lens = [rnd.randint(16, 16384) for _ in range(256)]
    qls = [1 if rnd.random() < 0.7 else 4 for _ in lens]
    w = S.decode_cost_weights(lens, qls, group=4)
    assert w[0] == lens[0] * (2 if qls[0] == 4 else 1)
    for world in (2, 4, 8):
        by_cost = S.shard_sequences(lens, world, w)
        assert sorted(i for p in by_cost for i in p) == list(range(256))
        loads = [sum(w[i] for i in p) for p in by_cost]
        assert max(loads) <= 1.01 * sum(loads) / world
        by_len = [sum(w[i] for i in p) for p in S.shard_sequences(lens, world)]
        assert max(loads) <= max(by_len)
    assert S.decode_cost_weights([5, 7], None, 4) == [5.0, 7.0]


def test_shard_sequences_balances_and_covers():
    lens = [8192, 100, 4000, 4100, 50, 7000, 1, 0, 3000]
    for world in (1, 2, 4, 8):
        parts = S.shard_sequences(lens, world)
        assert sorted(s for p in parts for s in p) == list(range(len(lens)))
        loads = [sum(lens[s] for s in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)


def test_shard_kv_heads_and_context_ranges():
    assert [S.shard_kv_heads(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        S.shard_kv_heads(8, 3, 0)
    for ctx in (0, 1, 63, 64, 65, 1000, 131072):
        for world in (1, 2, 4, 8):
            rng = [S.split_context(ctx, world, r, 64) for r in range(world)]
            assert rng[0][0] == 0 and rng[-1][1] == ctx
            for (b0, e0), (b1, e1) in zip(rng, rng[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 64 == 0 for b, _ in rng)


def _oracle_partial(wl):
    return O.ref_paged_decode(wl.query, to_oracle(wl), wl.softmax_scale, return_lse=True)


def _oracle_merge(parts_out, parts_lse, dtype):
    return O.merge_partials(parts_out, parts_lse)[0].to(dtype)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = W.build_workload("ctx", context_lens=[300, 64, 1, 129], q_lens=None, num_q_heads=8, num_kv_heads=2,
                              head_dim=64, page_size=16, q_dtype=torch.float32, scale_mode=W.SCALE_PER_TOKEN,
                              pool_factor=1.3, seed=7)
        full = O.ref_paged_decode(wl.query, to_oracle(wl), wl.softmax_scale)
        # (1) split-context: local partial -> all_gather -> merge
        local = S.slice_context(wl, world, rank)
        out = S.decode_split_context(local, partial_fn=_oracle_partial, merge_fn=_oracle_merge)
        err_ctx = (out - full).abs().max().item()
        # (2) KV-head sharding: final rows of the local heads, concatenated for the check
        lo, hi = S.shard_kv_heads(wl.num_kv_heads, world, rank)
        lw = S.slice_kv_heads(wl, lo, hi)
        lout = O.ref_paged_decode(lw.query, to_oracle(lw), lw.softmax_scale)
        err_head = (S.gather_head_shards(lout) - full).abs().max().item()
        # (3) sequence sharding: no collective; each rank checks its own rows
        ids = S.shard_sequences(wl.context_lens.tolist(), world)[rank]
        sw = S.slice_sequences(wl, ids)
        sout = O.ref_paged_decode(sw.query, to_oracle(sw), sw.softmax_scale)
        err_seq = (sout - full[ids]).abs().max().item() if ids else 0.0
        q.put((rank, err_ctx, err_head, err_seq))
    except Exception as e:                      # report instead of leaving the parent to time out
        q.put((rank, repr(e), None, None))
        raise
    finally:
        dist.destroy_process_group()


def test_world2_gloo_all_modes():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, e_ctx, e_head, e_seq in res:
        assert not isinstance(e_ctx, str), e_ctx
        assert e_ctx < 1e-5 and e_head < 1e-5 and e_seq < 1e-6, (rank, e_ctx, e_head, e_seq)
