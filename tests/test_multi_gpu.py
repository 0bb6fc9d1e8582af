"""Two NCCL ranks on two GPUs: the split-context mode (local partial, all-gather over NVLink, merge
kernel; from Python and from the single C++ entry point) and KV-head sharding against the oracle.  Skipped on a box with one GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from cuda_b200 import sharding as S, workloads as W
    from helpers import oracle_out
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        wl = W.make_config(4, batch=2, ctx_scale=1 / 64)           # 2 x 2048 tokens, page 64
        ref = oracle_out(wl)
        g = wl.to(f"cuda:{rank}")
        local = S.slice_context(g, world, rank)
        out = S.decode_split_context(local)
        e_ctx = (out.float().cpu() - ref).abs()
        # the same exchange issued from one C++ call (decode, one ncclAllGather, merge)
        dec = S.SplitContextDecoder(local)
        for _ in range(3):
            fused = dec(local, check_status=True)
        e_ctx = torch.maximum(e_ctx, (fused.float().cpu() - ref).abs())
        lo, hi = S.shard_kv_heads(wl.num_kv_heads, world, rank)
        from cuda_b200 import ops
        lout = ops.run_workload(S.slice_kv_heads(g, lo, hi))
        e_head = (S.gather_head_shards(lout).float().cpu() - ref).abs()
        torch.cuda.synchronize()
        q.put((rank, e_ctx.max().item(), e_ctx.mean().item(), e_head.max().item(), e_head.mean().item()))
    except Exception as e:
        q.put((rank, repr(e), 0, 0, 0))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_split_context_and_head_shards():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, mx_c, mean_c, mx_h, mean_h in res:
        assert not isinstance(mx_c, str), mx_c
        assert mx_c <= 2e-2 and mean_c <= 2e-3 and mx_h <= 2e-2 and mean_h <= 2e-3, res
