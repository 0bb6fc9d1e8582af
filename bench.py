"""Benchmark of the paged FP8 decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]
                    [--no-extra-workloads]

One step = one decode-attention pass over one batch of the workload (default: the
Llama-3-8B-shaped FP8 paged decode configuration: batch 64, 32/8 heads, head_dim 128, page 16,
context lengths U[1024, 8192], per-(token, KV-head) fp32 scales, pool 1.25x).  The metric is
HBM throughput on the algorithmic K+V bytes (payload + scales of valid tokens only), the
reference benchmark's own "effective KV GB/s" (benchmark_pytorch.py:160,611 in the reference
project).  With N > 1 (torchrun, one rank per GPU) every rank holds its own batch (sequence
sharding, no collective on the data path): weak scaling, value = all ranks' bytes / max time.

After the headline workload the same ranks also time the other three sharded configurations
(MXFP8 by KV-head shards, the long context by KV ranges with an NCCL all-gather and a merge, the
continuous-batching mix by sequence shards; total work fixed, i.e. strong scaling) and report them
under "workloads" in the same line, each with a parity figure of a sampled sequence against the
CPU oracle.  Every timed loop is repeated until at least 200 ms have been measured; the numbers
are medians over the repeats.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {"cfg1": 1, "cfg2": 2, "cfg3": 3, "cfg4": 4, "cfg5": 5}
# secondary lines for the unquantised entry points (same Llama-3-8B head shape, bf16 K/V)
AUX_WORKLOADS = ("pa16", "pa32", "fd16", "fd32", "prefill", "mxattn", "kvappend")
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic KV bytes of one decode-kernel launch,
# from an ncu capture of a batch-16 launch of the same workload (traffic grows with the bytes
# streamed, so the ratio carries over to the full-size launch)
DRAM_TRAFFIC_PER_KV_BYTE = {"cfg2_llama8b_fp8_pertoken": 1.03}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                               f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_reference_run(wl_cpu, budget_s: float, max_seqs=None):
    """Time the CPU restatement of the reference's PyTorch path (per sequence: gather pages
    through the block table, dequantise, scaled-dot-product attention) on the host cores.
    Returns (seconds, kv_bytes_processed, tokens, n_seqs, max_abs_vs_none)."""
    from oracle import paged_decode_oracle as O
    from cuda_b200.workloads import bytes_per_token_head
    kv = O.PagedKV(wl_cpu.key_cache, wl_cpu.value_cache, wl_cpu.block_tables, wl_cpu.context_lens,
                   wl_cpu.page_size, wl_cpu.head_dim, wl_cpu.k_format, wl_cpu.v_format,
                   wl_cpu.k_scale_mode, wl_cpu.v_scale_mode, wl_cpu.k_scale, wl_cpu.v_scale)
    per = (bytes_per_token_head(wl_cpu.head_dim, wl_cpu.k_format, wl_cpu.k_scale_mode)
           + bytes_per_token_head(wl_cpu.head_dim, wl_cpu.v_format, wl_cpu.v_scale_mode)) * wl_cpu.num_kv_heads
    S = wl_cpu.num_seqs if max_seqs is None else min(max_seqs, wl_cpu.num_seqs)
    cu = list(range(S + 1)) if wl_cpu.cu_q_lens is None else wl_cpu.cu_q_lens.tolist()
    t0 = time.perf_counter()
    done, nbytes, qtok = 0, 0, 0
    # whole passes over the batch until about two thirds of the budget is used (at least one pass,
    # cut short inside a pass when the budget runs out)
    for s in (i % S for i in range(S * 10000)):
        if s == 0 and done >= S and time.perf_counter() - t0 > 0.66 * budget_s:
            break
        sub = O.PagedKV(kv.key_cache, kv.value_cache, kv.block_tables[s:s + 1], kv.context_lens[s:s + 1],
                        kv.page_size, kv.head_dim, kv.k_format, kv.v_format, kv.k_scale_mode,
                        kv.v_scale_mode, kv.k_scale, kv.v_scale)
        q = wl_cpu.query[cu[s]:cu[s + 1]]
        if q.shape[0] == 1:
            O.ref_paged_decode_sdpa(q, sub, wl_cpu.softmax_scale)
        else:
            O.ref_paged_decode(q, sub, wl_cpu.softmax_scale,
                               torch.tensor([0, q.shape[0]], dtype=torch.int32))
        done += 1
        nbytes += int(wl_cpu.context_lens[s]) * per
        qtok += q.shape[0]
        if time.perf_counter() - t0 > budget_s:
            break
    return time.perf_counter() - t0, nbytes, qtok, done


def aux_workload(args, rank, world, local):
    """paged_attention (pa16) / async_flash_decode (fd16) over a bf16 cache, 32 query / 8 KV heads,
    head_dim 128, batch 64 per GPU: kernel + merge timed with CUDA events, one JSON line."""
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm covers the FP8 configurations only"}))
        return
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from cuda_b200 import ops, workloads
    batch = args.batch or 64
    g = torch.Generator().manual_seed(2000 + rank)
    if args.workload in ("prefill", "mxattn"):
        # GQA prefill over a whole prompt (fused_gqa_forward) / dense attention over microscaled FP8 tensors:
        # Llama-3-8B head shape, causal; tensor-core bound, so the roofline is the measured bf16 GEMM rate
        bsz, seq = args.batch or 4, int(4096 * args.ctx_scale)
        flops = 4.0 * bsz * 32 * seq * seq * 128 / 2            # causal: half of the score matrix
        if args.workload == "prefill":
            q = torch.randn(bsz, 32, seq, 128, generator=g).to(torch.bfloat16).to(dev)
            k = torch.randn(bsz, 8, seq, 128, generator=g).to(torch.bfloat16).to(dev)
            v = torch.randn(bsz, 8, seq, 128, generator=g).to(torch.bfloat16).to(dev)
            fn = lambda: ops.fused_gqa_forward(q, k, v, is_causal=True)
        else:
            mk = lambda h: (torch.randint(0, 0x7E, (bsz, h, seq, 128), generator=g, dtype=torch.uint8).to(dev),
                            (torch.rand(bsz, h, seq, 4, generator=g) * 0.01 + 0.001).to(dev))
            (q, qs), (k, ks), (v, vs) = mk(32), mk(8), mk(8)
            fn = lambda: ops.fused_microscaled_attention(q, qs, k, ks, v, vs, is_causal=True)
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        steps = min(args.steps, 50)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        tf_peak = None
        try:
            tf_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        except Exception:
            pass
        tf = flops / (ms * 1e-3) / 1e12
        if rank == 0:
            print(json.dumps({"metric": f"{args.workload}_attention_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
                              "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                              "dtype": ("bf16 mma.sync, f32 acc" if os.environ.get("CUDA_LLM_PREFILL_KERNEL") == "warp_mma"
                                        else "bf16 tcgen05.mma, f32 acc in TMEM") if args.workload == "prefill"
                                       else "e4m3 -> f16 (one rounding) -> tcgen05.mma, f32 acc",
                              "data": "synthetic",
                              "config": {"workload": args.workload, "batch": bsz, "heads": "32q/8kv", "seq_len": seq,
                                         "head_dim": 128, "causal": True},
                              "roofline": {"bound": "tensor", "achieved": tf, "peak": tf_peak or 1400.0,
                                           "unit": "TFLOP/s", "frac": tf / (tf_peak or 1400.0),
                                           "peak_source": "measured (sustained cuBLAS bf16)" if tf_peak else "fallback",
                                           "kernel": "gqa_prefill_sm100_kernel" if (args.workload == "prefill" and os.environ.get("CUDA_LLM_PREFILL_KERNEL") != "warp_mma") else "gqa_prefill_kernel",
                                           "traffic": None},
                              "gpu_launches": steps}), flush=True)
        return
    if args.workload == "kvappend":
        # quantise-and-store of new K/V tokens into the paged cache (the step in front of the decode path):
        # a prefill's worth of tokens [n, Hkv, D] bf16 -> E4M3 codes + per-token fp32 scales, pages of 16 tokens
        # in a shuffled pool, every sequence page-aligned
        n_seq = args.batch or 8                     # 8 x 4096 tokens: 134 MB in, 69 MB out, larger than L2
        seq = int(4096 * args.ctx_scale)
        n, hkv, d, page = n_seq * seq, 8, 128, 16
        k_new = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16).to(dev)
        v_new = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16).to(dev)
        pages = n_seq * ((seq + page - 1) // page)
        perm = torch.randperm(pages, generator=g).to(torch.int32)
        tok = torch.arange(n)
        page_of = (tok // seq) * ((seq + page - 1) // page) + (tok % seq) // page
        slot_block = perm[page_of].to(torch.int32).to(dev)
        slot_offset = ((tok % seq) % page).to(torch.int32).to(dev)
        kc = torch.zeros(pages, hkv, d, page, dtype=torch.uint8, device=dev)
        vc = torch.zeros_like(kc)
        ksc = torch.zeros(pages, hkv, page, dtype=torch.float32, device=dev)
        vsc = torch.zeros_like(ksc)
        fn = lambda: ops.kv_cache_append(k_new, v_new, slot_block, slot_offset, kc, vc, ksc, vsc)
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        peak, peak_src = measured_peak()
        moved = 2 * n * hkv * (d * 2 + d + 4)   # bf16 in, one code byte per element and one fp32 scale per token out
        if rank == 0:
            print(json.dumps({"metric": "kv_append_hbm_throughput", "value": moved / (ms * 1e-3) / 1e12, "unit": "TB/s",
                              "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                              "higher_is_better": True, "dtype": "bf16 -> e4m3 + f32 scale", "data": "synthetic",
                              "config": {"workload": "kvappend_prefill_llama8b", "tokens": n, "kv_heads": hkv, "head_dim": d,
                                         "page_size": page, "bytes_moved": moved,
                                         "l2": "inputs of %d MB and outputs of %d MB per step, larger than L2 at the default size" % (4 * n * hkv * d // 2 ** 20, 2 * n * hkv * (d + 4) // 2 ** 20)},
                              "roofline": {"bound": "hbm", "achieved": moved / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                           "frac": moved / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_src,
                                           "kernel": "kv_append_tile_kernel"},
                              "gpu_launches": args.steps}), flush=True)
        return
    if args.workload in ("pa16", "pa32"):  # paged_attention over a bf16 / an fp32 cache
        cdt = torch.bfloat16 if args.workload == "pa16" else torch.float32
        ctx = torch.randint(int(1024 * args.ctx_scale), int(4096 * args.ctx_scale) + 1, (batch,), generator=g).tolist()
        wl = workloads.build_workload("pa16_llama8b_bf16" if cdt == torch.bfloat16 else "pa32_llama8b_fp32",
                                      context_lens=ctx, q_lens=None, num_q_heads=32,
                                      num_kv_heads=8, head_dim=128, page_size=args.page_size, q_dtype=cdt,
                                      scale_mode="none", pool_factor=1.25, seed=2000 + rank,
                                      cache_dtype=cdt).to(dev)
        kv_bytes = sum(ctx) * 8 * 128 * 2 * (2 if cdt == torch.bfloat16 else 4)
        fn = lambda: ops.paged_attention_forward(wl.query, wl.key_cache, wl.value_cache, wl.block_tables,
                                                 wl.context_lens)
        cfg = {"workload": wl.name, "batch_per_gpu": batch, "kv_tokens_per_gpu": sum(ctx), "page_size": args.page_size}
    else:
        seq = int(2560 * args.ctx_scale)
        cdt = torch.float32 if args.workload == "fd32" else torch.bfloat16
        q = torch.randn(batch, 32, 1, 128, generator=g).to(cdt).to(dev)
        k = torch.randn(batch, 8, seq, 128, generator=g).to(cdt).to(dev)
        v = torch.randn(batch, 8, seq, 128, generator=g).to(cdt).to(dev)
        kv_bytes = 2 * k.numel() * k.element_size()
        fn = lambda: ops.async_flash_decode(q, k, v)
        cfg = {"workload": "fd32_llama8b_fp32" if cdt == torch.float32 else "fd16_llama8b_bf16", "batch_per_gpu": batch, "seq_len": seq}
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak, peak_src = measured_peak()
    cfg.update({"heads": "32q/8kv", "head_dim": 128, "kv_bytes_per_gpu": kv_bytes,
                "l2": "inputs larger than L2, no flush needed"})
    if rank != 0:
        return
    f32 = args.workload in ("pa32", "fd32")
    print(json.dumps({"metric": ("fp32" if f32 else "bf16") + "_decode_kv_hbm_throughput", "value": kv_bytes / (ms * 1e-3) / 1e12, "unit": "TB/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "higher_is_better": True, "dtype": "f32 SIMT" if f32 else "bf16 mma, f32 acc", "data": "synthetic", "config": cfg,
                      "roofline": {"bound": "hbm", "achieved": kv_bytes / (ms * 1e-3) / 1e9, "peak": peak,
                                   "unit": "GB/s", "frac": kv_bytes / (ms * 1e-3) / 1e9 / peak,
                                   "peak_source": peak_src,
                                   "kernel": "paged_f32_decode_kernel + merge_partials_kernel" if f32 else "paged_decode_kernel + merge_splits_kernel"},
                      "gpu_launches": 2 * args.steps}), flush=True)


MIN_TIMED_MS = 200.0


class Bench:
    """Device, process group and timing helpers shared by all legs of one run."""

    def __init__(self, args, rank, world, local):
        self.args, self.rank, self.world, self.local = args, rank, world, local
        self.dev = torch.device("cuda", local)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def timed_blocks(self, fn, steps, min_total_ms=None):
        """Time blocks of exactly `steps` calls (CUDA events on the launching stream, a barrier and a
        device synchronise on both sides of every block) until `min_total_ms` have been measured,
        three blocks at least; every block's time is the maximum over the ranks.  Returns the
        per-step milliseconds of every block."""
        if min_total_ms is None:
            min_total_ms = self.args.min_timed_ms
        blocks, total = [], 0.0
        while len(blocks) < 3 or (total < min_total_ms and len(blocks) < 400):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            ms = e0.elapsed_time(e1)
            if self.world > 1:                    # the ranks must agree on when to stop
                import torch.distributed as dist
                t = torch.tensor([ms], device=self.dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            blocks.append(ms / steps)
            total += ms
        return blocks

    def sum_over_ranks(self, *vals):
        if self.world == 1:
            return [float(v) for v in vals]
        import torch.distributed as dist
        t = torch.tensor([float(v) for v in vals], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t)
        return [float(x) for x in t.tolist()]


def median(xs):
    xs = sorted(xs)
    n = len(xs)
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def sample_parity(wl, out, kv_heads=None, want_partial=False):
    """Parity of ONE sequence of the workload (the one of median context length) against the CPU
    oracle: its pages are gathered through the block table, copied to the host and attended over in
    fp32.  `kv_heads` restricts the check to the first KV heads (a 131072-token context over all heads
    would cost the host tens of seconds).  Returns (max_abs, mean_abs, sequence, tokens) or, with
    `want_partial`, the oracle's (out, lse) and the matching rows of `out`."""
    from oracle import paged_decode_oracle as O
    ctx = wl.context_lens.tolist()
    order = sorted(range(len(ctx)), key=lambda i: (ctx[i], i))
    s = order[len(order) // 2]
    page = wl.page_size
    n = max(1, (ctx[s] + page - 1) // page)
    pages = wl.block_tables[s, :n].long()
    hk = wl.num_kv_heads if kv_heads is None else min(kv_heads, wl.num_kv_heads)
    group = wl.num_q_heads // wl.num_kv_heads

    def take(t, mode):
        if t is None:
            return None
        if mode == "per_head":
            return t[:hk].cpu()
        return t[pages][:, :hk].cpu()

    kv = O.PagedKV(wl.key_cache[pages][:, :hk].cpu(), wl.value_cache[pages][:, :hk].cpu(),
                   torch.arange(n, dtype=torch.int32).view(1, n), torch.tensor([ctx[s]], dtype=torch.int32),
                   page, wl.head_dim, wl.k_format, wl.v_format, wl.k_scale_mode, wl.v_scale_mode,
                   take(wl.k_scale, wl.k_scale_mode), take(wl.v_scale, wl.v_scale_mode))
    if wl.cu_q_lens is None:
        r0, r1, cu = s, s + 1, None
    else:
        c = wl.cu_q_lens.tolist()
        r0, r1 = c[s], c[s + 1]
        cu = torch.tensor([0, r1 - r0], dtype=torch.int32)
    q = wl.query[r0:r1, :hk * group].cpu()
    got = out[r0:r1, :hk * group].float().cpu()
    if want_partial:
        ro, rl = O.ref_paged_decode(q, kv, wl.softmax_scale, cu, return_lse=True)
        return ro, rl, got, s
    ref = O.ref_paged_decode(q, kv, wl.softmax_scale, cu)
    err = (got - ref).abs()
    return float(err.max()), float(err.mean()), s, ctx[s]


def parity_record(mx, mean, s, tokens, note=""):
    return {"max_abs": mx, "mean_abs": mean, "ok": bool(mx <= 2e-2 and mean <= 2e-3),
            "tolerance": "max-abs <= 2e-2, mean-abs <= 2e-3 (bf16 output)", "sequence": s, "tokens": tokens,
            "against": "CPU oracle (gather pages, dequantise, fp32 attention)" + note}


def build_leg(B, cfg_id, args, batch=None, ctx_scale=1.0):
    """The workload of configuration `cfg_id` as this rank sees it, and how it is sharded."""
    from cuda_b200 import workloads
    rank, world = B.rank, B.world
    seed = 1000 + cfg_id + 7919 * rank
    kw = dict(batch=batch, ctx_scale=ctx_scale, seed=seed, poison=False)
    scaling, split_ctx = "strong", False
    if cfg_id == 2:
        # weak scaling: the job holds `world` batches; every rank draws the same length list and
        # keeps the sequences the balancer deals to it (its own pages and tables, no collective)
        scaling = "weak"
        parallelism = f"sequence-sharded x{world}: {world} batches dealt longest-first by context length"
        if world > 1:
            kw.update(batch=(batch or 64) * world, len_seed=1002, deal=(world, rank))
    elif cfg_id == 3:
        parallelism = f"KV-head-sharded x{world} (no collective)"
        kw.update(head_shards=world, len_seed=1003)
    elif cfg_id == 4:
        parallelism = (f"KV-range-sharded x{world}: local decode, one NCCL all-gather of (out | lse), merge; "
                       "issued from one C++ call" if world > 1 else "single GPU: decode + split merge")
        kw.update(ctx_scale=ctx_scale / world, seed=1000 + cfg_id + 7919 * rank)
        split_ctx = world > 1
    elif cfg_id == 5:
        parallelism = (f"sequence-sharded x{world}, dealt heaviest-first by context length x row weight "
                       "(2 for more than 8 query rows per KV head; no collective)")
        if world > 1:
            kw.update(batch=(batch or 256), len_seed=1005, deal=(world, rank))
    else:
        parallelism = "replicas"
    wl = workloads.make_config(cfg_id, B.dev, **kw)
    if split_ctx:                                   # one query attends every rank's KV range
        import torch.distributed as dist
        dist.broadcast(wl.query, src=0)
    return wl, scaling, parallelism, split_ctx


def run_extra_leg(B, cfg_id, args):
    """Time one of the other configurations on the same ranks: resident step (decode + merge, and for
    the split context the all-gather) with CUDA events, median over repeats, plus a parity sample."""
    from cuda_b200 import ops, sharding
    wl, scaling, parallelism, split_ctx = build_leg(B, cfg_id, args)
    STABLE = ops.L.FLAG_STABLE_METADATA
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(
        wl.num_seqs, wl.num_q_heads, wl.num_kv_heads, wl.head_dim, wl.page_size, wl.max_q_len, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device=B.dev)
    out = torch.empty_like(wl.query)
    rec = {}
    if split_ctx:
        dec = sharding.SplitContextDecoder(wl)
        step = lambda: dec(wl, flags=STABLE)
        part = torch.empty(wl.query.shape, dtype=torch.float32, device=B.dev)
        local_only = lambda: ops.run_workload(wl, return_lse=True, out=part, workspace=ws, flags=STABLE)
    else:
        step = lambda: ops.run_workload(wl, out=out, workspace=ws, flags=STABLE)
        local_only = None
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    steps = max(5, min(args.steps, 100))
    ms = median(B.timed_blocks(step, steps))
    if local_only is not None:
        for _ in range(3):
            local_only()
        ms_local = median(B.timed_blocks(local_only, steps))
        rec["split_context_ms"] = {"local_decode_and_split_merge": ms_local, "all_gather_and_merge": ms - ms_local,
                                   "collective_share": (ms - ms_local) / ms,
                                   "all_gather_bytes_per_rank": wl.query.shape[0] * wl.num_q_heads * (wl.head_dim + 1) * 4}
    st = ops.decode_status(dec.workspace if split_ctx else ws)
    kv_bytes = wl.kv_bytes()
    tot_bytes, tot_q = B.sum_over_ranks(kv_bytes, wl.query.shape[0] if not split_ctx else
                                        (wl.query.shape[0] if B.rank == 0 else 0))
    # parity of one sampled sequence (per rank; the worst rank is reported)
    result = step()
    torch.cuda.synchronize()
    if split_ctx:
        import torch.distributed as dist
        ro, rl, got, s = sample_parity(wl, result, kv_heads=1, want_partial=True)
        po = [torch.empty_like(ro, device=B.dev) for _ in range(B.world)]
        pl = [torch.empty_like(rl, device=B.dev) for _ in range(B.world)]
        dist.all_gather(po, ro.to(B.dev))
        dist.all_gather(pl, rl.to(B.dev))
        from oracle import paged_decode_oracle as O
        ref, _ = O.merge_partials(torch.stack([x.cpu() for x in po]), torch.stack([x.cpu() for x in pl]))
        err = (got - ref).abs()
        mx, mean, tokens = float(err.max()), float(err.mean()), int(wl.context_lens[s]) * B.world
        note = "; per-rank oracle partials of KV head 0, all-gathered and merged by the oracle"
    else:
        mx, mean, s, tokens = sample_parity(wl, result, kv_heads=(1 if cfg_id == 4 else None))
        note = " (KV head 0 only)" if cfg_id == 4 else ""
    if B.world > 1:
        import torch.distributed as dist
        t = torch.tensor([mx, mean, float(st)], device=B.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        mx, mean, st = float(t[0]), float(t[1]), int(t[2])
    peak, _ = measured_peak()
    value = tot_bytes / (ms * 1e-3) / 1e12
    rec.update({
        "workload": wl.name, "ms_per_step": ms, "kv_tbps": value, "frac_of_measured_peak": value * 1e3 / (peak * B.world),
        "pct_of_nominal_8TBs": 100.0 * value * 1e3 / (NOMINAL_HBM_GBS * B.world),
        "tokens_per_s": tot_q / (ms * 1e-3), "scaling": scaling, "parallelism": parallelism,
        "kv_bytes_per_rank": kv_bytes, "kv_bytes_total": tot_bytes, "batch_per_rank": wl.num_seqs,
        "steps_per_block": steps, "device_status": st,
        "parity": parity_record(mx, mean, s, tokens, note),
    })
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + list(AUX_WORKLOADS))
    ap.add_argument("--batch", type=int, default=None, help="override the batch (smaller ncu captures)")
    ap.add_argument("--ctx-scale", type=float, default=1.0)
    ap.add_argument("--page-size", type=int, default=16, help="page size of the pa16 workload (16, 32 or 64)")
    ap.add_argument("--cpu-budget-s", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-workloads", action="store_true",
                    help="skip the cfg3 / cfg4 / cfg5 legs that follow the headline workload")
    ap.add_argument("--kernel-only", action="store_true", help="only the attention-kernel loop (ncu)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="repeat every timed loop until this much has been measured (lower it under a profiler)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.warmup < 3:
        args.warmup = 3
    from cuda_b200 import workloads
    if args.workload in AUX_WORKLOADS:
        return aux_workload(args, rank, world, local)
    cfg_id = WORKLOADS[args.workload]
    seed = 1000 + cfg_id + 7919 * rank

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return
        ncores = os.cpu_count() or 1
        torch.set_num_threads(ncores)
        wl = workloads.make_config(cfg_id, "cpu", batch=args.batch, ctx_scale=args.ctx_scale,
                                   seed=seed, poison=False)
        args.steps = min(args.steps, 20)          # CPU steps are seconds, not microseconds
        per_step_budget = max(1.0, min(20.0, 120.0 / max(1, args.steps + 1)))
        for _ in range(min(args.warmup, 1)):
            cpu_reference_run(wl, per_step_budget)
        tot_t, tot_b, tot_q, n = 0.0, 0, 0, 0
        for _ in range(args.steps):
            t, b, q, done = cpu_reference_run(wl, per_step_budget)
            tot_t, tot_b, tot_q, n = tot_t + t, tot_b + b, tot_q + q, n + done
        val = tot_b / tot_t / 1e12
        line = {
            "metric": "paged_fp8_decode_kv_hbm_throughput", "value": val, "unit": "TB/s", "impl": "reference",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": tot_t / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3->f32", "data": "synthetic",
            "tokens_per_s": tot_q / tot_t,
            "config": {"workload": wl.name, "sample": f"{n // max(1, args.steps)} sequence passes per step over the batch of {wl.num_seqs}",
                       "heads": f"{wl.num_q_heads}q/{wl.num_kv_heads}kv",
                       "head_dim": wl.head_dim, "page_size": wl.page_size},
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"{n} sequences in {tot_t:.1f} s"},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return

    # ------------------------------------------------------------------ our arm (GPU)
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local)
    B = Bench(args, rank, world, local)
    dev = B.dev
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from cuda_b200 import ops, sharding
    ops.L.load()

    wl, scaling, parallelism, split_ctx = build_leg(B, cfg_id, args, batch=args.batch, ctx_scale=args.ctx_scale)
    kv_bytes = wl.kv_bytes()
    q_tokens = wl.query.shape[0]
    need = ops.L.load().cuda_llm_paged_decode_workspace_bytes(
        wl.num_seqs, wl.num_q_heads, wl.num_kv_heads, wl.head_dim, wl.page_size, wl.max_q_len, 0)
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    out = torch.empty_like(wl.query)
    dec = sharding.SplitContextDecoder(wl) if split_ctx else None

    # In the resident loops the step inputs (lengths, block tables) are not rewritten between calls,
    # which is what a model does across its layers within one step: the library may then plan
    # while the previous kernel drains (CUDA_LLM_FLAG_STABLE_METADATA).  The step time without that
    # promise is measured beside it.  The end-to-end legs copy fresh inputs every step and do not
    # make the promise.
    STABLE = ops.L.FLAG_STABLE_METADATA

    def step(flags=STABLE):
        if split_ctx:
            return dec(wl, flags=flags)
        return ops.run_workload(wl, out=out, workspace=ws, flags=flags)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    st = ops.decode_status(dec.workspace if split_ctx else ws)
    assert st == 0, f"device status 0x{st:x}"

    if args.kernel_only:
        ms = median(B.timed_blocks(lambda: ops.run_workload(wl, out=out, workspace=ws,
                                                            flags=ops.L.FLAG_SKIP_MERGE | STABLE), args.steps, 0.0))
        if rank == 0:
            print(json.dumps({"kernel_only_ms": ms, "kv_bytes": kv_bytes, "GBs": kv_bytes / ms / 1e6}), flush=True)
        return

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # (1) whole step resident in HBM: attention kernel + split merge (+ all-gather and merge when split)
    blocks_total = B.timed_blocks(step, args.steps)
    ms_step = median(blocks_total)
    # (2) the dominant kernel alone (roofline numerator / denominator)
    ms_kernel = median(B.timed_blocks(
        lambda: ops.run_workload(wl, out=out, workspace=ws, flags=ops.L.FLAG_SKIP_MERGE | STABLE), args.steps))
    step()
    # (2b) the same whole step without the stable-metadata promise
    ms_step_unflagged = median(B.timed_blocks(lambda: step(0), args.steps))
    # (3) end to end through the public op with host buffers: the step's inputs (query, block
    #     tables, context lengths, query offsets) come from pinned host memory, the result goes back.
    #     The inputs sit in ONE pinned staging buffer and go over in one copy per step (a serving
    #     loop assembles its step inputs in such a buffer anyway); the device tensors are views.
    srcs = [wl.query, wl.block_tables, wl.context_lens] + ([wl.cu_q_lens] if wl.cu_q_lens is not None else [])
    sizes = [(t.numel() * t.element_size() + 255) // 256 * 256 for t in srcs]
    h2d = sum(t.numel() * t.element_size() for t in srcs)
    host_stage = torch.empty(sum(sizes), dtype=torch.uint8).pin_memory()
    dev_stage = torch.empty(sum(sizes), dtype=torch.uint8, device=dev)
    dev_in, off = [], 0
    for t, n in zip(srcs, sizes):
        nb = t.numel() * t.element_size()
        host_stage[off:off + nb].copy_(t.cpu().contiguous().view(torch.uint8).view(-1))
        dev_in.append(dev_stage[off:off + nb].view(t.dtype).view(t.shape))
        off += n
    dev_cu = dev_in[3] if wl.cu_q_lens is not None else None
    host_out = torch.empty(wl.query.shape, dtype=wl.query.dtype).pin_memory()
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step():
        dev_stage.copy_(host_stage, non_blocking=True)
        if split_ctx:
            import dataclasses
            o = dec(dataclasses.replace(wl, query=dev_in[0], block_tables=dev_in[1], context_lens=dev_in[2]))
        else:
            o = ops.fp8_paged_attention_forward(dev_in[0], wl.key_cache, wl.value_cache, wl.k_scale, wl.v_scale,
                                                dev_in[1], dev_in[2], wl.softmax_scale, cu_q_lens=dev_cu,
                                                max_q_len=wl.max_q_len, workspace=ws)
        host_out.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
    ms_e2e = median(B.timed_blocks(e2e_step, args.steps))

    # (4) the same end-to-end step double-buffered, as a serving loop with two batches in flight
    #     runs it: the copies of step i+1 (other staging buffer, copy streams) overlap the kernels
    #     of step i.  Every step still moves its inputs in and its result out.
    ms_e2e_pipe = None
    if not split_ctx:
        s_in, s_out, s_main = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.current_stream(dev)
        stage2 = [dev_stage, torch.empty_like(dev_stage)]
        views2 = []
        for buf in stage2:
            v, off = [], 0
            for t, n in zip(srcs, sizes):
                nb = t.numel() * t.element_size()
                v.append(buf[off:off + nb].view(t.dtype).view(t.shape))
                off += n
            views2.append(v)
        outs2 = [torch.empty_like(wl.query) for _ in range(2)]
        host_out2 = [host_out, torch.empty(wl.query.shape, dtype=wl.query.dtype).pin_memory()]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        counter = [0]

        def e2e_pipe_step():
            b = counter[0] & 1
            counter[0] += 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[b])          # the kernels that read this staging buffer are done
                stage2[b].copy_(host_stage, non_blocking=True)
                ev_in[b].record(s_in)
            s_main.wait_event(ev_in[b])
            s_main.wait_event(ev_out[b])             # the previous result in this output buffer has left
            v = views2[b]
            ops.fp8_paged_attention_forward(v[0], wl.key_cache, wl.value_cache, wl.k_scale, wl.v_scale, v[1], v[2],
                                            wl.softmax_scale, cu_q_lens=(v[3] if wl.cu_q_lens is not None else None),
                                            max_q_len=wl.max_q_len, workspace=ws, out=outs2[b])
            ev_done[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                host_out2[b].copy_(outs2[b], non_blocking=True)
                ev_out[b].record(s_out)

        def e2e_pipe_run():
            for _ in range(args.steps):
                e2e_pipe_step()
            s_main.wait_event(ev_out[0])             # the timed region ends when the last results are on the host
            s_main.wait_event(ev_out[1])

        for _ in range(4):
            e2e_pipe_step()
        torch.cuda.synchronize()
        ms_e2e_pipe = median(B.timed_blocks(e2e_pipe_run, 1)) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    st = ops.decode_status(dec.workspace if split_ctx else ws)
    assert st == 0, f"device status 0x{st:x}"

    # parity gate of the headline workload: one sampled sequence against the CPU oracle
    result = step()
    torch.cuda.synchronize()
    if split_ctx:
        parity = None                                  # covered by the cfg4 leg's own record
    else:
        mx, mean, s_id, tokens = sample_parity(wl, result, kv_heads=(1 if cfg_id == 4 else None))
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([mx, mean], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            mx, mean = float(t[0]), float(t[1])
        parity = parity_record(mx, mean, s_id, tokens)
        assert parity["ok"], f"parity gate failed: {parity}"

    tot_bytes, tot_q = B.sum_over_ranks(kv_bytes, q_tokens if not (split_ctx and rank) else 0)
    meta = {"name": wl.name, "batch": wl.num_seqs, "heads": f"{wl.num_q_heads}q/{wl.num_kv_heads}kv",
            "head_dim": wl.head_dim, "page_size": wl.page_size, "kv_tokens": int(wl.context_lens.sum().item()),
            "pool_pages": wl.meta["pool_pages"]}
    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        t, b, q, n = cpu_reference_run(wl.to("cpu"), args.cpu_budget_s)
        cpu_baseline = {"value": b / t / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(),
                        "kind": "port", "tokens_per_s": q / t,
                        "sample": f"{n} sequence passes over the same batch of {wl.num_seqs} ({n / wl.num_seqs:.1f} batches), {t:.1f} s"}

    # the other sharded configurations on the same ranks
    extra = {}
    if cfg_id == 2 and not args.no_extra_workloads and args.batch is None and args.ctx_scale == 1.0:
        del wl, out, ws, result
        torch.cuda.empty_cache()
        for other in (3, 4, 5):
            rec = run_extra_leg(B, other, args)
            extra[rec.pop("workload")] = rec
            torch.cuda.empty_cache()
        wl = None

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    value = tot_bytes / (ms_step * 1e-3) / 1e12
    achieved = kv_bytes / (ms_kernel * 1e-3) / 1e9
    name = meta["name"]
    # CUDA_LLM_DECODE_KERNEL=tcgen05 (read by the library) moves the calls it serves onto the tensor-memory kernel
    decode_kernel = "tcgen05" if os.environ.get("CUDA_LLM_DECODE_KERNEL") == "tcgen05" else "warp_mma"
    line = {
        "metric": "paged_fp8_decode_kv_hbm_throughput", "value": value, "unit": "TB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "fp8_e4m3->f16 mma, f32 acc",
        "data": "synthetic", "tokens_per_s": tot_q / (ms_step * 1e-3),
        "pct_of_nominal_8TBs": 100.0 * value * 1e3 / (NOMINAL_HBM_GBS * world),
        "pct_of_measured_copy_peak": 100.0 * value * 1e3 / (peak * world),
        "timing": {"method": "CUDA events around blocks of `steps` back-to-back steps, barrier + synchronize on both "
                             "sides of every block, max over ranks per block, median over blocks",
                   "blocks": len(blocks_total), "min_timed_ms": args.min_timed_ms,
                   "ms_per_step_min": min(blocks_total), "ms_per_step_max": max(blocks_total)},
        "stable_metadata": {"resident_loops_set_CUDA_LLM_FLAG_STABLE_METADATA": True,
                            "ms_per_step_with_flag": ms_step, "ms_per_step_without_flag": ms_step_unflagged,
                            "value_without_flag": tot_bytes / (ms_step_unflagged * 1e-3) / 1e12,
                            "note": "opt-in promise that the kernel in front of the call does not write lengths or "
                                    "block tables (true across the layers of one model step); `value` and `roofline` "
                                    "are measured with it, the end-to-end legs without it"},
        "config": {"workload": name, "batch_per_gpu": meta["batch"], "heads": meta["heads"],
                   "head_dim": meta["head_dim"], "page_size": meta["page_size"],
                   "kv_tokens_per_gpu": meta["kv_tokens"], "kv_bytes_per_gpu": kv_bytes,
                   "pool_pages": meta["pool_pages"], "parallelism": parallelism,
                   "decode_kernel": decode_kernel,
                   "l2": "inputs larger than L2 (KV working set per step >> 126 MB), no flush needed"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src,
                     "kernel": "paged_decode_sm100_kernel" if decode_kernel == "tcgen05" and name.startswith("cfg2") else "paged_decode_kernel",
                     "kernel_ms": ms_kernel,
                     "traffic": None},
        "e2e": {"value": tot_bytes / (ms_e2e * 1e-3) / 1e12, "unit": "TB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                "note": "KV cache resident in HBM (it is decode state, like weights); per-step inputs "
                        "(query, block tables, context lengths) from pinned host memory, output read back; "
                        "value = copy, kernels, copy back strictly one after the other on one stream",
                "double_buffered": (None if ms_e2e_pipe is None else
                                    {"value": tot_bytes / (ms_e2e_pipe * 1e-3) / 1e12, "unit": "TB/s",
                                     "ms_per_step": ms_e2e_pipe,
                                     "note": "same copies every step, two staging buffers and copy streams: "
                                             "the copies of step i+1 overlap the kernels of step i"})},
        "gpu_launches": (4 if split_ctx else 2) * args.steps,
        "parity": parity,
        "workloads": extra,
        "clocks": clocks,
    }
    ratio = DRAM_TRAFFIC_PER_KV_BYTE.get(name)
    if ratio is not None:
        line["roofline"]["traffic"] = ratio * kv_bytes
        line["roofline"]["traffic_source"] = "ncu dram__bytes_read+write of a batch-16 launch, scaled by KV bytes"
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
