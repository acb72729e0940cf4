#!/usr/bin/env python
"""Benchmark of the attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b2a|reference] [--only NAME]

Prints ONE JSON line (rank 0).  The headline workload is the Llama-3-8B-shaped causal bf16 prefill SDPA
(B=4, Hq=32, Hkv=8, S=4096, D=128); the same line carries the paged-decode half of the metric (KV GB/s on the
64-sequence u8-cache decode and on the 16 x 32768 long-context decode) under "decode".  With N > 1 the heads are
sharded over the ranks (Hkv/N KV heads each, no K/V crosses NVLink) and the per-head outputs are exchanged inside
the timed step by the kernels that produce them (peer stores over NVLink).  Every workload checks its own result
after the timed region - the device status word, and at N > 1 the full-width output against the single-GPU kernels
on each rank's shard gathered with NCCL - and reports it as "verified"; a failed check makes the exit code 1.

`--impl reference` times the CPU restatement of the reference's dense attention (oracle port, all host threads)
on a bounded slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PREFILL = dict(B=4, Hq=32, Hkv=8, S=4096, D=128)

# dram__bytes_read + dram__bytes_write per launch, from profiler captures of these kernels on these workloads.
# They are constants of this file, not measurements of the run that prints them (a profiler cannot run inside a
# timed benchmark); the line says so next to each figure.
NCU_TRAFFIC = {
    "prefill": 429.2e6,   # attn_tc_kernel<bf16, dense> on the full prefill workload
    "cfg3": 627.5e6,      # paged_decode_kernel<f16, 1> on the 64-sequence decode
}
TRAFFIC_SOURCE = "profiler capture of this kernel on this workload (a constant, not measured in this run)"
L2_BYTES = 126 * (1 << 20)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and clock-event reasons of one GPU through NVML (read-only queries) on a thread, every
    couple of milliseconds, while the timed region runs."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, index: int, period_s: float = 0.002):
        self.rows, self.handle, self.stop_flag, self.period = [], None, False, period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception as e:  # no NVML: the line says so instead of inventing clocks
            self.handle, self.error = None, f"NVML unavailable: {type(e).__name__}"

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.rows.append((time.time(), float(mhz), int(mask)))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self, t0: float, t1: float):
        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error]}
        self.stop_flag = True
        self.thread.join(timeout=1.0)
        inside = [r for r in self.rows if t0 <= r[0] <= t1]
        near = inside or self.rows[-3:]
        reasons = sorted({name for _, _, m in near for name, bit in self.REASONS if m & bit})
        mhz = [r[1] for r in near]
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def causal_flops(B, Hq, S, D):
    return 4 * B * Hq * D * (S * (S + 1) // 2)


# ----------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's dense attention (restating the reference's _dense_attention) on all host threads
# ----------------------------------------------------------------------------------------------------------

def cpu_prefill_sample(steps: int, warmup: int, budget_s: float = 20.0):
    """Times softmax(QK^T*scale + causal)V in float32 on the CPU for a slice of the prefill workload:
    one batch entry, the 4 query heads of one KV head, full S and D.  Returns (TFLOP/s, dict)."""
    from oracle.torch_cpu import dense_attention_cpu
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    S, D, g = PREFILL["S"], PREFILL["D"], PREFILL["Hq"] // PREFILL["Hkv"]
    gen = torch.Generator().manual_seed(1)
    q = (torch.randn(1, g, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    k = (torch.randn(1, 1, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    v = (torch.randn(1, 1, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    fl = causal_flops(1, g, S, D)
    times = []
    t_begin = time.time()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        dense_attention_cpu(q, k, v, causal=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.time() - t_begin > budget_s and len(times) >= 1:
            break
    ms = 1e3 * float(np.mean(times))
    tf = fl / (ms * 1e-3) / 1e12
    return tf, ms, dict(value=tf, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                        sample=f"B=1, Hq={g} (one KV head), S={S}, D={D} causal slice of the prefill workload, "
                               f"f32 math on bf16 data, {len(times)} timed passes")


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    tf, ms, base = cpu_prefill_sample(args.steps, args.warmup, budget_s=60.0)
    line = {"impl": "reference", "metric": "prefill attn TFLOP/s (causal bf16 SDPA, Llama-3-8B shape)",
            "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 on bf16 data", "data": "synthetic",
            "config": {"workload": "prefill_llama3_8b: B=4 Hq=32 Hkv=8 S=4096 D=128 causal, scale=1/sqrt(128)",
                       "step": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "OpenVINO runtime not present; CPU restatement of the reference's dense attention "
                    "(modules/genai_optimizations/genai_opt/sparse_attention.py:95-121) stands in"}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------

def timed(fn, steps, warmup, world, stream=None):
    """W warm-up calls, then K calls between two events; barrier + synchronize on both sides; max over ranks."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps, t0, t1


def timed_replay(fn, steps, warmup, world, multiple_of=1):
    """Like timed(), but the steps are captured into a CUDA graph and the timed region replays it - how the plugin's
    graph runner executes a captured topology (no host-side launch cost in the timed region).  A graph holds up to
    25 consecutive steps (a decoder's graph holds one such step per layer), and K steps are K/25 replays.  Falls
    back to plain calls when the capture fails (a collective library that refuses capture, for instance)."""
    for _ in range(max(1, warmup)):
        fn()
    torch.cuda.synchronize()
    # steps per graph: a divisor of the step count, a multiple of `multiple_of` (steps that walk through several
    # pools come back to the first pool at the start of every replay)
    steps = -(-steps // multiple_of) * multiple_of
    per_graph = max(g for g in range(multiple_of, max(26, multiple_of + 1), multiple_of) if steps % g == 0)
    try:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(per_graph):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
    except Exception:
        torch.cuda.synchronize()
        ms, t0, t1 = timed(fn, steps, 1, world)
        return ms, "plain calls (graph capture failed)"
    ms, _, _ = timed(graph.replay, steps // per_graph, 2, world)
    return ms / per_graph, f"graph replay, {per_graph} steps per graph, {steps} steps timed"


def bench_prefill(args, rank, world, local):
    import torch.distributed as dist
    import openvino_contrib_b200 as b2a
    B, Hq, Hkv, S, D = (PREFILL[k] for k in ("B", "Hq", "Hkv", "S", "D"))
    assert Hkv % world == 0
    hkv_l, hq_l = Hkv // world, Hq // world
    gen = torch.Generator().manual_seed(1)
    # the full problem is generated from one seed; each rank keeps its head shard
    sl_q = slice(rank * hq_l, (rank + 1) * hq_l)
    sl_k = slice(rank * hkv_l, (rank + 1) * hkv_l)
    q_h = (torch.randn(B, Hq, S, D, generator=gen) * 0.5).to(torch.bfloat16)[:, sl_q].contiguous().pin_memory()
    k_h = (torch.randn(B, Hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)[:, sl_k].contiguous().pin_memory()
    v_h = (torch.randn(B, Hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)[:, sl_k].contiguous().pin_memory()
    q, k, v = q_h.cuda(), k_h.cuda(), v_h.cuda()
    out = torch.empty(B, hq_l, S, D, dtype=torch.bfloat16, device="cuda")
    from openvino_contrib_b200.sharding import HeadShard, gather_heads_bhsd, gather_heads_rows  # noqa: F401
    shard = HeadShard(rank, world, Hq, Hkv)
    exchange, group = "none", None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if world > 1:
        exchange = ("peer stores from the attention kernel: its epilogue stores every tile into every rank's buffer "
                    "(from 4 GPUs on the CTAs take their items lightest first, so the stores start at once)")
        try:
            from openvino_contrib_b200.sharding import ShardGroup
            group = ShardGroup(shard, staging_bytes=B * Hq * S * D * 2)
        except Exception as e:  # CUDA IPC not available: the library collective instead
            exchange = f"nccl all-gather after the kernel (peer mapping failed: {type(e).__name__})"
    gathered = torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device="cuda") if world > 1 and group is None else None
    launches = [0]

    def step():
        launches[0] += 1
        if group is not None:
            return group.sdpa(q, k, v, causal=True, status=status)
        b2a.sdpa(q, k, v, causal=True, out=out, status=status)
        if world > 1:
            gather_heads_bhsd(out, shard, buffer=gathered)
            return gathered
        return out

    sampler = ClockSampler(local)
    ms, t0, t1 = timed(step, args.steps, args.warmup, world)
    clocks = sampler.stop(t0, t1)
    verified = verify_prefill(step, q, k, v, out, shard, status, world)
    n_launch = args.steps
    flops = causal_flops(B, Hq, S, D)
    value = flops / (ms * 1e-3) / 1e12

    # kernel-only duration (no collective) for the roofline of the dominant kernel
    def kern():
        b2a.sdpa(q, k, v, causal=True, out=out)
    kms, _, _ = timed(kern, args.steps, 1, 1)
    pk = peaks()
    achieved = causal_flops(B, hq_l, S, D) / (kms * 1e-3) / 1e12
    roof = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
            "frac": achieved / pk["tflops"],
            "traffic": NCU_TRAFFIC["prefill"] if world == 1 else None,
            "traffic_source": TRAFFIC_SOURCE if world == 1 else None,
            "peak_source": pk["source"] + " burst bf16 GEMM", "kernel_ms": kms}
    if world == 1 and args.only is None:
        roof["sustained"] = sustained_prefill(kern, causal_flops(B, hq_l, S, D), kms, local, pk)

    # end to end through the public API with host buffers: H2D of q,k,v, kernel, D2H of the output
    out_h = torch.empty(B, hq_l, S, D, dtype=torch.bfloat16).pin_memory()

    pipe = b2a.HostSdpaPipeline(B, hq_l, hkv_l, S, S, D, torch.bfloat16, causal=True) if world == 1 else None

    def e2e_step():
        if pipe is not None:  # upload, kernel and download of successive batch entries overlap on three streams
            pipe(q_h, k_h, v_h, out_h)
            return
        qd, kd, vd = q_h.cuda(non_blocking=True), k_h.cuda(non_blocking=True), v_h.cuda(non_blocking=True)
        if group is not None:
            o = group.sdpa(qd, kd, vd, causal=True)[:, sl_q]
        else:
            o = b2a.sdpa(qd, kd, vd, causal=True)
            if world > 1:
                gather_heads_bhsd(o, shard, buffer=gathered)
        out_h.copy_(o, non_blocking=True)
    ems, _, _ = timed(e2e_step, max(3, args.steps // 2), 2, world)
    h2d = (q_h.numel() + k_h.numel() + v_h.numel()) * 2
    e2e = {"value": flops / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": out_h.numel() * 2, "ms_per_step": ems,
           "api": f"C++ HostSdpaRunner: pinned upload, SdpaOp::Execute and download per piece of a few KV heads of one batch entry "
                  f"({pipe.pieces} pieces) on three streams" if pipe is not None
           else "sdpa on device copies of the host tensors"}
    if group is not None:
        torch.cuda.synchronize()
        dist.barrier()
        group.close()
    return dict(ms=ms, value=value, roofline=roof, e2e=e2e, clocks=clocks, launches=n_launch * (2 if group else 1),
                exchange=exchange, verified=verified)


def verify_prefill(step, q, k, v, out, shard, status, world):
    """After the timed region: the status word is clean, and (N > 1) one more step's full-width result equals, bit for
    bit, the plain single-GPU kernel run on every rank's shard and all-gathered with NCCL."""
    import torch.distributed as dist
    import openvino_contrib_b200 as b2a
    from openvino_contrib_b200.sharding import gather_heads_bhsd
    torch.cuda.synchronize()
    ok = int(status.item()) == 0
    if world > 1:
        full = step()
        b2a.sdpa(q, k, v, causal=True, out=out)
        ref = gather_heads_bhsd(out, shard)
        torch.cuda.synchronize()
        ok = ok and int(status.item()) == 0 and bool(torch.equal(full, ref))
        t = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(t.item())
    return ok


def sustained_prefill(kern, flops, burst_ms, local, pk, seconds=2.5):
    """The prefill kernel back to back for a couple of seconds - long enough for the power limit to pull the clock
    down - with the SM clock sampled meanwhile: the figure to set against the sustained GEMM peak."""
    n = max(50, int(seconds * 1e3 / burst_ms))
    sampler = ClockSampler(local, period_s=0.01)
    ms, t0, t1 = timed(kern, n, 3, 1)
    clocks = sampler.stop(t0 + 0.5 * (t1 - t0), t1)  # the second half: the clock has settled by then
    tf = flops / (ms * 1e-3) / 1e12
    peak = pk.get("tflops_sustained") or pk["tflops"]
    return {"achieved": tf, "peak": peak, "frac": tf / peak, "launches": n, "seconds": n * ms * 1e-3,
            "kernel_ms": ms, "sm_mhz_second_half": clocks["sm_mhz"], "reasons": clocks["reasons"],
            "peak_source": pk["source"] + " bf16 GEMM looped for seconds under the power limit"}


def build_decode_problem(n_seqs, ctx_lens, Hq, Hkv, D, seed, device="cuda"):
    """u8 pools filled on the device through b2a_paged_kv_store from N(0,1) rows; seeded shuffled block table."""
    import openvino_contrib_b200 as b2a
    bs = 16
    nblk = [(int(c) + bs - 1) // bs for c in ctx_lens]
    total = sum(nblk)
    perm = torch.randperm(total + 1, generator=torch.Generator().manual_seed(seed + 1))[:total].to(torch.int32)
    bb = torch.zeros(n_seqs + 1, dtype=torch.int32)
    bb[1:] = torch.cumsum(torch.tensor(nblk), 0)
    cache = b2a.PagedKvCache.allocate(total + 1, Hkv, D, bs, torch.uint8, device=device, poison=0xFF)
    bi, bbd = perm.to(device), bb.to(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    # fill in slices of at most 2048 positions per sequence
    maxc = int(max(ctx_lens))
    ctx_t = torch.tensor([int(c) for c in ctx_lens])
    for p0 in range(0, maxc, 2048):
        ql = torch.clamp(ctx_t - p0, 0, 2048).to(torch.int32)
        ntok = int(ql.sum())
        if ntok == 0:
            break
        sb = torch.zeros(n_seqs + 1, dtype=torch.int32)
        sb[1:] = torch.cumsum(ql, 0)
        past = torch.where(ql > 0, torch.full_like(ql, p0), ctx_t.to(torch.int32))
        key = torch.randn(ntok, Hkv * D, generator=gen, device=device, dtype=torch.float16)
        val = torch.randn(ntok, Hkv * D, generator=gen, device=device, dtype=torch.float16)
        b2a.paged_kv_store(key, val, cache, past.to(device), sb.to(device), bi, bbd)
    past = (ctx_t - 1).to(torch.int32).to(device)
    sb = torch.arange(n_seqs + 1, dtype=torch.int32, device=device)
    q = torch.randn(n_seqs, Hq * D, generator=gen, device=device, dtype=torch.float16)
    return cache, q, past, sb, bi, bbd


def bench_decode(name, steps, warmup, rank, world):
    """Paged decode, u8 KV: 'cfg3' = 64 sequences with contexts U[512, 8192]; 'cfg5' = 16 x 32768, Hq 64.

    A head shard of the cache can be small enough to sit in the 126 MB L2, which a serving step never enjoys (the
    cache of a decoder is read once per layer and step).  So when one rank's share is below four times the L2
    size, several pools with different contents and block tables are built and the steps walk through them in turn:
    every step finds its pool evicted."""
    import torch.distributed as dist
    import openvino_contrib_b200 as b2a
    if name == "cfg3":
        n, Hq, Hkv = 64, 32, 8
        ctx = np.random.default_rng(2).integers(512, 8193, size=n)
    else:
        n, Hq, Hkv = 16, 64, 8
        ctx = np.full(n, 32768)
    D = 128
    hkv_l, hq_l = Hkv // world, Hq // world
    tokens = int(ctx.sum())
    kv_bytes = tokens * Hkv * 2 * (D + 4)  # whole job: all ranks' heads
    per_rank = kv_bytes // world
    n_pools = 1 if per_rank >= 4 * L2_BYTES else -(-4 * L2_BYTES // per_rank)
    pools = [build_decode_problem(n, ctx, hq_l, hkv_l, D, seed=3 + rank + 100 * i) for i in range(n_pools)]
    maxc = int(ctx.max())
    out = torch.empty(n, hq_l * D, dtype=torch.float16, device="cuda")
    ws = torch.empty(max(16, b2a.ops.paged_workspace_bytes(torch.float16, pools[0][0], hq_l, n, n, maxc, 1)),
                     dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    from openvino_contrib_b200.sharding import HeadShard, ShardGroup, gather_heads_rows
    shard = HeadShard(rank, world, Hq, Hkv)
    gathered = torch.empty(world * n, hq_l * D, dtype=torch.float16, device="cuda") if world > 1 else None
    exchange = "none"
    group = None
    if world > 1:
        exchange = ("one kernel per step: the last CTA of a (sequence, KV head) merges the splits and sends the rows to every "
                    "rank as 8-byte words {two values, step number}; CTAs of the same kernel receive the other ranks' rows")
        try:
            group = ShardGroup(shard, staging_bytes=2 * n * Hq * D * 2)
        except Exception as e:  # CUDA IPC not available in this container: fall back to the library collective
            exchange = f"nccl all-gather after the kernels (peer mapping failed: {type(e).__name__})"
    out_full = torch.empty(n, Hq * D, dtype=torch.float16, device="cuda") if group is not None else None
    turn = [0]

    def step():
        cache, q, past, sb, bi, bb = pools[turn[0] % n_pools]
        turn[0] += 1
        if group is not None:
            group.paged_attention(q, cache, past, sb, bi, bb, max_context_len=maxc, out_full=out_full, workspace=ws,
                                  status=status, cache_rows_settled=True)
            return out_full
        # (cache_rows_settled: what the operator passes, whose attention call follows its own store of the new tokens)
        b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq_l, max_context_len=maxc, max_q_len=1, out=out,
                            workspace=ws, status=status, cache_rows_settled=True)
        if world > 1:
            return gather_heads_rows(out, shard, D, buffer=gathered)
        return out
    ms, how = timed_replay(step, steps, warmup, world, multiple_of=n_pools)
    # after the timed region: a clean status word, and (N > 1) one more step on every pool compared, bit for bit, with
    # the plain single-GPU kernels on each rank's shard all-gathered by NCCL
    torch.cuda.synchronize()
    verified = int(status.item()) == 0
    if world > 1:
        for i in range(n_pools):
            turn[0] = i
            full = step().clone()
            cache, q, past, sb, bi, bb = pools[i]
            o = b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq_l, max_context_len=maxc, max_q_len=1)
            ref = gather_heads_rows(o, shard, D)
            torch.cuda.synchronize()
            verified = verified and int(status.item()) == 0 and bool(torch.equal(full, ref))
        t = torch.tensor([1 if verified else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        verified = bool(t.item())
    if group is not None:
        torch.cuda.synchronize()
        dist.barrier()
        group.close()
    pk = peaks()
    gbs = kv_bytes / (ms * 1e-3) / 1e9
    return {"workload": name, "kv_gbs": gbs, "ms_per_step": ms, "kv_bytes_per_step": kv_bytes,
            "frac_of_hbm_peak": gbs / (pk["hbm_gbs"] * world), "peak_gbs_per_gpu": pk["hbm_gbs"],
            "peak_source": pk["source"], "cached_tokens": tokens, "verified": verified,
            "l2": (f"{n_pools} pools of {per_rank / 1e6:.0f} MB per GPU walked in turn: every step reads a pool that "
                   f"the steps in between evicted" if n_pools > 1 else
                   f"{per_rank / 1e6:.0f} MB of cache per GPU and step, read once, evict-first: nothing of it survives in the 126 MB L2"),
            "traffic": NCU_TRAFFIC.get(name) if world == 1 else None,
            "traffic_source": TRAFFIC_SOURCE if world == 1 and name in NCU_TRAFFIC else None,
            "launches_per_step": 1 if group is not None else 2, "output_exchange": exchange, "timing": how}


def bench_mixed(steps, warmup, rank, world):
    """Continuous-batching step through PagedAttentionExtension: 8 prefill sequences of 1024 tokens plus 120 decode
    sequences with contexts uniform in [256, 4096] (seed 4), bf16 queries, u8 KV, Hq 32 / Hkv 8 / D 128.
    One step = KV store of the 8312 new tokens + attention (tensor-core kernel for the prefill rows, split-K
    kernel for the decode rows).  Single GPU."""
    import openvino_contrib_b200 as b2a
    Hq, Hkv, D, bs = 32, 8, 128, 16
    rng = np.random.default_rng(4)
    dec_ctx = rng.integers(256, 4097, size=120)
    ctx = np.concatenate([np.full(8, 1024), dec_ctx])
    qlen = np.concatenate([np.full(8, 1024), np.ones(120, np.int64)])
    n = len(ctx)
    cache, _, _, _, bi, bb = build_decode_problem(n, ctx, Hq, Hkv, D, seed=11)
    past = torch.tensor(ctx - qlen, dtype=torch.int32, device="cuda")
    sb_h = np.zeros(n + 1, np.int64)
    sb_h[1:] = np.cumsum(qlen)
    sb = torch.tensor(sb_h, dtype=torch.int32, device="cuda")
    ntok = int(sb_h[-1])
    gen = torch.Generator(device="cuda").manual_seed(12)
    q = torch.randn(ntok, Hq * D, generator=gen, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(ntok, Hkv * D, generator=gen, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(ntok, Hkv * D, generator=gen, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(ntok, Hq * D, dtype=torch.bfloat16, device="cuda")
    rb = int(sum((int(x) + 127) // 128 for x in qlen if x >= 2))  # what the scheduler knows (KvBlockManager reports it)
    kvt = int(sum((int(c) + 127) // 128 * 128 for c, x in zip(ctx, qlen) if x >= 2))  # likewise
    ws = torch.empty(max(16, b2a.ops.paged_workspace_bytes(torch.bfloat16, cache, Hq, n, ntok, 4096, 1024, rb, kvt)),
                     dtype=torch.uint8, device="cuda")

    def attend():
        b2a.paged_attention(q, cache, past, sb, bi, bb, hq=Hq, max_context_len=4096, max_q_len=1024, out=out,
                            workspace=ws, prefill_row_blocks=rb, prefill_kv_tokens=kvt)

    def step():
        b2a.paged_kv_store(k, v, cache, past, sb, bi, bb)
        attend()
    ms, how = timed_replay(step, steps, warmup, 1)
    ams, _ = timed_replay(attend, steps, 1, 1)
    pk = peaks()
    prefill_flops = 8 * 4 * Hq * D * (1024 * 1025 // 2)
    decode_bytes = int(dec_ctx.sum()) * Hkv * 2 * (D + 4)
    store_bytes = ntok * Hkv * 2 * (D + 4)
    # time at the bars: 70 % of the tensor peak for the prefill rows plus 80 % of the HBM peak for the decode rows
    bar_ms = 1e3 * (prefill_flops / (0.7 * pk["tflops"] * 1e12) + decode_bytes / (0.8 * pk["hbm_gbs"] * 1e9))
    return {"workload": "cfg4", "ms_per_step": ms, "attention_ms": ams, "new_tokens": ntok,
            "prefill_flops": prefill_flops, "decode_kv_bytes": decode_bytes, "kv_store_bytes": store_bytes,
            "tokens_per_s": ntok / (ms * 1e-3), "bar_ms": bar_ms, "bar_over_measured": bar_ms / ams,
            "launches_per_step": 7 if kvt else 6, "timing": how, "prefill_kv": "de-quantised once into an f16 scratch" if kvt else
            "de-quantised inside the prefill kernel"}


def run_b2a(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import openvino_contrib_b200  # noqa: F401  (fails loudly if libb2a.so is missing)

    if args.only in ("cfg3", "cfg5", "cfg4"):  # a single paged workload, for profiler captures
        r = (bench_mixed(args.steps, args.warmup, rank, world) if args.only == "cfg4"
             else bench_decode(args.only, args.steps, args.warmup, rank, world))
        if rank == 0:
            print(json.dumps(r))
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        return
    failed = False
    pre = bench_prefill(args, rank, world, local)
    decode = {}
    if args.only is None:
        for name in ("cfg3", "cfg5"):
            decode[name] = bench_decode(name, max(args.steps, 24), max(args.warmup, 3), rank, world)
        if world == 1:
            decode["cfg4"] = bench_mixed(max(args.steps, 20), max(args.warmup, 3), rank, world)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        _, _, cpu = cpu_prefill_sample(3, 1, budget_s=20.0)
    if rank == 0:
        B, Hq, Hkv, S, D = (PREFILL[k] for k in ("B", "Hq", "Hkv", "S", "D"))
        line = {
            "metric": "prefill attn TFLOP/s (causal bf16 SDPA, Llama-3-8B shape)",
            "value": pre["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": pre["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"prefill_llama3_8b: B={B} Hq={Hq} Hkv={Hkv} S={S} D={D} causal, scale=1/sqrt(128), "
                                   f"Q,K,V ~ N(0,1)*0.5 seed 1",
                       "sharding": f"KV heads over {world} GPU(s), outputs exchanged inside the step: {pre['exchange']}"
                       if world > 1 else "single GPU",
                       "l2": "inputs + outputs (335 MB) exceed the 126 MB L2; no flush between steps"},
            "roofline": pre["roofline"], "cpu_baseline": cpu, "e2e": pre["e2e"], "gpu_launches": pre["launches"],
            "clocks": pre["clocks"], "verified": pre["verified"], "decode": decode,
        }
        print(json.dumps(line))
        if not pre["verified"] or not all(d.get("verified", True) for d in decode.values()):
            print("bench.py: a workload's result did not verify (status word or comparison with the single-GPU "
                  "kernels)", file=sys.stderr)
            failed = True
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b2a", choices=["b2a", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only", default=None, choices=["prefill", "cfg3", "cfg5", "cfg4"],
                    help="run one workload only (profiler captures); the default runs all and prints the full line")
    args = ap.parse_args()
    if args.impl == "b2a" and args.only is None:
        args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b2a(args)


if __name__ == "__main__":
    main()
