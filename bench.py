#!/usr/bin/env python
"""Benchmark of the selected-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE config 1 -- a varlen batch of 4 x 16384 tokens (64K), 4 KV heads,
GQA group 2, head_dim 128, block size 64, top-k 16, bf16, seeded synthetic inputs.  A step is one
forward + backward of the operator.  With N > 1 (one process per GPU, torchrun) every rank owns
one such 4-KV-head shard of a model with 4*N KV heads: selected attention never mixes KV heads,
so there is no collective on the path ("weak" scaling).

The JSON line carries: the device-resident throughput (`value`, effective TFLOP/s on the useful
FLOPs 14*d*P), the end-to-end number through the public operator with pinned host buffers
(`e2e`), the roofline of the dominant kernel, and a CPU baseline (the fp32 oracle timed on the
host cores on a bounded sample).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "flash-sparse-attention_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

# DRAM bytes (read + write) per launch of the main kernels from one ncu capture of the small case (one 16384-token
# sequence; profiles/sel_attn_kernels_small_case_ncu.md); traffic grows with the token count, so cfg1 is 4 x that.
NCU_TRAFFIC_SMALL = {"sel_bwd_main": 290.8e6 + 572.2e6, "sel_fwd_main": 79.3e6 + 496.9e6}
# the compressed pass of the decode step at batch 8 (profiles/decode_kernels_small_case_ncu.md); grows with the batch
NCU_TRAFFIC_DECODE_B8 = 268.5e6 + 6.7e6

METRIC = "sel-attn fwd+bwd effective TFLOPS @64K (4x16384 tok, Hk=4, G=2, d=128, B_K=64, T=16)"
UNIT = "TFLOP/s"
CFG = dict(seqlens=[16384] * 4, Hk=4, G=2, d=128, bs=64, T=16)


def workload_name():
    return "cfg1: varlen 4x16384 tokens, 4 KV heads, G=2, d=128, B_K=64, T=16, fwd+bwd"


def attended_pairs(idx_cpu, cu_cpu, bs, G):
    from oracle.sel_attn_oracle import attended_key_count  # counting helper only (integer work on the indices)

    return attended_key_count(idx_cpu, cu_cpu, bs, G)


def analytic_pairs(seqlens, Hk, G, bs, T):
    """Closed form of P for the synthetic generator: token t attends (n_t - 1) full blocks plus
    (t mod bs) + 1 keys of its own block, n_t = min(T, t // bs + 1)."""
    total = 0
    for L in seqlens:
        for b in range((L + bs - 1) // bs):
            n_tok = min(bs, L - b * bs)
            n_t = min(T, b + 1)
            total += n_tok * (n_t - 1) * bs + n_tok * (n_tok + 1) // 2
    return total * Hk * G


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join()
        s = sorted(self.samples)
        return {
            "sm_mhz": (s[len(s) // 2] if s else None),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(s),
        }


def cpu_baseline_sample(n_tokens, threads, repeats=1):
    """Time the fp32 oracle (forward + backward) on the first `n_tokens` of one cfg1 sequence."""
    from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx
    from oracle.sel_attn_oracle import sel_attn_forward_backward

    torch.set_num_threads(threads)
    Hk, G, d, bs, T = CFG["Hk"], CFG["G"], CFG["d"], CFG["bs"], CFG["T"]
    q, k, v, do = make_qkv(n_tokens, Hk * G, Hk, d, 43)
    idx = make_topk_idx([n_tokens], Hk, T, bs, 43)
    cu = make_cu_seqlens([n_tokens])
    P = analytic_pairs([n_tokens], Hk, G, bs, T)
    flops = 14 * d * P
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        sel_attn_forward_backward(q.float(), k.float(), v.float(), do.float(), idx, bs, cu, d ** -0.5)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return flops / best / 1e12, best, flops


def run_reference(args, rank, world):
    """Reference arm: the CPU restatement of the reference's nsa_ref path (the oracle) on the host
    cores.  The reference itself is Triton-only and has no CPU implementation to time."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    n_tok = 1024
    for _ in range(max(args.warmup, 0) and 1):
        cpu_baseline_sample(256, threads)
    t_tot, flops_tot = 0.0, 0.0
    for _ in range(args.steps):
        tf, dt, fl = cpu_baseline_sample(n_tok, threads)
        t_tot += dt
        flops_tot += fl
    val = flops_tot / t_tot / 1e12
    line = {
        "impl": "reference",
        "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t_tot / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded N(0,1) q/k/v/dO, seeded causal block ids)",
        "config": {"workload": workload_name(), "sample": f"first {n_tok} tokens of one sequence, fwd+bwd per step"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"fp32 oracle fwd+bwd on the first {n_tok} tokens of one cfg1 sequence, per step"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


DECODE_CFG = dict(batch=64, cache_len=131072, Hk=8, G=4, d=128, kernel_size=32, kernel_stride=16, block_size=64, topk=16,
                  init_blocks=1, local_blocks=2, window_size=512)
DECODE_METRIC = "NSA one-step decode tokens/s (batch 64 x 131072-token bf16 KV cache, Hk=8, G=4, d=128, ks=32/16, B_K=64, T=16, W=512)"


def decode_cpu_baseline(threads, cache_len=8192):
    """The decode oracle on the host cores: one sequence, one step."""
    from oracle.decode_oracle import decode_branches_ref

    c = DECODE_CFG
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1)
    Hk, d, Hq = c["Hk"], c["d"], c["Hk"] * c["G"]
    n_cmp = (cache_len - c["kernel_size"]) // c["kernel_stride"] + 1
    k, v = torch.randn(cache_len, Hk, d, generator=g), torch.randn(cache_len, Hk, d, generator=g)
    ck, cv = torch.randn(n_cmp, Hk, d, generator=g), torch.randn(n_cmp, Hk, d, generator=g)
    q = torch.randn(1, Hq, d, generator=g)
    t0 = time.perf_counter()
    decode_branches_ref(q, [k], [v], [ck], [cv], c)
    dt = time.perf_counter() - t0
    return 1.0 / dt, dt, cache_len


def run_decode(args, rank, world, local_rank):
    """One decode step of the three NSA branches + gate mix over a resident KV cache; with N > 1 the KV sequence is
    split over the ranks (same batch, same total cache: strong scaling) and partial outputs are merged by LSE after an
    NCCL all-gather."""
    import torch.distributed as dist

    from fsa_preview.module import FlashSparseAttentionDecodeKernel, GraphedShardedAttention, GraphedStep
    from fsa_preview.ops.decode import CudaDecodeOps, DecodeStepPlan, nsa_decode_attention, nsa_decode_mixed, shard_plan

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = dict(DECODE_CFG)
    if args.case == "small":
        c.update(batch=8)                   # 4.3 GB of cache: small enough for a profiler capture, larger than L2
    B, Lc, Hk, G, d = c["batch"], c["cache_len"], c["Hk"], c["G"], c["d"]
    Hq = Hk * G
    nsa = {n: c[n] for n in ("kernel_size", "kernel_stride", "block_size", "topk", "init_blocks", "local_blocks", "window_size")}
    margin = 64
    max_len = Lc + margin
    shard = shard_plan(max_len, c["kernel_size"], c["kernel_stride"], rank, world, align=64)
    mod = FlashSparseAttentionDecodeKernel(Hq * d, Hq, Hk, d, **nsa).to(dev).to(torch.bfloat16)
    torch.manual_seed(7)
    with torch.no_grad():
        for p in mod.parameters():
            p.normal_(0, 0.02)
    cache = mod.new_cache(B, max_len, shard=shard, device=dev)
    torch.manual_seed(100 + rank)
    for t in (cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.k_tail, cache.v_tail):
        t.normal_()
    cache.host_len = [Lc] * B
    cache.seq_len.fill_(Lc)
    g = torch.Generator().manual_seed(3)
    qh = torch.randn(B, Hq, d, generator=g).to(torch.bfloat16).pin_memory()
    knh = torch.randn(B, Hk, d, generator=g).to(torch.bfloat16).pin_memory()
    vnh = torch.randn(B, Hk, d, generator=g).to(torch.bfloat16).pin_memory()
    qd = qh.to(dev)
    from fsa.ops.gate import gate_mix

    def eager_step():
        if world == 1:
            return nsa_decode_mixed(qd, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0, cache.cmp_row0,
                                    mod.gate(qd.view(B, -1)), max_len=max_len, **nsa)[0]
        oc, os_, ow, *_ = nsa_decode_attention(qd, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                               cache.cmp_row0, max_len=max_len, shard=shard, **nsa)
        return gate_mix(mod.gate(qd.view(B, -1)), oc, os_.contiguous(), ow.contiguous())

    # N > 1: the step holds two NCCL all-gathers; capturing them in a graph stalled here, so the sharded step is three
    # graphs (its collective-free parts) with the two all-gathers launched in between
    use_graph = not args.no_graph
    step = eager_step
    if use_graph and world > 1:
        plan = DecodeStepPlan(max_len=max_len, shard=shard, **nsa)
        step = GraphedShardedAttention(plan, qd, cache, lambda oc, os_, ow: gate_mix(mod.gate(qd.view(B, -1)), oc, os_.contiguous(),
                                                                                      ow.contiguous()))
    elif use_graph:
        # the attention step at a fixed cache length, captured once and replayed
        with torch.no_grad():
            for _ in range(3):
                eager_step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"), torch.no_grad():
            eager_step()
        step = graph.replay

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / n

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step()
        sampler = ClockSampler(local_rank)
        sampler.start()
        ms_step = timed(step, args.steps)
        clocks = sampler.stop()
        # dominant kernel alone: the compressed branch's partial pass (all visible compressed K/V rows of this rank)
        ops = CudaDecodeOps()
        ks_, st_ = c["kernel_size"], c["kernel_stride"]
        n_cmp = (Lc - ks_) // st_ + 1
        n_loc = max(min(n_cmp, shard.cmp_hi) - shard.cmp_lo, 0)
        lo = cache.cmp_row0.view(B, 1, 1).expand(B, Hk, 1).contiguous()
        hi = (lo + n_loc).contiguous()
        nchunk = max(-(-n_loc // 1024), 1)
        cmp_pass = lambda: ops.attn_partial(qd, cache.cmp_k, cache.cmp_v, lo, hi, 1024, nchunk, d ** -0.5, want_scores=True)  # noqa: E731
        for _ in range(3):
            cmp_pass()
        torch.cuda.synchronize()
        g_cmp = torch.cuda.CUDAGraph()                    # replayed, so that the host cost of a launch is not in the figure
        with torch.cuda.graph(g_cmp, capture_error_mode="thread_local"):
            cmp_pass()
        ms_cmp = timed(g_cmp.replay, args.steps)

        # end to end: host q / k_new / v_new in, output row out, through the module's step (append + attention + gate mix)
        gstep = GraphedStep(mod.step, cache, [qd, knh.to(dev), vnh.to(dev)]) if use_graph and world == 1 else None

        y_host = torch.empty((B, Hq * d), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            # inputs from pinned host memory, output row back to pinned host memory, all queued on the stream
            if gstep is not None:
                y = gstep(qh, knh, vnh)
            else:
                y = mod.step(qh.to(dev, non_blocking=True), knh.to(dev, non_blocking=True), vnh.to(dev, non_blocking=True), cache)
            y_host.copy_(y, non_blocking=True)

        e2e_n = 0 if args.no_e2e else max(1, min(args.steps, margin // 2 - 4))
        if e2e_n:
            e2e_step()
            e2e_ms = timed(e2e_step, e2e_n)
    elem = 2
    T, BK, W = c["topk"], c["block_size"], c["window_size"]
    bytes_cmp = B * Hk * n_cmp * d * elem * 2
    bytes_sel = B * Hk * T * BK * d * elem * 2
    bytes_win = B * Hk * (W + 1) * d * elem * 2
    bytes_step = bytes_cmp + bytes_sel + bytes_win
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 0) or 0)
        src = "MEASURED_PEAKS.json hbm_gbs"
        if not peak:
            peak, src = 6650.0, "fallback"
        achieved = B * Hk * n_loc * d * elem * 2 / (ms_cmp * 1e-3) / 1e9
        cpu = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, dt, n = decode_cpu_baseline(threads)
            cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                   "sample": f"decode oracle, one sequence with a {n}-token cache, one step ({dt:.2f} s); cost grows with the cache length"}
        line = {
            "metric": DECODE_METRIC, "value": B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded N(0,1) cache and query)",
            "config": {"workload": f"decode: batch {B} x {Lc}-token cache" + (" (small case)" if args.case == "small" else ""),
                       "parallelism": f"kv-sequence shards x{world}, LSE merge after all-gather" if world > 1 else "one GPU",
                       "l2": "the cache read per step exceeds L2", "algorithmic_bytes_per_step": bytes_step,
                       "step_gbs": bytes_step / world / (ms_step * 1e-3) / 1e9},
            "roofline": {"bound": "hbm", "kernel": "decode_partial_tma (compressed branch)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_DECODE_B8 * B / 8 / world,
                         "traffic_source": "ncu capture at batch 8 scaled by the batch", "peak_source": src, "ms": ms_cmp},
            "cpu_baseline": cpu,
            "e2e": ({"value": B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": (qh.numel() + knh.numel() + vnh.numel()) * 2, "d2h_bytes_per_step": B * Hq * d * 2}
                    if e2e_n else None),
            "gpu_launches": (7 if world == 1 else 9) * args.steps, "cuda_graph": use_graph,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


LAYER_CFG = dict(hidden=4096, Hq=32, Hk=8, d=128, kernel_size=32, kernel_stride=16, block_size=64, topk=16, init_blocks=1,
                 local_blocks=2, window_size=512, rope_theta=500000.0, seqlens=[32768, 32768])
LAYER_METRIC = "NSA layer fwd+bwd tokens/s (2x32768 tok, hidden 4096, 32 Q / 8 KV heads, d=128, ks=32/16, B_K=64, T=16, W=512)"


def run_layer(args, rank, world, local_rank):
    """Forward + backward of the whole FlashSparseAttention layer.  With N > 1 the heads are split over the ranks
    (8/N KV heads and 32/N query heads each: the attention kernels need no collective); the layer output and the
    gradient of the input are summed over the ranks with one NCCL all-reduce each, as any head-parallel layer does."""
    import torch.distributed as dist

    from fsa.module.fsa import FlashSparseAttention, RopeConfig

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = dict(LAYER_CFG)
    if args.case == "small":
        c["seqlens"] = [8192, 8192]
    if c["Hk"] % world:
        raise SystemExit(f"--gpus must divide the {c['Hk']} KV heads")
    seqlens = c["seqlens"]
    N = sum(seqlens)
    rope = RopeConfig(max_position_embeddings=131072, head_dim=c["d"], rope_theta=c["rope_theta"])
    layer = FlashSparseAttention(c["hidden"], c["Hq"] // world, c["Hk"] // world, c["d"], c["kernel_size"], c["kernel_stride"],
                                 c["block_size"], c["topk"], c["init_blocks"], c["local_blocks"], c["window_size"], rope)
    torch.manual_seed(11 + rank)
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.02)
    layer = layer.to(dev).to(torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    xh = torch.randn(N, c["hidden"], generator=g).to(torch.bfloat16).pin_memory()
    dyh = torch.randn(N, c["hidden"], generator=g).to(torch.bfloat16).pin_memory()
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32, device=dev)
    xd, dyd = xh.to(dev), dyh.to(dev)

    def step(x=None, dy=None):
        x = (xd if x is None else x).detach().requires_grad_(True)
        y = layer(x, cu, seqlens)
        if world > 1:
            dist.all_reduce(y.data)
        y.backward(dyd if dy is None else dy)
        if world > 1:
            dist.all_reduce(x.grad)
        layer.zero_grad(set_to_none=True)
        return y, x.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / n

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_step = timed(step, args.steps)
    clocks = sampler.stop()

    def e2e_step():
        y, gx = step(xh.to(dev, non_blocking=True), dyh.to(dev, non_blocking=True))
        return torch.stack([y.float().norm(), gx.float().norm()]).cpu()

    e2e_n = 0 if args.no_e2e else max(1, min(args.steps, 3))
    if e2e_n:
        e2e_step()
        e2e_ms = timed(e2e_step, e2e_n)
    if rank == 0:
        line = {
            "metric": LAYER_METRIC, "value": N / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded N(0,1) hidden states, N(0,0.02) weights)",
            "config": {"workload": f"layer fwd+bwd: {len(seqlens)}x{seqlens[0]} tokens" + (" (small case)" if args.case == "small" else ""),
                       "parallelism": f"head-parallel x{world}: {c['Hk'] // world} KV heads per GPU, all-reduce of the output and of dX only",
                       "l2": "activations exceed L2"},
            "roofline": None, "cpu_baseline": None,
            "e2e": ({"value": N / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": 2 * xh.numel() * 2, "d2h_bytes_per_step": 8} if e2e_n else None),
            "gpu_launches": None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="sel_attn", choices=["sel_attn", "decode", "layer"],
                    help="sel_attn (default): selected attention fwd+bwd, the headline; decode: one NSA decode step; "
                         "layer: the whole NSA layer fwd+bwd")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default="cfg1", choices=["cfg1", "small", "cfg2"],
                    help="small = one 16384-token sequence of cfg1 (a quarter of it), for profiler captures; "
                         "cfg2 = one 65536-token sequence, 4 KV heads, --group / --head-dim (the GQA sweep)")
    ap.add_argument("--group", type=int, default=2, help="cfg2: GQA group size (1..16)")
    ap.add_argument("--head-dim", type=int, default=128, help="cfg2: 128 or 256")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="decode workload: launch the step's kernels one by one")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "decode":
        run_decode(args, rank, world, local_rank)
        return
    if args.workload == "layer":
        run_layer(args, rank, world, local_rank)
        return

    import torch.distributed as dist
    from ctypes import byref, c_float, c_int

    from fsa import _lib
    from fsa.ops import FSA_topk_sparse_attention
    from fsa.ops.FSA_topk_sparse_attention import sel_attn_bwd, sel_attn_fwd
    from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    L = _lib.lib()
    seqlens, Hk, G, d, bs, T = (CFG[k] for k in ("seqlens", "Hk", "G", "d", "bs", "T"))
    if args.case == "small":
        seqlens = seqlens[:1]
    if args.case == "cfg2":
        seqlens, G, d = [65536], args.group, args.head_dim
    N = sum(seqlens)
    scale = d ** -0.5
    # each rank owns one 4-KV-head shard with its own seed
    q, k, v, do = make_qkv(N, Hk * G, Hk, d, 43 + rank)
    idx = make_topk_idx(seqlens, Hk, T, bs, 43 + rank)
    cu = make_cu_seqlens(seqlens)
    P = analytic_pairs(seqlens, Hk, G, bs, T)
    flops_step = 14 * d * P
    host = [x.pin_memory() for x in (q, k, v, do, idx)]
    qd, kd, vd, dod, idxd = (x.to(dev) for x in host)
    cud = cu.to(dev)

    def step():
        o, lse, ws = sel_attn_fwd(qd, kd, vd, idxd, bs, cud, scale)
        return sel_attn_bwd(qd, kd, vd, o, lse, dod, idxd, bs, cud, scale, ws)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    L.fsa_profile_enable(1)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    clocks = sampler.stop()
    ms_total = ev0.elapsed_time(ev1)
    # per-kernel durations recorded inside the timed region
    kern = {}
    for name, kid in (("sel_fwd_main", 0), ("sel_fwd_reduce", 1), ("sel_bwd_main", 2), ("sel_bwd_dq_reduce", 3)):
        ms, n = c_float(0), c_int(0)
        _lib.check(L.fsa_profile_read(kid, byref(ms), byref(n)), "fsa_profile_read")
        kern[name] = {"ms_avg": (ms.value / n.value if n.value else None), "launches": n.value}
    L.fsa_profile_enable(0)

    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_step = ms_max / args.steps
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public operator, host buffers in, scalar results out.  Every step copies its inputs
    # from pinned host memory and reads its result back; the copies of step i + 1 run on a second stream into a second
    # set of device buffers while step i computes.
    e2e_steps = max(2, min(args.steps, 6))
    copy_stream = torch.cuda.Stream(device=dev)
    dev_bufs = [[torch.empty(x.shape, dtype=x.dtype, device=dev) for x in host] for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    res_host = [torch.empty(3, dtype=torch.float32).pin_memory() for _ in range(2)]

    def issue_copy(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])          # the step that last used these buffers is done with them
            for dst, src in zip(dev_bufs[b], host):
                dst.copy_(src, non_blocking=True)
            copied[b].record(copy_stream)

    def compute(i):
        b = i % 2
        cur = torch.cuda.current_stream()
        cur.wait_event(copied[b])
        qh, kh, vh, doh, ih = dev_bufs[b]
        qh, kh, vh = (x.detach().requires_grad_(True) for x in (qh, kh, vh))
        o = FSA_topk_sparse_attention(qh, kh, vh, ih, bs, cud, scale)
        o.backward(doh)
        res_host[b].copy_(torch.stack([qh.grad.float().norm(), kh.grad.float().norm(), vh.grad.float().norm()]), non_blocking=True)
        consumed[b].record(cur)

    def e2e_run(n):
        issue_copy(0)
        for i in range(n):
            if i + 1 < n:
                issue_copy(i + 1)
            compute(i)

    if args.no_e2e:
        e2e_steps = 0
    else:
        e2e_run(2)
    barrier()
    ev0.record()
    copy_stream.wait_event(ev0)
    e2e_run(e2e_steps)
    ev1.record()
    barrier()
    e2e_steps = max(e2e_steps, 1)
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    h2d = sum(x.numel() * x.element_size() for x in host)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak_tf = float(peaks.get("bf16_tflops_sustained", 0) or 0)
        peak_src = "MEASURED_PEAKS.json bf16_tflops_sustained (kernel timed inside a long step)"
        if not peak_tf:
            peak_tf, peak_src = 1400.0, "fallback (sustained cuBLAS bf16 on this pool)"
        # dominant kernel: the backward main kernel (10*d*P useful FLOPs per launch)
        dom = "sel_bwd_main" if (kern["sel_bwd_main"]["ms_avg"] or 0) >= (kern["sel_fwd_main"]["ms_avg"] or 0) else "sel_fwd_main"
        dom_flops = (10 if dom == "sel_bwd_main" else 4) * d * P
        dom_ms = kern[dom]["ms_avg"]
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12 if dom_ms else None
        cpu = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            n_tok = 2048
            tf, dt, _ = cpu_baseline_sample(n_tok, threads)
            cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"fp32 oracle fwd+bwd on the first {n_tok} tokens of one cfg1 sequence ({dt:.1f} s)"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded N(0,1) q/k/v/dO, seeded causal block ids)",
            "config": {"workload": workload_name() if args.case == "cfg1" else ("small: 1x16384 tokens of cfg1" if args.case == "small" else
                                    f"cfg2: 1x65536 tokens, 4 KV heads, G={G}, d={d}, B_K=64, T=16, fwd+bwd"), "parallelism": f"kv-head shards x{world}, no collective",
                       "l2": "inputs and partial buffers exceed L2 (q 134 MB, partials > 4 GB per step)",
                       "useful_flops_per_step": flops_step, "tokens_per_s": world * N / (ms_step * 1e-3)},
            "kernels": kern,
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": (achieved / peak_tf if achieved else None),
                         "traffic": (NCU_TRAFFIC_SMALL[dom] * (4 if args.case == "cfg1" else 1)) if args.case != "cfg2" else None,
                         "traffic_source": "ncu capture of the small case scaled by the token count", "peak_source": peak_src},
            "cpu_baseline": cpu,
            "e2e": {"value": world * flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 12,
                    "overlap": "copies of step i+1 on a second stream while step i computes"},
            "gpu_launches": 10 * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
