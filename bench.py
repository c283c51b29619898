#!/usr/bin/env python
"""Benchmark of the selected-attention hot path (forward + backward) on B200, with the NSA layer and the decode step
measured beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload sel_attn|layer|decode]

Headline (`value`): BASELINE config 1 -- a varlen batch of 4 x 16384 tokens (64K), 4 KV heads, GQA group 2, head_dim
128, block size 64, top-k 16, bf16, seeded synthetic inputs.  A step is one forward + backward of the operator.  With
N > 1 (one process per GPU, torchrun) THE SAME problem is split over the ranks: its 16 independent (sequence, kv head)
pairs are dealt to the GPUs (by kv head up to 4 GPUs, then by sequence), so the total work is fixed ("strong" scaling)
and there is no collective on the path -- selected attention never mixes kv heads or sequences.

The JSON line carries: the device-resident throughput (`value`, effective TFLOP/s on the useful FLOPs 14*d*P), the
end-to-end number through the public operator with pinned host buffers (`e2e`), the roofline of the dominant kernel, a
CPU baseline (the fp32 oracle timed on the host cores), and two sub-records measured in the same process group:
`layer` (BASELINE config 3, the whole NSA layer forward + backward, head-parallel over the ranks) and `decode`
(BASELINE config 4, one decode step, KV sequence sharded over the ranks).  `--workload layer|decode` print those
records as lines of their own.
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
# sequence of config 1); traffic grows with the token count, so config 1 is 4 x that.
NCU_TRAFFIC_SMALL = {"sel_bwd_main": 210.3e6 + 582.7e6, "sel_fwd_main": 73.3e6 + 479.6e6}
# the compressed pass of the decode step at batch 8, from one ncu capture; grows with the batch
NCU_TRAFFIC_DECODE_B8 = 268.5e6 + 6.7e6

METRIC = "sel-attn fwd+bwd effective TFLOPS @64K (4x16384 tok, Hk=4, G=2, d=128, B_K=64, T=16)"
UNIT = "TFLOP/s"
CFG = dict(seqlens=[16384] * 4, Hk=4, G=2, d=128, bs=64, T=16)


def workload_name():
    return "cfg1: varlen 4x16384 tokens, 4 KV heads, G=2, d=128, B_K=64, T=16, fwd+bwd"


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
    """Time the fp32 oracle (forward + backward) on the first `n_tokens` of one config-1 sequence."""
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


def cpu_baseline_config0(threads, repeats=3):
    """The fp32 oracle forward on BASELINE config 0 (1 x 8192 tokens, 4 KV heads, G = 1), best of `repeats`."""
    from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx
    from oracle.sel_attn_oracle import sel_attn_forward

    torch.set_num_threads(threads)
    n, Hk, G, d, bs, T = 8192, 4, 1, 128, 64, 16
    q, k, v = make_qkv(n, Hk * G, Hk, d, 42, with_do=False)
    idx = make_topk_idx([n], Hk, T, bs, 42)
    cu = make_cu_seqlens([n])
    flops = 4 * d * analytic_pairs([n], Hk, G, bs, T)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        sel_attn_forward(q.float(), k.float(), v.float(), idx, bs, cu, d ** -0.5)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return flops / best / 1e12, best


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def tensor_peak(burst):
    """Measured dense bf16 peak: the burst figure for a kernel timed alone or inside a step of milliseconds, the
    sustained one for a step that runs for seconds."""
    peaks = load_peaks()
    key = "bf16_tflops" if burst else "bf16_tflops_sustained"
    v = float(peaks.get(key, 0) or 0)
    if v:
        return v, f"MEASURED_PEAKS.json {key}"
    return (1590.0, "fallback (burst cuBLAS bf16 of an earlier B200 measurement)") if burst else (1400.0, "fallback (sustained cuBLAS bf16 of an earlier B200 measurement)")


class Dist:
    """The process group of the run (one rank per GPU) and the timing helpers built on it."""

    def __init__(self, rank, world, local_rank):
        import torch.distributed as dist

        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
        self.rank, self.world, self.dist = rank, world, dist
        torch.cuda.set_device(local_rank)
        self.dev = torch.device("cuda", local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, ms):
        t = torch.tensor([ms], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, n):
        """CUDA-event time of n calls between two barriers, max over the ranks, per call (ms)."""
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        self.barrier()
        return self.max_ms(ev0.elapsed_time(ev1)) / n

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def run_reference(args, rank, world):
    """Reference arm: the CPU restatement of the reference's nsa_ref path (the oracle) on the host
    cores.  The reference itself is Triton-only and has no CPU implementation to time."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    n_tok = 2048
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
        "ms_per_step": t_tot / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
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


def run_decode(args, dd, steps, sub=False):
    """One decode step of the three NSA branches + gate mix over a resident KV cache; with N > 1 the KV sequence is
    split over the ranks (same batch, same total cache: strong scaling) and partial outputs are merged by LSE after an
    NCCL all-gather.  Returns the record on rank 0 (None elsewhere)."""
    from fsa_preview.module import FlashSparseAttentionDecodeKernel, GraphedShardedAttention, GraphedStep
    from fsa_preview.ops.decode import CudaDecodeOps, DecodeStepPlan, nsa_decode_attention, nsa_decode_mixed, shard_plan

    rank, world, dev, dist = dd.rank, dd.world, dd.dev, dd.dist
    barrier, timed = dd.barrier, dd.timed
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

    # N > 1: the step holds two NCCL all-gathers, which are kept out of the graphs (a captured collective did not complete), so the sharded step is three
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

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step()
        sampler = ClockSampler(dev.index)
        sampler.start()
        ms_step = timed(step, steps)
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
        ms_cmp = timed(g_cmp.replay, steps)

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

        e2e_n = 0 if args.no_e2e else max(1, min(steps, margin // 2 - 4))
        if e2e_n:
            e2e_step()
            e2e_ms = timed(e2e_step, e2e_n)
    # the two packed all-gathers of the sharded step, alone (same message sizes: o + lse + local score rows, then the
    # selected and window partials)
    ag_ms = None
    if world > 1:
        max_cmp = (max_len - ks_) // st_ + 1
        ld = 1024 * -(-max(min(max_cmp, shard.cmp_hi - shard.cmp_lo), 1) // 1024)
        m1 = torch.empty(B * Hq * (d + 1) + B * Hk * ld, dtype=torch.float32, device=dev)
        m2 = torch.empty(2 * B * Hq * (d + 1), dtype=torch.float32, device=dev)
        g1 = torch.empty(world * m1.numel(), dtype=torch.float32, device=dev)
        g2 = torch.empty(world * m2.numel(), dtype=torch.float32, device=dev)

        def gathers():
            dist.all_gather_into_tensor(g1, m1)
            dist.all_gather_into_tensor(g2, m2)

        gathers()
        ag_ms = timed(gathers, max(steps, 5))
    elem = 2
    T, BK, W = c["topk"], c["block_size"], c["window_size"]
    bytes_cmp = B * Hk * n_cmp * d * elem * 2
    bytes_sel = B * Hk * T * BK * d * elem * 2
    bytes_win = B * Hk * (W + 1) * d * elem * 2
    bytes_step = bytes_cmp + bytes_sel + bytes_win
    line = None
    if rank == 0:
        peaks = load_peaks()
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
            "metric": DECODE_METRIC, "value": B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded N(0,1) cache and query)",
            "config": {"workload": f"decode: batch {B} x {Lc}-token cache" + (" (small case)" if args.case == "small" else ""),
                       "parallelism": f"kv-sequence shards x{world}, LSE merge after all-gather" if world > 1 else "one GPU",
                       "l2": "the cache read per step exceeds L2", "algorithmic_bytes_per_step": bytes_step,
                       "step_gbs": bytes_step / world / (ms_step * 1e-3) / 1e9},
            "tokens_per_s": B / (ms_step * 1e-3), "step_gbs": bytes_step / world / (ms_step * 1e-3) / 1e9,
            "frac_hbm": bytes_step / world / (ms_step * 1e-3) / 1e9 / peak, "allgather_ms": ag_ms,
            "roofline": {"bound": "hbm", "kernel": "decode_partial_tma (compressed branch)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_DECODE_B8 * B / 8 / world,
                         "traffic_source": "ncu capture at batch 8 scaled by the batch", "peak_source": src, "ms": ms_cmp},
            "cpu_baseline": cpu,
            "e2e": ({"value": B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": (qh.numel() + knh.numel() + vnh.numel()) * 2, "d2h_bytes_per_step": B * Hq * d * 2}
                    if e2e_n else None),
            "gpu_launches": (7 if world == 1 else 9) * steps, "cuda_graph": use_graph,
            "clocks": clocks,
        }
    del cache, mod
    torch.cuda.empty_cache()
    return line


LAYER_CFG = dict(hidden=4096, Hq=32, Hk=8, d=128, kernel_size=32, kernel_stride=16, block_size=64, topk=16, init_blocks=1,
                 local_blocks=2, window_size=512, rope_theta=500000.0, seqlens=[32768, 32768])
LAYER_METRIC = "NSA layer fwd+bwd tokens/s (2x32768 tok, hidden 4096, 32 Q / 8 KV heads, d=128, ks=32/16, B_K=64, T=16, W=512)"


def layer_useful_flops(c, seqlens):
    """Algorithmic FLOPs of one forward + backward of the layer: projections (2 * tokens * in * out, x3 for forward,
    dX and dW), the three attention branches on their attended (query head, token, key) triples (4 * d forward,
    10 * d backward per triple), the two compressors (x3)."""
    N = sum(seqlens)
    hid, Hq, Hk, d = c["hidden"], c["Hq"], c["Hk"], c["d"]
    ks, st, bs, T, W = c["kernel_size"], c["kernel_stride"], c["block_size"], c["topk"], c["window_size"]
    proj = 2 * N * hid * (Hq * d + 2 * Hk * d) + 2 * N * (Hq * d) * hid + 2 * N * hid * 3
    p_cmp = p_sel = p_win = ncmp = 0
    for L in seqlens:
        ncmp += (L - ks) // st + 1 if L >= ks else 0
        for t in range(L):
            p_cmp += min((t - (ks - 1)) // st + 1, (L - ks) // st + 1) if t >= ks - 1 else 0
            p_win += min(t, W) + 1
        for b in range((L + bs - 1) // bs):
            n_tok = min(bs, L - b * bs)
            n_t = min(T, b + 1)
            p_sel += n_tok * (n_t - 1) * bs + n_tok * (n_tok + 1) // 2
    attn = 14 * d * Hq * (p_cmp + p_sel + p_win)
    compress = 3 * 2 * (2 * ncmp * Hk * (ks * d) * d)
    return 3 * proj + attn + compress


def layer_cpu_baseline(threads, n_tokens=512):
    """The layer oracle (forward only) on one short sequence with the layer's dimensions."""
    from fsa.module.rope import RopeConfig, compute_inv_freq
    from oracle.nsa_layer_oracle import layer_forward_ref

    c = LAYER_CFG
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(9)
    Hq, Hk, d, hid = c["Hq"], c["Hk"], c["d"], c["hidden"]
    params = {
        "proj_q.weight": torch.randn(Hq * d, hid, generator=g) * 0.02, "proj_k.weight": torch.randn(Hk * d, hid, generator=g) * 0.02,
        "proj_v.weight": torch.randn(Hk * d, hid, generator=g) * 0.02, "proj_o.weight": torch.randn(hid, Hq * d, generator=g) * 0.02,
        "compress_key": torch.randn(Hk, c["kernel_size"] * d, d, generator=g) * 0.02,
        "compress_value": torch.randn(Hk, c["kernel_size"] * d, d, generator=g) * 0.02,
        "intra_block_pe": torch.randn(Hk, c["kernel_size"], d, generator=g) * 0.02, "gate.0.weight": torch.randn(3, hid, generator=g) * 0.02,
    }
    x = torch.randn(n_tokens, hid, generator=g).to(torch.bfloat16)
    cfg = dict(num_q_heads=Hq, num_kv_heads=Hk, head_dim=d, kernel_size=c["kernel_size"], kernel_stride=c["kernel_stride"],
               block_size=c["block_size"], topk=c["topk"], init_blocks=c["init_blocks"], local_blocks=c["local_blocks"],
               window_size=c["window_size"])
    inv = compute_inv_freq(RopeConfig(max_position_embeddings=131072, head_dim=d, rope_theta=c["rope_theta"]))
    t0 = time.perf_counter()
    layer_forward_ref(params, x, [n_tokens], cfg, inv)
    dt = time.perf_counter() - t0
    return n_tokens / dt, dt


def run_layer(args, dd, steps, sub=False):
    """Forward + backward of the whole FlashSparseAttention layer.  With N > 1 the heads are split over the ranks
    (8/N KV heads and 32/N query heads each: the attention kernels need no collective); the layer output and the
    gradient of the input are summed over the ranks with one NCCL all-reduce each, as any head-parallel layer does.
    Returns the record on rank 0 (None elsewhere)."""
    from fsa.module.fsa import FlashSparseAttention, RopeConfig

    rank, world, dev, dist = dd.rank, dd.world, dd.dev, dd.dist
    timed = dd.timed
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

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(dev.index)
    sampler.start()
    ms_step = timed(step, steps)
    clocks = sampler.stop()

    # the two all-reduces of a step, alone (layer output and dX, [tokens, hidden] bf16 each)
    ar_ms = None
    if world > 1:
        buf = torch.empty_like(xd)

        def reduces():
            dist.all_reduce(buf)
            dist.all_reduce(buf)

        reduces()
        ar_ms = timed(reduces, 3)

    # end to end: every step takes x and dy from pinned host memory and reads the norms of its results back; the copies of
    # step i + 1 run on a second stream into a second pair of device buffers while step i computes
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [[torch.empty_like(xd), torch.empty_like(dyd)] for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def issue_copy(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])          # the step that last used these buffers is done with them
            bufs[b][0].copy_(xh, non_blocking=True)
            bufs[b][1].copy_(dyh, non_blocking=True)
            copied[b].record(copy_stream)

    def e2e_run(n):
        out = None
        issue_copy(0)
        for i in range(n):
            if i + 1 < n:
                issue_copy(i + 1)
            b = i % 2
            torch.cuda.current_stream().wait_event(copied[b])
            y, gx = step(bufs[b][0], bufs[b][1])
            consumed[b].record()
            out = torch.stack([y.float().norm(), gx.float().norm()]).cpu()
        return out

    e2e_n = 0 if args.no_e2e else max(2, min(steps, 6))
    if e2e_n:
        e2e_run(2)
        copy_stream.synchronize()
        e2e_ms = timed(lambda: e2e_run(e2e_n), 1) / e2e_n
    line = None
    if rank == 0:
        flops = layer_useful_flops(c, seqlens)
        peak, peak_src = tensor_peak(burst=False)       # a step of tens of milliseconds, dozens of them back to back
        achieved = flops / world / (ms_step * 1e-3) / 1e12
        cpu = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, dt = layer_cpu_baseline(threads)
            cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                   "sample": f"layer oracle, forward only, one 512-token sequence with the layer's dimensions ({dt:.1f} s)"}
        line = {
            "metric": LAYER_METRIC, "value": N / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded N(0,1) hidden states, N(0,0.02) weights)",
            "config": {"workload": f"layer fwd+bwd: {len(seqlens)}x{seqlens[0]} tokens" + (" (small case)" if args.case == "small" else ""),
                       "parallelism": f"head-parallel x{world}: {c['Hk'] // world} KV heads per GPU, all-reduce of the output and of dX only",
                       "l2": "activations exceed L2", "useful_flops_per_step": flops},
            "tokens_per_s": N / (ms_step * 1e-3), "parallelism": f"head-parallel x{world}", "allreduce_ms": ar_ms,
            "roofline": {"bound": "tensor", "kernel": "whole step (library GEMMs + attention kernels)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None, "peak_source": peak_src},
            "cpu_baseline": cpu,
            "e2e": ({"value": N / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": 2 * xh.numel() * 2, "d2h_bytes_per_step": 8,
                     "overlap": "copies of step i+1 on a second stream while step i computes"} if e2e_n else None),
            "gpu_launches": None, "clocks": clocks,
        }
    del layer
    torch.cuda.empty_cache()
    return line


def shard_config1(rank, world, seqlens, Hk):
    """The (sequence, kv head) pairs of config 1 dealt to the ranks: by kv head while there are heads to deal, then by
    sequence.  Returns (kv heads of this rank, sequence indices of this rank)."""
    if world <= Hk:
        if Hk % world:
            raise SystemExit(f"--gpus must divide the {Hk} KV heads or be a multiple of them")
        per = Hk // world
        return list(range(rank * per, (rank + 1) * per)), list(range(len(seqlens)))
    if world % Hk or len(seqlens) % (world // Hk):
        raise SystemExit(f"--gpus {world}: cannot deal {Hk} KV heads x {len(seqlens)} sequences evenly")
    m = world // Hk
    per = len(seqlens) // m
    return [rank // m], list(range((rank % m) * per, (rank % m + 1) * per))


def run_sel(args, dd):
    """The headline: selected attention forward + backward on config 1 (or --case small / cfg2)."""
    from ctypes import byref, c_float, c_int

    from fsa import _lib
    from fsa.ops import FSA_topk_sparse_attention
    from fsa.ops.FSA_topk_sparse_attention import sel_attn_bwd, sel_attn_fwd
    from fsa.synthetic import make_cu_seqlens, make_qkv, make_topk_idx

    rank, world, dev, dist = dd.rank, dd.world, dd.dev, dd.dist
    barrier = dd.barrier
    L = _lib.lib()
    seqlens, Hk, G, d, bs, T = (CFG[k] for k in ("seqlens", "Hk", "G", "d", "bs", "T"))
    if args.case == "small":
        seqlens = seqlens[:1]
    if args.case == "cfg2":
        seqlens, G, d = [65536], args.group, args.head_dim
    scale = d ** -0.5
    # the whole problem from one seed on every rank, then this rank's (sequence, kv head) pairs of it
    N_all = sum(seqlens)
    q, k, v, do = make_qkv(N_all, Hk * G, Hk, d, 43)
    idx = make_topk_idx(seqlens, Hk, T, bs, 43)
    flops_step = 14 * d * analytic_pairs(seqlens, Hk, G, bs, T)          # of the WHOLE problem
    P_all = analytic_pairs(seqlens, Hk, G, bs, T)
    if world > 1:
        heads, seqs = shard_config1(rank, world, seqlens, Hk)
        starts = [sum(seqlens[:i]) for i in range(len(seqlens))]
        tok = torch.cat([torch.arange(starts[i], starts[i] + seqlens[i]) for i in seqs])
        qh = [h * G + g for h in heads for g in range(G)]
        q, do = q[tok][:, qh].contiguous(), do[tok][:, qh].contiguous()
        k, v = k[tok][:, heads].contiguous(), v[tok][:, heads].contiguous()
        idx = idx[heads][:, tok].contiguous()
        seqlens_r, Hk_r = [seqlens[i] for i in seqs], len(heads)
    else:
        seqlens_r, Hk_r = seqlens, Hk
    P_r = analytic_pairs(seqlens_r, Hk_r, G, bs, T)
    cu = make_cu_seqlens(seqlens_r)
    host = [x.pin_memory() for x in (q, k, v, do, idx)]
    qd, kd, vd, dod, idxd = (x.to(dev) for x in host)
    cud = cu.to(dev)

    def step():
        o, lse, ws = sel_attn_fwd(qd, kd, vd, idxd, bs, cud, scale)
        return sel_attn_bwd(qd, kd, vd, o, lse, dod, idxd, bs, cud, scale, ws)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    sampler = ClockSampler(dev.index)
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
    ms_step = dd.max_ms(ev0.elapsed_time(ev1)) / args.steps
    # per-kernel durations recorded inside the timed region (library-owned events around each launch, this rank's)
    kern = {}
    for name, kid in (("sel_fwd_main", 0), ("sel_fwd_reduce", 1), ("sel_bwd_main", 2), ("sel_bwd_dq_reduce", 3), ("sel_index_build", 4)):
        ms, n = c_float(0), c_int(0)
        _lib.check(L.fsa_profile_read(kid, byref(ms), byref(n)), "fsa_profile_read")
        kern[name] = {"ms_avg": (ms.value / n.value if n.value else None), "launches": n.value}
    L.fsa_profile_enable(0)
    value = flops_step / (ms_step * 1e-3) / 1e12

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
        qh_, kh_, vh_, doh_, ih_ = dev_bufs[b]
        qh_, kh_, vh_ = (x.detach().requires_grad_(True) for x in (qh_, kh_, vh_))
        o = FSA_topk_sparse_attention(qh_, kh_, vh_, ih_, bs, cud, scale)
        o.backward(doh_)
        res_host[b].copy_(torch.stack([qh_.grad.float().norm(), kh_.grad.float().norm(), vh_.grad.float().norm()]), non_blocking=True)
        consumed[b].record(cur)

    def e2e_run(n):
        issue_copy(0)
        for i in range(n):
            if i + 1 < n:
                issue_copy(i + 1)
            compute(i)

    e2e_ms = None
    if not args.no_e2e:
        e2e_run(2)
        barrier()
        ev0.record()
        copy_stream.wait_event(ev0)
        e2e_run(e2e_steps)
        ev1.record()
        barrier()
        e2e_ms = dd.max_ms(ev0.elapsed_time(ev1)) / e2e_steps
    h2d = sum(x.numel() * x.element_size() for x in host) * world       # all ranks' shards: the whole problem

    line = None
    if rank == 0:
        # the timed region is tens of milliseconds at full clocks: the burst figure is the denominator
        peak_tf, peak_src = tensor_peak(burst=True)
        # dominant kernel: the backward main kernel (10*d*P useful FLOPs per launch, P of this rank's shard)
        dom = "sel_bwd_main" if (kern["sel_bwd_main"]["ms_avg"] or 0) >= (kern["sel_fwd_main"]["ms_avg"] or 0) else "sel_fwd_main"
        dom_flops = (10 if dom == "sel_bwd_main" else 4) * d * P_r
        dom_ms = kern[dom]["ms_avg"]
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12 if dom_ms else None
        cpu = None
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tf, dt = cpu_baseline_config0(threads)
            cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"fp32 oracle FORWARD on config 0 (1x8192 tokens, 4 KV heads, G=1), best of 3 ({dt:.1f} s), on 4*d*P useful FLOPs"}
        wl = workload_name() if args.case == "cfg1" else ("small: 1x16384 tokens of cfg1" if args.case == "small" else
                                                          f"cfg2: 1x65536 tokens, 4 KV heads, G={G}, d={d}, B_K=64, T=16, fwd+bwd")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded N(0,1) q/k/v/dO, seeded causal block ids)",
            "config": {"workload": wl,
                       "parallelism": (f"the problem's (sequence, kv head) pairs dealt to {world} GPUs "
                                       f"({Hk_r} kv head(s) x {len(seqlens_r)} sequence(s) each), no collective") if world > 1 else "one GPU",
                       "l2": "inputs and partial buffers exceed L2 (q 134 MB, partials > 4 GB per step)",
                       "useful_flops_per_step": flops_step, "tokens_per_s": N_all / (ms_step * 1e-3)},
            "kernels": kern,
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": (achieved / peak_tf if achieved else None),
                         "traffic": (NCU_TRAFFIC_SMALL[dom] * (4 if args.case == "cfg1" else 1) * P_r / P_all) if args.case != "cfg2" else None,
                         "traffic_source": "ncu capture of the small case scaled by the token count", "peak_source": peak_src},
            "cpu_baseline": cpu,
            "e2e": ({"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 12 * world,
                     "overlap": "copies of step i+1 on a second stream while step i computes"} if e2e_ms else None),
            # kernels of this library per step: 5 of the index build, forward main + merge, delta, backward main,
            # dQ merge, dK/dV slab reduce (the two memsets of dk / dv are not kernels)
            "gpu_launches": 11 * args.steps,
            "clocks": clocks,
        }
    del qd, kd, vd, dod, idxd, dev_bufs, host
    torch.cuda.empty_cache()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="sel_attn", choices=["sel_attn", "decode", "layer"],
                    help="sel_attn (default): selected attention fwd+bwd, the headline, with the layer and the decode step as "
                         "sub-records; decode: one NSA decode step alone; layer: the whole NSA layer fwd+bwd alone")
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
    ap.add_argument("--no-sub", action="store_true", help="sel_attn workload: skip the layer and decode sub-records")
    ap.add_argument("--no-graph", action="store_true", help="decode workload: launch the step's kernels one by one")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    dd = Dist(rank, world, local_rank)
    if args.workload == "decode":
        line = run_decode(args, dd, args.steps)
    elif args.workload == "layer":
        line = run_layer(args, dd, args.steps)
    else:
        line = run_sel(args, dd)
        if not args.no_sub and args.case == "cfg1":
            # the quantities the reference's headline also names, measured in the same process group
            sub_l = run_layer(args, dd, max(2, min(args.steps, 5)), sub=True) if LAYER_CFG["Hk"] % world == 0 else None
            sub_d = run_decode(args, dd, args.steps, sub=True)
            if rank == 0:
                keep_l = ("tokens_per_s", "ms_per_step", "n_gpus", "parallelism", "allreduce_ms", "roofline", "cpu_baseline", "e2e", "config")
                keep_d = ("tokens_per_s", "ms_per_step", "n_gpus", "step_gbs", "frac_hbm", "allgather_ms", "roofline", "cpu_baseline", "e2e",
                          "config", "cuda_graph")
                line["layer"] = {k: sub_l[k] for k in keep_l} if sub_l else None
                line["decode"] = {k: sub_d[k] for k in keep_d} if sub_d else None
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    dd.close()


if __name__ == "__main__":
    main()
