#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one causal prefill forward over the headline workload (bf16, B=4 per GPU, Hq=Hkv=32,
L=4096, D=128: 5.498e11 algorithmic FLOP). With N > 1 (launched by torchrun, one rank per GPU) the
global batch is 4*N; the (batch, kv head) units are split over the ranks by
``torch_mlu_b200.sharding.partition_units`` and each rank runs the units it owns (weak scaling; attention
is independent per unit, so the data path needs no collective). Rank 0 prints ONE JSON line.

`value`   : whole-job TFLOP/s with inputs resident in HBM (CUDA events, max over ranks).
`e2e`     : same metric with HOST tensors through torch_mlu_b200.host_pipeline.HostPipeline: every step
            copies its q, k, v from pinned host memory and reads out + logsumexp back, all inside the
            timed region; consecutive steps overlap on a copy-in, a compute and a copy-out stream.
            `copy_ceiling` beside it is the same loop with the copies only.
`roofline`: dominant kernel vs the measured dense-bf16 peak in MEASURED_PEAKS.json.
`sustained`: the headline step repeated for about two seconds, against the sustained peak.
`gathered`: (N > 1) the step followed by the all-gather that reassembles the outputs on every rank, the
            gather of step i running on a side stream under the kernel of step i+1.
`cpu_baseline` / `--impl reference`: torch's CPU fused SDPA in fp32 (the host-runnable reference path)
            on the same per-GPU workload, all host threads.
`also`    : forward+backward (also with dropout), head_dim 256, varlen GQA, split-KV decode (and at N > 1 their
            sharded forms and the ring / context-parallel prefill of one long sequence: send/receive with a sweep
            of the SMs left to it, and from four GPUs up the peer-copy transport; `--ring-only` measures just that).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "SDPA TFLOP/s per B200 (fwd, fwd+bwd) at 1/2/4/8 GPUs; decode HBM GB/s"
WORKLOAD = "bf16 causal prefill forward B=4 per GPU Hq=Hkv=32 L=4096 D=128 (batch slice r drawn from seed 1+r)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per launch of the prefill kernel on the headline workload: 2 x the 316 MB an ncu capture of half the
# batch measured (profiles/fwd_prefill_kernel_b2_h32_l4096_causal.md; traffic grows in proportion to the batch)
NCU_TRAFFIC_BYTES = {"prefill_c2": 6.32e8}
PER_GPU_BATCH = 4


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def bench_config(world: int) -> dict:
    """The `config` object; both arms print the same one."""
    return {"workload": WORKLOAD, "per_gpu_batch": PER_GPU_BATCH, "global_batch": PER_GPU_BATCH * world,
            "l2": "inputs 384 MiB per step > 126 MB L2, no flush",
            "parallelism": f"(batch, kv head) units sharded x{world}"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) in a thread
    while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index = index
        self.period_s = period_s
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                try:
                    idx = int(visible.split(",")[self.index])
                except ValueError:
                    idx = self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
        except Exception:
            self.nvml = None
            return self
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def _run(self):
        nv = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((mhz, reasons))
            except Exception:
                break
            time.sleep(self.period_s)

    def stop(self):
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                "hw_power_brake_slowdown": 0x80}
        seen = set()
        for _, r in self.samples:
            for name, bit in bits.items():
                if r & bit:
                    seen.add(name)
        mhz = [m for m, _ in self.samples]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(mhz)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------
# CPU reference arm
# ------------------------------------------------------------------------------------------
def host_threads() -> int:
    """Every core this process may run on. torchrun exports OMP_NUM_THREADS=1 to its children; the CPU arm sets
    its thread count itself so that it is the same at every N."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_steps(steps: int, warmup: int, budget_s: float):
    """torch CPU fused SDPA (fp32) on one GPU's share of the headline workload (B=4, H=32, L=4096, D=128, causal:
    the whole step of one rank), `warmup` untimed and `steps` timed repetitions, stopping early after `budget_s`
    seconds. Returns (info dict, seconds per step, steps timed)."""
    from oracle import sdpa_oracle as orc  # the checker doubles as the timed CPU baseline
    from torch_mlu_b200 import workloads
    threads = host_threads()
    torch.set_num_threads(threads)
    c = workloads.config2_causal_prefill(batch=PER_GPU_BATCH)
    q, k, v = c.q.float(), c.k.float(), c.v.float()
    flops = c.forward_flops()
    orc.cpu_sdpa_forward(q[:1, :2], k[:1, :2], v[:1, :2], causal=True, scale=c.softmax_scale)  # page in the kernel
    for _ in range(warmup):
        orc.cpu_sdpa_forward(q, k, v, causal=True, scale=c.softmax_scale)
    done = 0
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.cpu_sdpa_forward(q, k, v, causal=True, scale=c.softmax_scale)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    per_step = (time.perf_counter() - t0) / done
    info = {"value": flops / per_step / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"torch CPU fused SDPA fp32 on one GPU's whole step (B=4 H=32 L=4096 D=128 causal), {warmup} warm-up + "
                      f"{done} timed repetitions, {per_step:.3f} s each, {threads} threads of {os.cpu_count()} logical CPUs"}
    return info, per_step, done


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    world = max(world, args.gpus)
    info, per_step, done = cpu_reference_steps(args.steps, args.warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": info["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(world),
        "cpu_baseline": info,
        "e2e": {"value": info["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "one host runs one GPU's share of the global batch per step, at every N: the host does not grow with N",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class Job:
    """Rank, device and the reductions over ranks the measurements need."""

    def __init__(self):
        self.rank, self.world, self.local = dist_env()
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def sync(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return float(x)
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather_floats(self, x: float):
        if self.dist is None:
            return [float(x)]
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        out = torch.empty(self.world, device=self.dev, dtype=torch.float64)
        self.dist.all_gather_into_tensor(out, t)
        return [float(v) for v in out.tolist()]

    def timed(self, fn, steps, warmup, reduce=True):
        """ms per step of `fn` on the current stream: barrier + synchronize on both sides, CUDA events, max over ranks."""
        for _ in range(warmup):
            fn()
        self.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.sync()
        ms = e0.elapsed_time(e1) / steps
        return self.max_over_ranks(ms) if reduce else ms


def guarded(name, out, fn):
    """Run one secondary measurement; a failure is reported under its name instead of ending the run."""
    try:
        out[name] = fn()
    except Exception as e:  # say so, do not hide it
        out[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    torch.cuda.empty_cache()


def device_randn(dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    return lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)


def measure_fwd_bwd(job: Job, n: int):
    """Config 3 (B8 H16 L2048 D128 causal) forward + backward. At N > 1 the 128 (batch, head) units are also split
    over the ranks with sharding.partition_units (strong scaling: the whole job is one config-3 step)."""
    from torch_mlu_b200 import ops, sharding
    rn = device_randn(job.dev, 2)
    q, k, v, do = (rn(8, 16, 2048, 128) for _ in range(4))
    fwd_flops = 4.0 * 8 * 16 * 2048 * 2048 * 128 / 2
    sc = 128 ** -0.5

    def pair(q, k, v, do):
        o, lse = ops.gqa_prefill(q, k, v, is_causal=True)
        f = lambda: ops.gqa_prefill(q, k, v, is_causal=True)
        b = lambda: ops._dense_backward(do, q, k, v, o, lse, True, sc)
        bd = lambda: ops._dense_backward(do, q, k, v, o, lse, True, sc, deterministic=True)
        return f, b, bd

    f, b, bd = pair(q, k, v, do)
    ms_f, ms_b, ms_bd = job.timed(f, n, 3), job.timed(b, n, 3), job.timed(bd, n, 3)
    entry = {"workload": "bf16 causal B=8 H=16 L=2048 D=128", "fwd_ms": ms_f, "fwd_tflops": fwd_flops / ms_f / 1e9,
             "bwd_ms": ms_b, "bwd_tflops": 2.5 * fwd_flops / ms_b / 1e9,
             "fwd_bwd_tflops": 3.5 * fwd_flops / (ms_f + ms_b) / 1e9,
             "bwd_deterministic_ms": ms_bd, "bwd_deterministic_tflops": 2.5 * fwd_flops / ms_bd / 1e9}
    if job.world > 1:
        shards = sharding.partition_units(8 * 16, job.world)
        mine = shards[job.rank]
        ql, kl, vl = sharding.dense_shard_views(q, k, v, mine)
        dl = do.reshape(8 * 16, 1, 2048, 128)[mine.unit_begin:mine.unit_end]
        f, b, _ = pair(ql, kl, vl, dl)
        ms_fs, ms_bs = job.timed(f, n, 3), job.timed(b, n, 3)
        agg = 3.5 * fwd_flops / (ms_fs + ms_bs) / 1e9
        entry["sharded"] = {"units_per_rank": mine.unit_end - mine.unit_begin, "scaling": "strong", "fwd_ms": ms_fs, "bwd_ms": ms_bs,
                            "aggregate_tflops": agg, "per_gpu_tflops": agg / job.world,
                            "efficiency": agg / (job.world * entry["fwd_bwd_tflops"])}
    return entry


def measure_dropout(job: Job, n: int):
    """Config 3 with dropout through the operator pair, forward and backward alternating as in training: the forward
    draws the keep-masks (one extra kernel) and leaves them for its backward."""
    from torch_mlu_b200 import ops
    rn = device_randn(job.dev, 2)
    q, k, v, do = (rn(8, 16, 2048, 128) for _ in range(4))
    fwd_flops = 4.0 * 8 * 16 * 2048 * 2048 * 128 / 2
    fo = lambda: ops._scaled_dot_product_flash_attention(q, k, v, 0.1, True, False)

    def pair():
        r = fo()
        return ops._scaled_dot_product_flash_attention_backward(do, q, k, v, r[0], r[1], r[2], r[3], r[4], r[5], 0.1, True,
                                                                r[6], r[7])

    ms_f = job.timed(fo, n, 3)
    ms_pair = job.timed(pair, n, 3)
    torch.use_deterministic_algorithms(True)
    try:
        ms_pair_det = job.timed(pair, n, 3)
    finally:
        torch.use_deterministic_algorithms(False)
    return {"workload": "config 3 with dropout_p=0.1 through the operator pair, forward then backward (keep-mask kernel included)",
            "fwd_ms": ms_f, "fwd_bwd_ms": ms_pair, "fwd_bwd_tflops": 3.5 * fwd_flops / ms_pair / 1e9,
            "fwd_bwd_deterministic_ms": ms_pair_det, "fwd_bwd_deterministic_tflops": 3.5 * fwd_flops / ms_pair_det / 1e9}


def measure_head_dim_256(job: Job, n: int):
    """Causal forward and backward at head_dim 256 (B4 H16 L4096): the kernels that keep the stationary operand in
    tensor memory. Fractions are of the measured burst bf16 peak."""
    from torch_mlu_b200 import ops
    rn = device_randn(job.dev, 6)
    B, H, L, D = 4, 16, 4096, 256
    q, k, v, do = (rn(B, H, L, D) for _ in range(4))
    fwd_flops = 4.0 * B * H * L * L * D / 2
    o, lse = ops.gqa_prefill(q, k, v, is_causal=True)
    ms_f = job.timed(lambda: ops.gqa_prefill(q, k, v, is_causal=True), n, 3)
    ms_b = job.timed(lambda: ops._dense_backward(do, q, k, v, o, lse, True, D ** -0.5), n, 3)
    peak = float(load_peaks()["bf16_tflops"])
    f_tf, b_tf = fwd_flops / ms_f / 1e9, 2.5 * fwd_flops / ms_b / 1e9
    return {"workload": "bf16 causal B=4 H=16 L=4096 D=256", "fwd_ms": ms_f, "fwd_tflops": f_tf, "fwd_frac_of_peak": f_tf / peak,
            "bwd_ms": ms_b, "bwd_tflops": b_tf, "bwd_frac_of_peak": b_tf / peak,
            "fwd_bwd_tflops": 3.5 * fwd_flops / (ms_f + ms_b) / 1e9, "peak": peak}


def measure_varlen(job: Job, n: int):
    """Config 4 (16 packed sequences, Hq 32 / Hkv 8, causal). At N > 1 the 128 (sequence, kv head) units are packed
    onto the ranks by sharding.plan_varlen (longest first by L^2); each rank's units form one packed call with
    4 query heads over 1 KV head."""
    from torch_mlu_b200 import ops, sharding, workloads
    dev = job.dev
    lens = workloads.CONFIG4_SEQLENS
    total = sum(lens)
    cu_h = [0]
    for l in lens:
        cu_h.append(cu_h[-1] + l)
    cu = torch.tensor(cu_h, dtype=torch.int32, device=dev)
    rn = device_randn(dev, 3)
    q, k, v = rn(total, 32, 128), rn(total, 8, 128), rn(total, 8, 128)
    fl = sum(4.0 * 32 * l * l * 128 for l in lens) / 2
    f = lambda: ops._flash_attention_forward(q, k, v, cu, cu, max(lens), max(lens), 0.0, True, False)
    ms = job.timed(f, n, 3)
    entry = {"workload": "bf16 varlen GQA causal 16 seqs (34004 tokens) Hq=32 Hkv=8 D=128", "ms": ms, "tflops": fl / ms / 1e9}
    if job.world > 1:
        plan = sharding.plan_varlen(lens, 8, job.world)[job.rank]
        qs, ks, vs, cul = [], [], [], [0]
        for seq, h in plan:
            lo, hi = cu_h[seq], cu_h[seq + 1]
            qs.append(q[lo:hi, 4 * h:4 * h + 4])
            ks.append(k[lo:hi, h:h + 1])
            vs.append(v[lo:hi, h:h + 1])
            cul.append(cul[-1] + hi - lo)
        ql, kl, vl = torch.cat(qs).contiguous(), torch.cat(ks).contiguous(), torch.cat(vs).contiguous()
        cu_l = torch.tensor(cul, dtype=torch.int32, device=dev)
        mx = max(lens[s] for s, _ in plan)
        fs = lambda: ops._flash_attention_forward(ql, kl, vl, cu_l, cu_l, mx, mx, 0.0, True, False)
        ms_rank = job.timed(fs, n, 3, reduce=False)
        per_rank = job.gather_floats(ms_rank)
        ms_s = max(per_rank)
        agg = fl / ms_s / 1e9
        entry["sharded"] = {"units_per_rank": len(plan), "scaling": "strong", "ms": ms_s, "ms_per_rank": per_rank,
                            "time_imbalance_max_over_mean": ms_s / (sum(per_rank) / len(per_rank)),
                            "planned_imbalance": sharding.plan_imbalance(lens, 8, job.world),
                            "aggregate_tflops": agg, "per_gpu_tflops": agg / job.world,
                            "efficiency": agg / (job.world * entry["tflops"])}
    return entry


def measure_decode(job: Job, n: int):
    """Config 5 (B64 Lkv 32768 Hq32 Hkv8): at N > 1 each rank holds 64/N batch elements of the cache (strong scaling)."""
    from torch_mlu_b200 import ops
    dev = job.dev
    B, Hq, Hkv, Lk = 64 // job.world, 32, 8, 32768
    rn = device_randn(dev, 4 + job.rank)
    q = rn(B, Hq, 1, 128)
    k = torch.empty(B, Hkv, Lk, 128, device=dev, dtype=torch.bfloat16)
    v = torch.empty_like(k)
    for b in range(B):
        k[b] = rn(Hkv, Lk, 128)
        v[b] = rn(Hkv, Lk, 128)
    by = 2.0 * k.numel() * 2
    ms = job.timed(lambda: ops.decode_attention(q, k, v), n, 3)
    peaks = load_peaks()
    gbs = by / ms / 1e6
    return {"workload": f"bf16 split-KV decode B=64 Lq=1 Lkv=32768 Hq=32 Hkv=8 D=128, {B} batch elements per GPU "
                        f"({by / 2**30:.0f} GiB of K+V per GPU > L2)",
            "ms": ms, "hbm_gbs_per_gpu": gbs, "hbm_gbs": gbs * job.world, "frac_of_peak": gbs / peaks["hbm_gbs"],
            "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["_source"], "scaling": "strong"}


def measure_ring(job: Job, n: int):
    """Ring / context-parallel prefill of one long causal sequence (B=1 H=32 L=65536 D=128, zig-zag slices), N > 1 only:
    the whole hop loop, the same loop with the kernels only, and with the exchanges only."""
    import torch.distributed as dist
    from torch_mlu_b200 import ops, ring
    dev, W = job.dev, job.world
    L, H = 65536, 32
    Ls = L // W
    rn = device_randn(dev, 50 + job.rank)
    q, k, v = rn(1, H, Ls, 128), rn(1, H, Ls, 128), rn(1, H, Ls, 128)
    flops = 4.0 * H * L * L * 128 / 2
    # the hop's send/receive kernels need SMs beside the persistent forward kernel: sweep what it leaves them
    by_margin = {m: job.timed(lambda: ring.ring_prefill(q, k, v, is_causal=True, layout="zigzag", sm_margin=m), n, 2)
                 for m in (0, 8, 16, 32)}
    # The other transport: slices pulled by the copy engines through CUDA IPC mappings, hops ordered by stream memory
    # operations. It pays where a hop's kernels are shorter than its send/receive, i.e. from four GPUs up
    # (SDPA_BENCH_RING_PEER=1 measures it on two as well). Timed with local events and no collective inside, so that a
    # rank that runs into the transport's time limit cannot leave the others in a different collective; the one
    # all-reduce behind it is made by every rank whatever happened.
    peer_ms, peer_error = None, "not measured on fewer than four GPUs (SDPA_BENCH_RING_PEER=1 forces it)"
    if W >= 4 or os.environ.get("SDPA_BENCH_RING_PEER") == "1":
        ok, ms_local = 1.0, 0.0
        try:
            peer_fn = lambda: ring.ring_prefill(q, k, v, is_causal=True, layout="zigzag", exchange="peer")
            for _ in range(2):
                peer_fn()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(n):
                peer_fn()
            t1.record()
            torch.cuda.synchronize()
            ms_local = t0.elapsed_time(t1) / n
        except Exception as e:  # say so, do not hide it
            ok, peer_error = 0.0, f"{type(e).__name__}: {str(e)[:200]}"
        agreed = torch.tensor([ok, -ms_local], dtype=torch.float32, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)  # every rank succeeded? and the slowest rank's time
        if agreed[0].item() == 1.0:
            peer_ms = -agreed[1].item()
            ring.release_peer_buffers()
        elif ok == 1.0:
            peer_error = "another rank could not complete the peer-copy ring"
    best = min(by_margin, key=by_margin.get)
    ms_full = by_margin[best]
    transport = "NCCL send/recv"
    if peer_ms is not None and peer_ms < ms_full:
        ms_full, best, transport = peer_ms, 0, "peer copies (CUDA IPC)"
    no_comm = lambda: ring.ring_prefill(q, k, v, is_causal=True, layout="zigzag", exchange=False)
    ms_kernels = job.timed(no_comm, n, 2)
    nxt, prv = (job.rank + 1) % W, (job.rank - 1) % W
    kb, vb = torch.empty_like(k), torch.empty_like(v)

    def comm_only():
        for _ in range(W - 1):
            reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, k, nxt), dist.P2POp(dist.isend, v, nxt),
                                           dist.P2POp(dist.irecv, kb, prv), dist.P2POp(dist.irecv, vb, prv)])
            for r in reqs:
                r.wait()

    ms_comm = job.timed(comm_only, n, 2)
    hop_bytes = 2 * k.numel() * 2
    hidden = (ms_kernels + ms_comm - ms_full) / ms_comm if ms_comm > 0 else None
    return {"workload": f"ring prefill bf16 causal B=1 H=32 L=65536 D=128, zig-zag slices of {Ls} rows per GPU",
            "ms": ms_full, "transport": transport, "sm_margin": best, "ms_by_sm_margin": by_margin,
            "ms_peer_copies": peer_ms if peer_ms is not None else peer_error,
            "aggregate_tflops": flops / ms_full / 1e9, "per_gpu_tflops": flops / ms_full / 1e9 / W,
            "kernels_only_ms": ms_kernels, "exchange_only_ms": ms_comm, "hops": W - 1,
            "exchange_ms_per_hop": ms_comm / (W - 1), "kernel_ms_per_hop": ms_kernels / W,
            "exchange_gbs_per_gpu_per_direction": hop_bytes * (W - 1) / ms_comm / 1e6,
            "fraction_of_exchange_hidden": hidden}


def run_ours(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    job = Job()
    rank, world, dev = job.rank, job.world, job.dev
    from torch_mlu_b200 import _cabi, ops, sharding, workloads
    from torch_mlu_b200.host_pipeline import HostPipeline
    _cabi.load()
    if args.ring_only:
        # the long-sequence ring alone, both transports (not the bench line: a separate, short measurement)
        os.environ["SDPA_BENCH_RING_PEER"] = "1"
        if world < 2:
            raise SystemExit("bench.py --ring-only needs --gpus 2 or more")
        res = measure_ring(job, max(3, min(args.steps, 6)))
        job.sync()
        if rank == 0:
            print(json.dumps({"ring": res, "n_gpus": world}), flush=True)
        job.dist.destroy_process_group()
        return

    # The global batch is 4 * world; batch slice r is the seeded config-2 draw with seed 1 + r (slice 0 is the
    # BASELINE recipe itself). partition_units splits the global (batch, kv head) units; a rank draws what it owns.
    heads = 32
    shards = sharding.partition_units(PER_GPU_BATCH * world * heads, world)
    mine = shards[rank]
    assert (mine.unit_begin, mine.unit_end) == (rank * PER_GPU_BATCH * heads, (rank + 1) * PER_GPU_BATCH * heads)
    case = workloads.config2_causal_prefill(batch=PER_GPU_BATCH, seed=1 + rank)
    qh, kh, vh = case.q.pin_memory(), case.k.pin_memory(), case.v.pin_memory()
    q, k, v = qh.to(dev), kh.to(dev), vh.to(dev)
    flops = case.forward_flops()
    scale = case.softmax_scale

    def step():
        return ops.gqa_prefill(q, k, v, is_causal=True, scale=scale)

    # ---- device-resident timing (value, roofline)
    for _ in range(args.warmup):
        step()
    job.sync()
    launches0 = _cabi.launch_count()
    sampler = ClockSampler(job.local).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    job.sync()
    clocks = sampler.stop()
    launches = _cabi.launch_count() - launches0
    status = ops.device_status()
    ms_per_step = job.max_over_ranks(e0.elapsed_time(e1)) / args.steps
    value = world * flops / ms_per_step / 1e9  # TFLOP/s, whole job

    # ---- the same step for about two seconds: what a loop that runs under the power cap gets
    reps = max(args.steps, int(args.sustained_seconds * 1000.0 / ms_per_step))
    sampler = ClockSampler(job.local, period_s=0.02).start()
    ms_sus = job.timed(step, reps, 0)
    sus_clocks = sampler.stop()
    peaks = load_peaks()
    sus_tflops = flops / ms_sus / 1e9
    sustained = {"seconds": reps * ms_sus / 1e3, "steps": reps, "ms_per_step": ms_sus, "per_gpu_tflops": sus_tflops,
                 "peak": float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])),
                 "peak_source": f"{peaks['_source']} sustained cuBLAS bf16", "clocks": sus_clocks,
                 "ms_times_mhz": (ms_sus * sus_clocks["sm_mhz"]) if sus_clocks["sm_mhz"] else None}
    sustained["frac"] = sus_tflops / sustained["peak"]

    # ---- end to end: host tensors in, host results out, every step (double-buffered copy / compute / copy pipeline)
    out_h = torch.empty((PER_GPU_BATCH, 4096, heads, 128), dtype=torch.bfloat16).pin_memory()
    lse_h = torch.empty((PER_GPU_BATCH, heads, 4096), dtype=torch.float32).pin_memory()
    pipe = HostPipeline(dev, is_causal=True, scale=scale)
    host_out = [(out_h, lse_h), (torch.empty_like(out_h).pin_memory(), torch.empty_like(lse_h).pin_memory())]
    e2e_count = [0]

    def e2e_step():
        oh, lh = host_out[e2e_count[0] % 2]
        e2e_count[0] += 1
        pipe.submit(qh, kh, vh, oh, lh)

    def pipelined(fn, steps, join):
        for _ in range(2):
            fn()
        join()
        job.sync()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        join()  # the timing events sit on the current stream
        ev1.record()
        job.sync()
        return job.max_over_ranks(ev0.elapsed_time(ev1)) / steps

    e2e_steps = max(4, min(args.steps, 10))
    e2e_ms = pipelined(e2e_step, e2e_steps, pipe.join)
    h2d = 3 * qh.numel() * 2
    d2h = out_h.numel() * 2 + lse_h.numel() * 4

    # the ceiling of that loop: the same three host-to-device copies per step and nothing else, on every rank at once
    copy_stream = torch.cuda.Stream(dev)
    sink = [torch.empty_like(q) for _ in range(3)]

    def copy_step():
        with torch.cuda.stream(copy_stream):
            for dst, src in zip(sink, (qh, kh, vh)):
                dst.copy_(src, non_blocking=True)

    copy_ms = pipelined(copy_step, e2e_steps, lambda: torch.cuda.current_stream().wait_stream(copy_stream))

    # ... and with the step's device-to-host copies (out, logsumexp) running beside them on a second stream: what the
    # host side of the box allows when both directions are busy on every rank, still without any kernel
    back_stream = torch.cuda.Stream(dev)
    o_dev = torch.empty((PER_GPU_BATCH, 4096, heads, 128), dtype=torch.bfloat16, device=dev)
    l_dev = torch.empty((PER_GPU_BATCH, heads, 4096), dtype=torch.float32, device=dev)

    def both_step():
        copy_step()
        with torch.cuda.stream(back_stream):
            out_h.copy_(o_dev, non_blocking=True)
            lse_h.copy_(l_dev, non_blocking=True)

    def both_join():
        torch.cuda.current_stream().wait_stream(copy_stream)
        torch.cuda.current_stream().wait_stream(back_stream)

    both_ms = pipelined(both_step, e2e_steps, both_join)
    del sink, o_dev, l_dev
    e2e = {"value": world * flops / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_ms,
           "copy_ceiling": {"what": "the step's three pinned host-to-device copies alone, all ranks at once",
                            "ms_per_step": copy_ms, "h2d_gbs_per_rank": h2d / copy_ms / 1e6,
                            "value_if_copy_bound": world * flops / copy_ms / 1e9,
                            "e2e_over_ceiling": copy_ms / e2e_ms,
                            "both_directions_ms_per_step": both_ms,
                            "e2e_over_both_directions": both_ms / e2e_ms}}

    # ---- N > 1: the step plus the reassembly of the outputs on every rank, gather i under kernel i+1
    gathered = None
    allgather_ms = None
    if job.dist is not None:
        dist = job.dist
        side = torch.cuda.Stream(dev)
        bufs = [torch.empty((world, PER_GPU_BATCH, 4096, heads, 128), dtype=torch.bfloat16, device=dev) for _ in range(2)]

        def gathered_ms(margin):
            keep, works, cnt = [None, None], [None, None], [0]

            def gather_step():
                i = cnt[0] % 2
                cnt[0] += 1
                if works[i] is not None:
                    works[i].wait()  # the buffer's previous gather has finished (orders the current stream behind it)
                o, _ = ops.gqa_prefill(q, k, v, is_causal=True, scale=scale, sm_margin=margin)
                keep[i] = o
                done = torch.cuda.Event()
                done.record()
                with torch.cuda.stream(side):
                    side.wait_event(done)
                    works[i] = dist.all_gather_into_tensor(bufs[i], o.transpose(1, 2), async_op=True)

            def gather_join():
                for w in works:
                    if w is not None:
                        w.wait()
                torch.cuda.current_stream().wait_stream(side)

            return pipelined(gather_step, e2e_steps, gather_join)

        # the persistent kernel holds every SM it is given until its last unit is done; a collective's CTAs get in
        # beside it only on SMs it leaves free (sm_margin)
        by_margin = {m: gathered_ms(m) for m in (0, 8, 16, 32)}
        best = min(by_margin, key=by_margin.get)
        g_ms = by_margin[best]
        o, _ = step()
        oc = o.transpose(1, 2)
        allgather_ms = job.timed(lambda: dist.all_gather_into_tensor(bufs[0], oc), 5, 2)
        gathered = {"value": world * flops / g_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": g_ms, "sm_margin": best,
                    "ms_per_step_by_sm_margin": by_margin,
                    "allgather_alone_ms": allgather_ms, "kernel_alone_ms": ms_per_step,
                    "bytes_received_per_gpu": (world - 1) * oc.numel() * 2,
                    "what": "kernel + all_gather_into_tensor of out on a side stream, gather i under kernel i+1; the "
                            "kernel leaves sm_margin SMs to the collective"}
        del bufs

    # ---- secondary configurations
    also = {}
    cpu_info = None
    if not args.no_extras:
        del q, k, v, pipe
        torch.cuda.empty_cache()
        n = max(3, min(args.steps, 10))
        guarded("fwd_bwd", also, lambda: measure_fwd_bwd(job, n))
        if world == 1:
            guarded("fwd_bwd_dropout", also, lambda: measure_dropout(job, n))
            guarded("head_dim_256", also, lambda: measure_head_dim_256(job, n))
        guarded("varlen_gqa", also, lambda: measure_varlen(job, n))
        guarded("decode", also, lambda: measure_decode(job, n))
        if world > 1:
            guarded("ring", also, lambda: measure_ring(job, max(2, n // 2)))
        if rank == 0 and world == 1:
            cpu_info, _, _ = cpu_reference_steps(steps=40, warmup=1, budget_s=12.0)
    job.sync()

    if rank == 0:
        peak = float(peaks["bf16_tflops"])
        achieved = flops / ms_per_step / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world), "per_gpu_tflops": value / world,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES["prefill_c2"],
                         "traffic_source": "ncu capture of half the batch, scaled by 2 (profiles/)",
                         "peak_source": f"{peaks['_source']} burst cuBLAS bf16", "kernel": "fwd_prefill_kernel",
                         "algorithmic_flops_per_launch": flops, "frac_of_nominal_2250": achieved / 2250.0},
            "cpu_baseline": cpu_info,
            "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "device_status": status,
            "sustained": sustained, "gathered": gathered, "allgather_ms": allgather_ms, "also": also,
        }
        print(json.dumps(line), flush=True)
    if job.dist is not None:
        job.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs and the CPU baseline")
    ap.add_argument("--ring-only", action="store_true",
                    help="N > 1: measure only the ring prefill of one long sequence, with both transports")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the loop behind the `sustained` figure (a profiler run may want it short)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ and args.impl == "ours":
        # started by hand without torchrun: launch one rank per GPU on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
