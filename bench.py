#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one causal prefill forward over the headline workload (bf16, B=4, Hq=Hkv=32,
L=4096, D=128, seed 1: 5.498e11 algorithmic FLOP). With N > 1 (launched by torchrun, one rank
per GPU) every rank runs that workload on its own batch slice (weak scaling; attention is
independent per batch x head, so the data path needs no collective - the all-gather that
reassembles outputs is timed separately). Rank 0 prints ONE JSON line.

`value`   : whole-job TFLOP/s with inputs resident in HBM (CUDA events, max over ranks).
`e2e`     : same metric with HOST tensors through torch_mlu_b200.host_pipeline.HostPipeline: every step
            copies its q, k, v from pinned host memory and reads out + logsumexp back, all inside the
            timed region; consecutive steps overlap on a copy-in, a compute and a copy-out stream.
`roofline`: dominant kernel vs the measured dense-bf16 peak in MEASURED_PEAKS.json.
`cpu_baseline` / `--impl reference`: torch's CPU fused SDPA in fp32 (the host-runnable
            reference path) on a bounded sample of the same workload, all host threads.
Secondary measurements (forward+backward config, varlen GQA config, split-KV decode GB/s) ride
along under "also".
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
WORKLOAD = "bf16 causal prefill forward B=4 Hq=Hkv=32 L=4096 D=128 (seed 1)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram bytes per launch of the prefill kernel on the headline workload, from the ncu capture
# summarised in profiles/ (None until a capture exists)
NCU_TRAFFIC_BYTES = {"prefill_c2": 6.32e8}  # 2 x 316 MB measured at half the batch (traffic scales with batch)


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


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) in a thread
    while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
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
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

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
            time.sleep(0.002)

    def stop(self):
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        nv = self.nvml
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
def cpu_reference_sample(budget_s: float = 12.0, max_reps: int = 400):
    """Times torch CPU fused SDPA (fp32) on one batch element of the headline workload
    (B=1, H=32, L=4096, D=128, causal: 1/4 of a step), repeated for about `budget_s` seconds.
    Returns (info, best seconds per repetition, FLOP per repetition)."""
    from oracle import sdpa_oracle as orc  # the checker doubles as the timed CPU baseline
    from torch_mlu_b200 import workloads
    c = workloads.config2_causal_prefill(batch=1)
    q, k, v = c.q.float(), c.k.float(), c.v.float()
    flops = c.forward_flops()
    orc.cpu_sdpa_forward(q[:, :2], k[:, :2], v[:, :2], causal=True, scale=c.softmax_scale)  # warm-up
    times = []
    t_start = time.perf_counter()
    for _ in range(max_reps):
        t0 = time.perf_counter()
        orc.cpu_sdpa_forward(q, k, v, causal=True, scale=c.softmax_scale)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    best = min(times)
    info = {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"torch CPU fused SDPA fp32, one batch element of the workload (B=1 H=32 L=4096 D=128 causal, "
                      f"1/4 step), best of {len(times)} repetitions over {sum(times):.1f} s, {best:.3f} s each; "
                      f"host has {os.cpu_count()} logical CPUs"}
    return info, best, flops


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    info, best, flops = cpu_reference_sample(budget_s=min(20.0, 2.0 * max(1, args.steps)), max_reps=400)
    line = {
        "impl": "reference", "metric": METRIC, "value": info["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": best * 4 * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "timed": "bounded sample: 1/4 step per repetition on host cores"},
        "cpu_baseline": info,
        "e2e": {"value": info["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def timed_loop(fn, steps, warmup, sync):
    for _ in range(warmup):
        fn()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    return e0.elapsed_time(e1)  # ms for all steps


def secondary_measurements(dev, steps):
    """Forward+backward, varlen-GQA and decode configs, a few launches each (not the headline)."""
    from torch_mlu_b200 import ops
    out = {}
    n = max(3, min(steps, 10))
    g = torch.Generator(device=dev).manual_seed(2)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    sync = torch.cuda.synchronize
    # config 3: B8 H16 L2048 causal forward + backward
    try:
        q, k, v, do = rn(8, 16, 2048, 128), rn(8, 16, 2048, 128), rn(8, 16, 2048, 128), rn(8, 16, 2048, 128)
        fwd_flops = 4.0 * 8 * 16 * 2048 * 2048 * 128 / 2
        o, lse = ops.gqa_prefill(q, k, v, is_causal=True)
        ms_f = timed_loop(lambda: ops.gqa_prefill(q, k, v, is_causal=True), n, 3, sync) / n
        entry = {"workload": "bf16 causal B=8 H=16 L=2048 D=128", "fwd_ms": ms_f, "fwd_tflops": fwd_flops / ms_f / 1e9}
        try:
            ms_b = timed_loop(lambda: ops._dense_backward(do, q, k, v, o, lse, True, 128 ** -0.5), n, 3, sync) / n
            entry.update({"bwd_ms": ms_b, "bwd_tflops": 2.5 * fwd_flops / ms_b / 1e9,
                          "fwd_bwd_tflops": 3.5 * fwd_flops / (ms_f + ms_b) / 1e9})
        except Exception as e:  # backward kernel absent or failing: say so, do not hide it
            entry["bwd_error"] = str(e)[:200]
        out["fwd_bwd"] = entry
        # the same step with dropout through the operator pair: each call also makes its keep-masks
        try:
            fo = lambda: ops._scaled_dot_product_flash_attention(q, k, v, 0.1, True, False)
            r = fo()
            bo = lambda: ops._scaled_dot_product_flash_attention_backward(do, q, k, v, r[0], r[1], r[2], r[3], r[4], r[5], 0.1,
                                                                         True, r[6], r[7])
            ms_fd, ms_bd = timed_loop(fo, n, 3, sync) / n, timed_loop(bo, n, 3, sync) / n
            out["fwd_bwd_dropout"] = {"workload": "the same with dropout_p=0.1 (mask kernel included in both)", "fwd_ms": ms_fd,
                                      "bwd_ms": ms_bd, "fwd_bwd_tflops": 3.5 * fwd_flops / (ms_fd + ms_bd) / 1e9}
            del r
        except Exception as e:
            out["fwd_bwd_dropout"] = {"error": str(e)[:200]}
        del q, k, v, do, o, lse
    except Exception as e:
        out["fwd_bwd"] = {"error": str(e)[:200]}
    # config 4: varlen GQA causal
    try:
        from torch_mlu_b200 import workloads
        lens = workloads.CONFIG4_SEQLENS
        total = sum(lens)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        cu = cu.to(dev)
        q, k, v = rn(total, 32, 128), rn(total, 8, 128), rn(total, 8, 128)
        fl = sum(4.0 * 32 * l * l * 128 for l in lens) / 2
        f = lambda: ops._flash_attention_forward(q, k, v, cu, cu, max(lens), max(lens), 0.0, True, False)
        ms = timed_loop(f, n, 3, sync) / n
        out["varlen_gqa"] = {"workload": "bf16 varlen GQA causal 16 seqs (34004 tokens) Hq=32 Hkv=8 D=128", "ms": ms,
                             "tflops": fl / ms / 1e9}
        del q, k, v
    except Exception as e:
        out["varlen_gqa"] = {"error": str(e)[:200]}
    # config 5: split-KV decode
    try:
        B, Hq, Hkv, Lk = 64, 32, 8, 32768
        q = rn(B, Hq, 1, 128)
        k = torch.empty(B, Hkv, Lk, 128, device=dev, dtype=torch.bfloat16)
        v = torch.empty_like(k)
        for b in range(B):
            k[b] = rn(Hkv, Lk, 128)
            v[b] = rn(Hkv, Lk, 128)
        by = 2.0 * k.numel() * 2
        ms = timed_loop(lambda: ops.decode_attention(q, k, v), n, 3, sync) / n
        peaks = load_peaks()
        out["decode"] = {"workload": "bf16 split-KV decode B=64 Lq=1 Lkv=32768 Hq=32 Hkv=8 D=128 (8 GiB K+V > L2)",
                         "ms": ms, "hbm_gbs": by / ms / 1e6, "frac_of_peak": by / ms / 1e6 / peaks["hbm_gbs"],
                         "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["_source"]}
        del q, k, v
    except Exception as e:
        out["decode"] = {"error": str(e)[:200]}
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from torch_mlu_b200 import _cabi, ops, workloads
    _cabi.load()

    # every rank draws the same seeded workload; rank r owns batch slice r of a global batch 4*N
    case = workloads.config2_causal_prefill()
    qh, kh, vh = case.q.pin_memory(), case.k.pin_memory(), case.v.pin_memory()
    q, k, v = qh.to(dev), kh.to(dev), vh.to(dev)
    flops = case.forward_flops()
    scale = case.softmax_scale

    def sync():
        torch.cuda.synchronize()
        if use_dist:
            dist.barrier()
            torch.cuda.synchronize()

    def step():
        return ops.gqa_prefill(q, k, v, is_causal=True, scale=scale)

    # ---- device-resident timing (value, roofline)
    sampler = ClockSampler(local)
    for _ in range(args.warmup):
        step()
    sync()
    launches0 = _cabi.launch_count()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync()
    clocks = sampler.stop()
    launches = _cabi.launch_count() - launches0
    status = ops.device_status()
    total_ms = e0.elapsed_time(e1)
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * flops / ms_per_step / 1e9  # TFLOP/s, whole job

    # ---- end to end: host tensors in, host results out, every step
    out_h = torch.empty((4, 4096, 32, 128), dtype=torch.bfloat16).pin_memory()
    lse_h = torch.empty((4, 32, 4096), dtype=torch.float32).pin_memory()

    # Double-buffered copy / compute / copy pipeline (torch_mlu_b200.host_pipeline): every step still
    # moves its q, k, v in and its out, lse out; consecutive steps overlap on three streams. Each
    # step writes its own pair of host result buffers (two pairs, reused alternately).
    from torch_mlu_b200.host_pipeline import HostPipeline
    pipe = HostPipeline(dev, is_causal=True, scale=scale)
    host_out = [(out_h, lse_h), (torch.empty_like(out_h).pin_memory(), torch.empty_like(lse_h).pin_memory())]
    e2e_count = [0]

    def e2e_step():
        oh, lh = host_out[e2e_count[0] % 2]
        e2e_count[0] += 1
        pipe.submit(qh, kh, vh, oh, lh)

    def e2e_sync():
        pipe.join()  # the timing events sit on the current stream
        sync()

    e2e_steps = max(4, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_sync()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    pipe.join()
    ev1.record()
    e2e_sync()
    e2e_ms = ev0.elapsed_time(ev1)
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    h2d = 3 * qh.numel() * 2
    d2h = out_h.numel() * 2 + lse_h.numel() * 4

    # ---- output reassembly across ranks (not part of `value`)
    allgather_ms = None
    if use_dist:
        o, lse = step()
        o_c = o.transpose(1, 2).contiguous()
        gathered = torch.empty((world,) + tuple(o_c.shape), dtype=o_c.dtype, device=dev)
        ag = lambda: dist.all_gather_into_tensor(gathered, o_c)
        allgather_ms = timed_loop(ag, 5, 2, sync) / 5
        del gathered

    also = {}
    cpu_info = None
    if rank == 0 and world == 1 and not args.no_extras:
        del q, k, v
        torch.cuda.empty_cache()
        also = secondary_measurements(dev, args.steps)
        cpu_info, _, _ = cpu_reference_sample()
    if use_dist:
        dist.barrier()

    if rank == 0:
        peaks = load_peaks()
        peak = float(peaks["bf16_tflops"])
        achieved = flops / ms_per_step / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_batch": 4, "global_batch": 4 * world,
                       "l2": "inputs 384 MiB per step > 126 MB L2, no flush", "parallelism": f"batch-sharded x{world}",
                       "per_gpu_tflops": value / world},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES["prefill_c2"],
                         "peak_source": f"{peaks['_source']} burst cuBLAS bf16", "kernel": "fwd_prefill_kernel",
                         "algorithmic_flops_per_launch": flops, "frac_of_nominal_2250": achieved / 2250.0},
            "cpu_baseline": cpu_info,
            "e2e": {"value": world * flops / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks, "device_status": status,
            "allgather_ms": allgather_ms, "also": also,
        }
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs and the CPU baseline")
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
