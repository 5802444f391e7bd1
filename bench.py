#!/usr/bin/env python
"""Benchmark of the FP8 attention-forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--scaling weak|strong]
    python bench.py --impl reference ...      # the reference's CPU path on the host cores
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one forward over one batch of synthetic inputs (one kernel launch per
rank).  Rank 0 prints ONE JSON line.  `value` is aggregate attention-forward TFLOP/s
(4*B*H*S^2*D, halved for causal) with inputs resident in HBM; `e2e` is the same metric
through the operator with HOST tensors (pinned host -> device copies and the device ->
host copy of O inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_FP8_TFLOPS = 4500.0      # B200 dense FP8 (2x the 2250 dense bf16 figure)
FALLBACK_BF16_TFLOPS = 1590.0    # earlier measurement on this pool, used if MEASURED_PEAKS.json is absent
FALLBACK_HBM_GBS = 6650.0
DEFAULT_WORKLOAD = "mid_s4096_d128"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the default workload, from the
# ncu capture summarised under profiles/ (None until one has been taken).
NCU_TRAFFIC_BYTES = {
    # captured on mid_s4096_d128_b2 (64 slices): 100.74 MB read + 30.30 MB written (part of the
    # fp16 output is still dirty in L2 at kernel end); traffic is proportional to the slice count,
    # the bench workload has 8x the slices
    "mid_s4096_d128_b2": 131.0e6,
    "mid_s4096_d128": 8 * 131.0e6,
    "mid_s4096_d128_b2_causal": 128.6e6,
    "mid_s4096_d128_causal": 8 * 128.6e6,
    "prefill_s1024_d64": 129.9e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML while the timed
    region runs (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def cpu_attention_tflops(w, budget_s: float, max_slices: int, label: str):
    """Times the CPU restatement of the reference's naive attention (test.py:25-33, fp32)
    on a bounded sample of (batch, head) slices of workload `w`, all host threads."""
    from cutlass_flash_atten_fp8_b200 import synth
    from oracle.attention_oracle import attention_fp32
    torch.set_num_threads(os.cpu_count() or 1)
    n = min(max_slices, w.n_slices)
    q8, k8, v8, (dq, dk, dv) = synth.make_qkv(w, "cpu", 0, n, transpose_v=False)
    q8, k8, v8 = (t.view(1, n, w.seqlen, w.head_dim) for t in (q8, k8, v8))
    done, t0 = 0, time.perf_counter()
    while done < n:
        attention_fp32(q8[:, done:done + 1], k8[:, done:done + 1], v8[:, done:done + 1], w.causal, w.softmax_scale, dq, dk, dv)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return {"value": w.flops(done) / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{done} of {w.n_slices} (batch,head) slices of {label}, {dt:.1f} s, naive fp32 torch attention on dequantised inputs",
            "seconds_per_slice": dt / done}


def fp8_gemm_peak(device) -> float | None:
    """Burst FP8 GEMM rate of this GPU through torch._scaled_mm (cuBLASLt), 8192^3."""
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        return 2.0 * n ** 3 / best / 1e9
    except Exception:
        return None


def quantize_rate(device, peaks):
    """HBM rate of the fp16 -> e4m3 per-tensor quantisation pre-pass (two kernels, 5 bytes of
    algorithmic traffic per element) on a 1 GiB tensor; reported beside the attention result."""
    try:
        from cutlass_flash_atten_fp8_b200 import quantize_e4m3
        n = 512 * 1024 * 1024
        x = torch.randn(n // 4, device=device).half().repeat(4)
        for _ in range(2):
            quantize_e4m3(x)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            quantize_e4m3(x)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 5
        gbs = 5.0 * n / ms / 1e6
        return {"elements": n, "ms": ms, "algorithmic_gbs": gbs, "hbm_peak_gbs": peaks["hbm_gbs"], "frac": gbs / peaks["hbm_gbs"]}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}


def reference_kernel_tflops(w, q8, k8, vt8, steps: int):
    """Optional: the reference's own Ada kernel (built by oracle/build_ref.sh into oracle/_ref,
    sm_89 PTX assembled for sm_100) timed on this GPU on the same inputs.  Reported beside the
    result; not part of `value`."""
    import glob
    import importlib.util
    sos = glob.glob(os.path.join(ROOT, "oracle", "_ref", "attention_cutlass_fp8_ref*.so"))
    if not sos:
        return {"unavailable": "oracle/_ref not built"}
    try:
        spec = importlib.util.spec_from_file_location("attention_cutlass_fp8_ref", sos[0])
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        for _ in range(2):
            mod.flash_attention_v2_cutlass(q8, k8, vt8, w.causal, w.softmax_scale)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(2, min(steps, 5))
        e0.record()
        for _ in range(n):
            mod.flash_attention_v2_cutlass(q8, k8, vt8, w.causal, w.softmax_scale)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        return {"ms": ms, "tflops": w.flops(q8.shape[1]) / ms / 1e9, "note": "reference kernel, e4m3 output, includes its cudaDeviceSynchronize"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}


def run_reference_arm(args, w):
    """--impl reference: the reference's CPU path (naive torch attention in fp32, the CPU
    restatement of test.py:25-33) on the host cores; each step is a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # each step times a sample of the workload's slices; the whole run stays within ~3 minutes
    per_step_budget = max(0.5, min(5.0, 150.0 / max(1, args.warmup + args.steps)))
    vals = []
    for i in range(args.warmup + args.steps):
        r = cpu_attention_tflops(w, per_step_budget, w.n_slices, w.name)
        if i >= args.warmup:
            vals.append(r)
    v = sum(x["value"] for x in vals) / len(vals)
    ms = 1e3 * sum(x["seconds_per_slice"] for x in vals) / len(vals) * w.n_slices
    line = {
        "impl": "reference", "metric": "fp8_attn_fwd_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "batch": w.batch, "heads": w.heads, "seqlen": w.seqlen, "head_dim": w.head_dim,
                   "causal": w.causal, "note": "ms_per_step extrapolated from the sampled slices to the whole workload"},
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": vals[0]["cores"], "kind": "port", "sample": vals[0]["sample"]},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", action="store_true", help="also time the optional NCCL gather of O on rank 0")
    ap.add_argument("--v-layout", default="transposed", choices=["transposed", "natural"],
                    help="V as the reference passes it ([.., head_dim, seqlen]) or untransposed")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end, CPU-baseline, FP8-GEMM and reference-kernel legs (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from cutlass_flash_atten_fp8_b200 import synth
    w = synth.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    import torch.distributed as dist
    from cutlass_flash_atten_fp8_b200 import HostRunner, check_status, flash_attention_v2_cutlass
    from cutlass_flash_atten_fp8_b200.shard import gather_output, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    # Weak scaling: every rank owns a whole copy of the workload's slices (distinct seeds per
    # rank); strong scaling: the workload's slices are partitioned across the ranks.
    if args.scaling == "weak":
        lo, hi = 0, w.n_slices
        wl = synth.Workload(w.name, w.batch, w.heads, w.seqlen, w.head_dim, w.causal, w.outliers, w.seed + 17 * rank)
        total_slices = w.n_slices * world
    else:
        lo, hi = shard_range(w.n_slices, world, rank)
        wl = w
        total_slices = w.n_slices
    n_local = hi - lo
    natural = args.v_layout == "natural"
    q8, k8, vt8, (dq, dk, dv) = synth.make_qkv(wl, device, lo, hi, transpose_v=not natural)
    S, D = w.seqlen, w.head_dim
    q4, k4 = q8.view(1, n_local, S, D), k8.view(1, n_local, S, D)
    v4 = vt8.view(1, n_local, S, D) if natural else vt8.view(1, n_local, D, S)
    out = torch.empty((1, n_local, S, D), dtype=torch.float16, device=device)
    scale = w.softmax_scale * dq * dk

    def step():
        flash_attention_v2_cutlass(q4, k4, v4, w.causal, scale, o_scale=dv, out=out, v_layout=args.v_layout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    check_status(device)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    check_status(device)
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    tflops = w.flops(total_slices) / ms_step / 1e9
    tflops_gpu = tflops / world

    # Power settles over seconds on a 1 kW part: the same launch back to back for at least two
    # seconds, reported beside the K-step figure (rank 0 of a single-GPU run only).
    sustained = None
    if world == 1 and not args.kernel_only:
        n_sus = max(args.steps, int(2000.0 / ms_step) + 1)
        sampler2 = ClockSampler(local_rank)
        torch.cuda.synchronize()
        sampler2.start()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_sus):
            step()
        s1.record()
        torch.cuda.synchronize()
        clocks2 = sampler2.stop()
        check_status(device)
        ms_sus = s0.elapsed_time(s1) / n_sus
        sustained = {"steps": n_sus, "ms_per_step": ms_sus, "value": w.flops(total_slices) / ms_sus / 1e9,
                     "unit": "TFLOP/s", "clocks": clocks2}

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": "fp8_attn_fwd_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                              "config": {"workload": w.name}, "kernel_only": True, "clocks": clocks}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- end to end: host tensors in, host tensor out, copies inside the timed region
    runner = HostRunner(device)
    hq, hk, hv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (q4, k4, v4))
    for _ in range(2):
        runner(hq, hk, hv, w.causal, scale, o_scale=dv, v_layout=args.v_layout)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        runner(hq, hk, hv, w.causal, scale, o_scale=dv, v_layout=args.v_layout)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= args.e2e_steps
    h2d, d2h = runner.bytes_per_call(hq, hv, hk)
    e2e = {"value": w.flops(total_slices) / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world}

    gather_ms = None
    if args.gather and world > 1:
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        gather_output(out[0], n_local * world if args.scaling == "weak" else w.n_slices)
        g1.record()
        barrier()
        gather_ms = g0.elapsed_time(g1)

    if rank == 0:
        peaks = measured_peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        gemm = fp8_gemm_peak(device)
        line = {
            "metric": "fp8_attn_fwd_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": w.name, "batch": w.batch, "heads": w.heads, "seqlen": w.seqlen, "head_dim": w.head_dim,
                       "causal": w.causal, "outliers": w.outliers, "slices_per_gpu": n_local, "v_layout": args.v_layout,
                       "out_dtype": "fp16", "parallelism": f"(batch x head) shards x{world}, no collective",
                       "l2": f"inputs+output {w.hbm_bytes(n_local) / 1e6:.0f} MB per step exceed the 126 MB L2"},
            "tflops_per_gpu": tflops_gpu,
            "pct_of_fp8_peak_nominal": 100.0 * tflops_gpu / NOMINAL_FP8_TFLOPS,
            "fp8_gemm_tflops_measured": gemm,
            "pct_of_fp8_gemm_measured": (100.0 * tflops_gpu / gemm) if gemm else None,
            "algorithmic_hbm_gbs": w.hbm_bytes(n_local) / ms_step / 1e6,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": args.steps * world,
            "roofline": {"bound": "tensor", "achieved": tflops_gpu, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": tflops_gpu / fp8_peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                         "peak_source": f"2 x bf16 cuBLAS burst of {peaks['source']} ({peaks['bf16_tflops']:.0f} TF): FP8 issues at twice the bf16 rate",
                         "hbm": {"achieved_gbs": w.hbm_bytes(n_local) / ms_step / 1e6, "peak_gbs": peaks["hbm_gbs"]}},
        }
        if gather_ms is not None:
            line["gather_o_ms"] = gather_ms
        if sustained is not None:
            line["sustained"] = sustained
        if world == 1:
            line["quantize_prepass"] = quantize_rate(device, peaks)
            line["reference_kernel"] = (reference_kernel_tflops(w, q4, k4, v4, args.steps) if not natural
                                        else {"unavailable": "the reference kernel needs V transposed"})
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_attention_tflops(w, 12.0, w.n_slices, w.name)
                line["cpu_baseline"].pop("seconds_per_slice", None)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
