#!/usr/bin/env python
"""Benchmark of the FP8 attention-forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--scaling weak|strong]
    python bench.py --impl reference ...      # the reference's CPU path on the host cores
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one forward over one batch of synthetic inputs (one kernel launch per
rank).  Rank 0 prints ONE JSON line.  `value` is aggregate attention-forward TFLOP/s
(4*B*H*S^2*D, halved for causal) with inputs resident in HBM; `e2e` is the same metric
through the operator with HOST tensors (pinned host -> device copies and the device ->
host copy of O inside the timed region), with the busy time of each stage per rank.

Beside the headline the line carries: `sustained` (the same launch for two seconds), `strong`
(the box-scale causal workload, its 2 048 slices partitioned over the N ranks) and, for N > 1,
`gather_o_ms` (the optional NCCL gather of that workload's O on rank 0); at N = 1 also
`reference_protocol` (the 18 shapes of the reference's own benchmark, test.py:93-100, this
kernel beside the reference's kernel where oracle/_ref is built, timed with CUDA events and
with the reference's wall-clock-plus-synchronise method, test.py:36-46), `quantize_prepass`,
`reference_kernel` and `cpu_baseline`.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_FP8_TFLOPS = 4500.0      # B200 dense FP8 (2x the 2250 dense bf16 figure)
FALLBACK_BF16_TFLOPS = 1590.0    # cuBLAS bf16 burst of a B200, used if MEASURED_PEAKS.json is absent
FALLBACK_HBM_GBS = 6650.0
DEFAULT_WORKLOAD = "mid_s4096_d128"
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised
# under profiles/.  A full-size launch is too large to capture with many passes, so the
# batch-2 cut of the same shape (64 slices instead of 512) was captured and the figure of the
# full workload is that capture times 8: traffic is proportional to the number of slices.
NCU_TRAFFIC_BYTES = {
    # captured on mid_s4096_d128_b2 (64 slices): 100.74 MB read + 36.30 MB written (part of the
    # fp16 output is still dirty in L2 at kernel end); traffic is proportional to the slice count,
    # the bench workload has 8x the slices
    "mid_s4096_d128_b2": 137.0e6,
    "mid_s4096_d128": 8 * 137.0e6,
    "mid_s4096_d128_b2_causal": 134.9e6,
    "mid_s4096_d128_causal": 8 * 134.9e6,
    "prefill_s1024_d64": 134.8e6,
    "mid_s4096_d256_b2": 137.8e6,
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

    def __init__(self, index: int, period_s: float = 0.005):
        # `index` is the CUDA ordinal; NVML numbers the GPUs of the whole machine and ignores
        # CUDA_VISIBLE_DEVICES, so the handle is looked up by the device's UUID
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
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


CPU_SAMPLE_SLICES = 16


def cpu_sample(w):
    """The first CPU_SAMPLE_SLICES (batch, head) slices of workload `w` as host tensors, drawn
    once (the generator's two passes over 512 slices on the host would cost more than the
    timing itself)."""
    from cutlass_flash_atten_fp8_b200 import synth
    n = min(CPU_SAMPLE_SLICES, w.n_slices)
    q8, k8, v8, descales = synth.make_qkv(w, "cpu", 0, n, transpose_v=False)
    return tuple(t.view(1, n, w.seqlen, w.head_dim) for t in (q8, k8, v8)) + (descales,)


def cpu_attention_tflops(w, budget_s: float, sample, label: str):
    """Times the CPU restatement of the reference's naive attention (test.py:25-33, fp32)
    on the slices of `sample` (cpu_sample), one after the other and round again until
    `budget_s` has passed; all host threads."""
    from oracle.attention_oracle import attention_fp32
    torch.set_num_threads(os.cpu_count() or 1)
    q8, k8, v8, (dq, dk, dv) = sample
    n = q8.shape[1]
    done, t0 = 0, time.perf_counter()
    while True:
        i = done % n
        attention_fp32(q8[:, i:i + 1], k8[:, i:i + 1], v8[:, i:i + 1], w.causal, w.softmax_scale, dq, dk, dv)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return {"value": w.flops(done) / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{done} slice passes over the first {n} of {w.n_slices} (batch,head) slices of {label}, {dt:.1f} s, "
                      "naive fp32 torch attention on dequantised inputs",
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


def config_of(w, slices_per_gpu: int, world: int, v_layout: str) -> dict:
    """The `config` object of the JSON line; both arms (this kernel and --impl reference) print
    the same keys for the same workload."""
    return {"workload": w.name, "batch": w.batch, "heads": w.heads, "seqlen": w.seqlen, "head_dim": w.head_dim,
            "causal": w.causal, "outliers": w.outliers, "slices_per_gpu": slices_per_gpu, "v_layout": v_layout,
            "out_dtype": "fp16", "parallelism": f"(batch x head) shards x{world}, no collective",
            "l2": f"inputs+output {w.hbm_bytes(slices_per_gpu) / 1e6:.0f} MB per step exceed the 126 MB L2"}


_REF_MODULE = []


def reference_module():
    """The reference's own extension built by oracle/build_ref.sh (unmodified sources, sm_89 PTX
    assembled for sm_100), or None.  Test infrastructure: only the legs that report the
    reference's kernel beside this one load it."""
    if not _REF_MODULE:
        import glob
        import importlib.util
        mod = None
        sos = glob.glob(os.path.join(ROOT, "oracle", "_ref", "attention_cutlass_fp8_ref*.so"))
        if sos:
            try:
                spec = importlib.util.spec_from_file_location("attention_cutlass_fp8_ref", sos[0])
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
            except Exception:  # noqa: BLE001
                mod = None
        _REF_MODULE.append(mod)
    return _REF_MODULE[0]


def compiled_binding():
    """The compiled torch module attention_cutlass_fp8 (csrc/torch_binding.cpp), or None."""
    import importlib.util
    from cutlass_flash_atten_fp8_b200.build import binding_is_stale, binding_path
    try:
        if binding_is_stale():
            return None
        spec = importlib.util.spec_from_file_location("attention_cutlass_fp8", binding_path())
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    except Exception:  # noqa: BLE001
        return None


# cutlass_fp8 column of the reference's published table (README.md:10, benchmark.png: an
# unspecified Ada GPU), milliseconds per call, keyed by (heads, seqlen, head_dim).
ADA_PUBLISHED_MS = {
    (16, 1024, 64): 0.03515, (16, 1024, 128): 0.05003, (16, 2048, 64): 0.08332, (16, 2048, 128): 0.11688,
    (16, 4096, 64): 0.19367, (16, 4096, 128): 0.30943, (32, 1024, 64): 0.04519, (32, 1024, 128): 0.06174,
    (32, 2048, 64): 0.10240, (32, 2048, 128): 0.16526, (32, 4096, 64): 0.30444, (32, 4096, 128): 0.53580,
    (64, 1024, 64): 0.06011, (64, 1024, 128): 0.09259, (64, 2048, 64): 0.16325, (64, 2048, 128): 0.27739,
    (64, 4096, 64): 0.53362, (64, 4096, 128): 0.97014,
}


def reference_protocol(device):
    """The reference's own benchmark (test.py:93-100): batch 1 x heads {16,32,64} x seqlen
    {1024,2048,4096} x head_dim {64,128}, causal, softmax_scale 1/sqrt(seqlen), inputs N(0, 0.5^2)
    clamped to +-0.1 and cast to e4m3 (test.py:12-23), V transposed (test.py:71).  Every shape
    is timed two ways: CUDA events around back-to-back calls, and the reference's method
    (test.py:36-46: host wall clock with a synchronise after every call, 5 warm-up + 20 timed
    calls) - for this kernel through the ctypes operator and through the compiled module, and
    for the reference's kernel where oracle/_ref is built."""
    from cutlass_flash_atten_fp8_b200 import flash_attention_v2_cutlass
    ref = reference_module()
    compiled = compiled_binding()
    rows = []
    g = torch.Generator(device=device)
    g.manual_seed(180)

    def events(fn, n=20):
        for _ in range(5):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def wall(fn, n=20):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / n

    for heads in (16, 32, 64):
        for seqlen in (1024, 2048, 4096):
            for head_dim in (64, 128):
                q, k, v = (torch.empty((1, heads, seqlen, head_dim), dtype=torch.float16, device=device)
                           .normal_(mean=0.0, std=0.5, generator=g).clamp(-0.1, 0.1).to(torch.float8_e4m3fn)
                           for _ in range(3))
                vt = v.transpose(2, 3).contiguous()
                sc = 1.0 / math.sqrt(seqlen)
                flops = 4.0 * heads * seqlen * seqlen * head_dim / 2
                out = torch.empty((1, heads, seqlen, head_dim), dtype=torch.float16, device=device)
                row = {"heads": heads, "seqlen": seqlen, "head_dim": head_dim,
                       "ada_published_ms": ADA_PUBLISHED_MS[(heads, seqlen, head_dim)]}
                ms = events(lambda: flash_attention_v2_cutlass(q, k, vt, True, sc, out=out))
                row["ours_ms_events"] = ms
                row["ours_tflops"] = flops / ms / 1e9
                row["ours_ms_wall_sync"] = wall(lambda: flash_attention_v2_cutlass(q, k, vt, True, sc))
                if compiled is not None:
                    row["ours_compiled_ms_wall_sync"] = wall(lambda: compiled.flash_attention_v2_cutlass(q, k, vt, True, sc))
                if ref is not None:
                    try:
                        rms = events(lambda: ref.flash_attention_v2_cutlass(q, k, vt, True, sc))
                        row["reference_kernel_ms_events"] = rms
                        row["reference_kernel_tflops"] = flops / rms / 1e9
                        row["reference_kernel_ms_wall_sync"] = wall(lambda: ref.flash_attention_v2_cutlass(q, k, vt, True, sc))
                    except Exception as e:  # noqa: BLE001
                        row["reference_kernel"] = f"unavailable: {type(e).__name__}: {str(e)[:80]}"
                rows.append(row)
    # Host cost of one call (no synchronise inside the loop) on the smallest shape, where the
    # 20-microsecond kernel makes the binding's own overhead visible.
    q, k, v = (torch.zeros((1, 16, 1024, 64), device=device).to(torch.float8_e4m3fn) for _ in range(3))
    vt = v.transpose(2, 3).contiguous()
    out = torch.empty((1, 16, 1024, 64), dtype=torch.float16, device=device)

    def per_call_us(fn, n=500):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        host = (time.perf_counter() - t0) * 1e6 / n
        torch.cuda.synchronize()
        return {"host_us_enqueue": host, "us_per_call_incl_drain": (time.perf_counter() - t0) * 1e6 / n}

    latency = {"shape": "H16 S1024 D64 causal",
               "ctypes_operator": per_call_us(lambda: flash_attention_v2_cutlass(q, k, vt, True, 1 / 32.0, out=out))}
    if compiled is not None:
        latency["compiled_module"] = per_call_us(lambda: compiled.flash_attention_v2_cutlass(q, k, vt, True, 1 / 32.0))
    return {"shapes": rows, "host_latency": latency,
            "reference_kernel": "oracle/_ref" if ref is not None else "unavailable: oracle/_ref not built",
            "note": "batch 1, causal, scale 1/sqrt(seqlen), clamp(+-0.1) e4m3 inputs; ada_published_ms is the "
                    "reference's README figure on an unspecified Ada GPU"}


def strong_and_gather(device, world: int, rank: int, steps: int = 5):
    """The box-scale causal workload (batch 64 x 32 heads x 8 192 x 128), its 2 048 (batch,
    head) slices partitioned over the ranks with no collective: device-timed, max over ranks.
    For N > 1 also the optional gather of its O on rank 0 over NCCL, timed apart."""
    import torch.distributed as dist
    from cutlass_flash_atten_fp8_b200 import check_status, flash_attention_v2_cutlass, synth
    from cutlass_flash_atten_fp8_b200.shard import gather_output, shard_range
    w = synth.WORKLOADS["box_s8192_d128_causal"]
    lo, hi = shard_range(w.n_slices, world, rank)
    n = hi - lo
    q8, k8, vt8, (dq, dk, dv) = synth.make_qkv(w, device, lo, hi)
    q4, k4, v4 = q8.view(1, n, w.seqlen, w.head_dim), k8.view(1, n, w.seqlen, w.head_dim), vt8.view(1, n, w.head_dim, w.seqlen)
    out = torch.empty((1, n, w.seqlen, w.head_dim), dtype=torch.float16, device=device)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(3):
        flash_attention_v2_cutlass(q4, k4, v4, True, w.softmax_scale * dq * dk, o_scale=dv, out=out)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        flash_attention_v2_cutlass(q4, k4, v4, True, w.softmax_scale * dq * dk, o_scale=dv, out=out)
    e1.record()
    sync_all()
    check_status(device)
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    rec = {"strong": {"workload": w.name, "slices_total": w.n_slices, "slices_per_gpu": n, "steps": steps,
                      "ms_per_step": ms, "value": w.flops() / ms / 1e9, "unit": "TFLOP/s", "scaling": "strong",
                      "pct_of_fp8_peak_nominal_per_gpu": 100.0 * w.flops() / ms / 1e9 / world / NOMINAL_FP8_TFLOPS}}
    if world > 1:
        gather_output(out[0], w.n_slices)          # warm-up: communicator set-up, receive buffer
        sync_all()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        full = gather_output(out[0], w.n_slices)
        g1.record()
        sync_all()
        gms = max_over_ranks(g0.elapsed_time(g1))
        inbound = 2.0 * (w.n_slices - n) * w.seqlen * w.head_dim if rank == 0 else 0.0
        t = torch.tensor([inbound], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rec["gather_o_ms"] = gms
        rec["gather_o"] = {"ms": gms, "bytes_into_rank0": float(t.item()), "gbs_into_rank0": float(t.item()) / gms / 1e6,
                           "workload": w.name, "note": "NCCL gather of fp16 O, outside `value`"}
        del full
    return rec


def reference_kernel_tflops(w, q8, k8, vt8, steps: int):
    """Optional: the reference's own Ada kernel (built by oracle/build_ref.sh into oracle/_ref,
    sm_89 PTX assembled for sm_100) timed on this GPU on the same inputs.  Reported beside the
    result; not part of `value`."""
    mod = reference_module()
    if mod is None:
        return {"unavailable": "oracle/_ref not built"}
    try:
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
    per_step_budget = max(0.25, min(5.0, 150.0 / max(1, args.warmup + args.steps)))
    sample = cpu_sample(w)
    vals = []
    for i in range(args.warmup + args.steps):
        r = cpu_attention_tflops(w, per_step_budget, sample, w.name)
        if i >= args.warmup:
            vals.append(r)
    v = sum(x["value"] for x in vals) / len(vals)
    ms = 1e3 * sum(x["seconds_per_slice"] for x in vals) / len(vals) * w.n_slices
    line = {
        "impl": "reference", "metric": "fp8_attn_fwd_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(w, w.n_slices, 1, "transposed"),
        "note": "ms_per_step extrapolated from the sampled slices to the whole workload",
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
    ap.add_argument("--e2e-groups", type=int, default=None, help="slice groups of the end-to-end pipeline (default: HostRunner's)")
    ap.add_argument("--e2e-taper", type=float, default=None, help="shrink factor of the tail groups (default: HostRunner's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", action="store_true",
                    help="kept for old command lines: the gather of O is always timed when N > 1 (gather_o_ms)")
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
    from cutlass_flash_atten_fp8_b200.shard import shard_range

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
    # Every step uploads the step's Q, K, V from pinned host memory and downloads O into a
    # pinned host tensor (the caller's `out=`, so that no allocation sits in the timed region).
    runner_kw = {k: v for k, v in (("chunks", args.e2e_groups), ("taper", args.e2e_taper)) if v is not None}
    runner = HostRunner(device, **runner_kw)
    hq, hk, hv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (q4, k4, v4))
    ho = torch.empty(out.shape, dtype=torch.float16, pin_memory=True)
    for _ in range(2):
        runner(hq, hk, hv, w.causal, scale, o_scale=dv, v_layout=args.v_layout, out=ho)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        runner(hq, hk, hv, w.causal, scale, o_scale=dv, v_layout=args.v_layout, out=ho)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    h2d, d2h = runner.bytes_per_call(hq, hv, hk)
    # The stages' busy times come from the same steps run again with an event around every copy
    # group and kernel (66 events per step, read back after each step: 0.4 ms per step, which is
    # why they are not in the timed steps above).
    runner.timing = True
    stage = {"h2d": 0.0, "kernel": 0.0, "d2h": 0.0}
    for _ in range(args.e2e_steps):
        runner(hq, hk, hv, w.causal, scale, o_scale=dv, v_layout=args.v_layout, out=ho)
        for key in stage:
            stage[key] += runner.last_timing[key]
    barrier()
    # busy time of each stage on this rank (summed over the slice groups, which overlap one
    # another across the three streams), and the slowest rank's figures
    mine = [e2e_ms / args.e2e_steps] + [stage[key] / args.e2e_steps for key in ("h2d", "kernel", "d2h")]
    if world > 1:
        t = torch.tensor(mine, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        mine = [float(x) for x in t.tolist()]
    e2e_ms, h2d_ms, kern_ms, d2h_ms = mine
    e2e = {"value": w.flops(total_slices) / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
           "per_rank": {"h2d_busy_ms": h2d_ms, "kernel_busy_ms": kern_ms, "d2h_busy_ms": d2h_ms,
                        "h2d_gbs": h2d / h2d_ms / 1e6, "d2h_gbs": d2h / d2h_ms / 1e6,
                        "kernel_share_of_step": kern_ms / e2e_ms,
                        "note": "slowest rank; stage times are busy times on that stage's stream, from the same "
                                "steps repeated with events around every copy group and kernel"},
           "host_link_gbs_all_ranks": (h2d + d2h) * world / e2e_ms / 1e6}
    del hq, hk, hv, ho, runner
    torch.cuda.empty_cache()

    extra = strong_and_gather(device, world, rank)

    if rank == 0:
        peaks = measured_peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        gemm = fp8_gemm_peak(device)
        line = {
            "metric": "fp8_attn_fwd_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": config_of(w, n_local, world, args.v_layout),
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
        line.update(extra)
        line["clocks"]["ms_x_median_sm_mhz"] = (ms_step * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None
        if sustained is not None:
            line["sustained"] = sustained
        if world == 1:
            line["reference_protocol"] = reference_protocol(device)
            line["quantize_prepass"] = quantize_rate(device, peaks)
            line["reference_kernel"] = (reference_kernel_tflops(w, q4, k4, v4, args.steps) if not natural
                                        else {"unavailable": "the reference kernel needs V transposed"})
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_attention_tflops(w, 12.0, cpu_sample(w), w.name)
                line["cpu_baseline"].pop("seconds_per_slice", None)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
