"""Seeded synthetic workloads standing in for a dataset (the reference uses none:
its benchmark draws random tensors, test.py:12-23).

Each (batch, head) slice is drawn from its own generator seeded with
seed + slice index, so a slice has the same values whichever rank owns it and
however many ranks there are; the per-tensor quantisation scale 448/amax uses a
global amax (all-reduce MAX at set-up when sharded).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .shard import global_amax

E4M3_MAX = 448.0


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    heads: int
    seqlen: int
    head_dim: int
    causal: bool
    outliers: bool = False      # 0.1% of entries replaced by +-8 sigma before quantisation
    seed: int = 1000

    @property
    def n_slices(self) -> int:
        return self.batch * self.heads

    @property
    def softmax_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    def flops(self, n_slices: Optional[int] = None) -> float:
        n = self.n_slices if n_slices is None else n_slices
        f = 4.0 * n * self.seqlen * self.seqlen * self.head_dim
        return f / 2 if self.causal else f

    def hbm_bytes(self, n_slices: Optional[int] = None) -> float:
        """Algorithmic traffic: Q, K, V read once (1 byte each), fp16 O written once."""
        n = self.n_slices if n_slices is None else n_slices
        return 5.0 * n * self.seqlen * self.head_dim


WORKLOADS: Dict[str, Workload] = {
    "tiny": Workload("tiny", 1, 2, 128, 64, False, seed=1001),
    "prefill_s1024_d64": Workload("prefill_s1024_d64", 16, 32, 1024, 64, False, seed=1002),
    "mid_s4096_d128": Workload("mid_s4096_d128", 16, 32, 4096, 128, False, outliers=True, seed=1003),
    "mid_s4096_d128_causal": Workload("mid_s4096_d128_causal", 16, 32, 4096, 128, True, outliers=True, seed=1003),
    # batch-2 cuts of the mid-length shape: small enough for a multi-pass profiler capture, still larger than L2
    "mid_s4096_d128_b2": Workload("mid_s4096_d128_b2", 2, 32, 4096, 128, False, outliers=True, seed=1003),
    "mid_s4096_d128_b2_causal": Workload("mid_s4096_d128_b2_causal", 2, 32, 4096, 128, True, outliers=True, seed=1003),
    # head_dim 256 (one query tile per CTA), sized like the batch-2 cuts
    "mid_s4096_d256_b2": Workload("mid_s4096_d256_b2", 2, 16, 4096, 256, False, outliers=True, seed=1006),
    "long_s16384_d128_causal": Workload("long_s16384_d128_causal", 1, 32, 16384, 128, True, seed=1004),
    "box_s8192_d128_causal": Workload("box_s8192_d128_causal", 64, 32, 8192, 128, True, seed=1005),
}


def _draw_slice(w: Workload, slice_idx: int, device: torch.device) -> torch.Tensor:
    """fp32 [3, seqlen, head_dim] (q, k, v) of one (batch, head) slice."""
    g = torch.Generator(device=device)
    g.manual_seed(w.seed * 1000003 + slice_idx)
    x = torch.randn((3, w.seqlen, w.head_dim), generator=g, device=device, dtype=torch.float32)
    if w.outliers:
        u = torch.rand((3, w.seqlen, w.head_dim), generator=g, device=device)
        sign = torch.where(u < 0.0005, -1.0, 1.0)
        x = torch.where(u < 0.001, 8.0 * sign, x)
    return x


def make_qkv(w: Workload, device, lo: int = 0, hi: Optional[int] = None, group=None,
             transpose_v: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Tuple[float, float, float]]:
    """Quantised inputs of slices [lo, hi): (q8, k8, v8, (dq, dk, dv)).

    q8, k8 are float8_e4m3fn [hi-lo, seqlen, head_dim]; v8 is [hi-lo, head_dim, seqlen]
    when transpose_v (the reference's layout, test.py:71) else [hi-lo, seqlen, head_dim].
    x_true = d * x8.  Two passes over the slices: amax first, then quantisation."""
    device = torch.device(device)
    hi = w.n_slices if hi is None else hi
    n = hi - lo
    amax = torch.zeros(3, device=device)
    for s in range(lo, hi):
        amax = torch.maximum(amax, _draw_slice(w, s, device).abs().amax(dim=(1, 2)))
    amax = global_amax(amax, group)
    scale = E4M3_MAX / amax.clamp_min(1e-12)
    q8 = torch.empty((n, w.seqlen, w.head_dim), dtype=torch.float8_e4m3fn, device=device)
    k8 = torch.empty_like(q8)
    v_shape = (n, w.head_dim, w.seqlen) if transpose_v else (n, w.seqlen, w.head_dim)
    v8 = torch.empty(v_shape, dtype=torch.float8_e4m3fn, device=device)
    for s in range(lo, hi):
        x = _draw_slice(w, s, device) * scale.view(3, 1, 1)
        q8[s - lo] = x[0].to(torch.float8_e4m3fn)
        k8[s - lo] = x[1].to(torch.float8_e4m3fn)
        xv = x[2].to(torch.float8_e4m3fn)
        v8[s - lo] = xv.t() if transpose_v else xv
    d = (1.0 / scale).tolist()
    return q8, k8, v8, (d[0], d[1], d[2])
