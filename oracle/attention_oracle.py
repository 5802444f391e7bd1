"""CPU oracle for the FP8 attention-forward path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this module; the product package never does (it fails loudly when its
CUDA library is missing instead of falling back to anything here).

What is restated, and from where in the reference:

* ``attention_fp32``        - the naive attention of test.py:25-33
  (``p = q @ k^T * scale``; causal fill with -inf above the diagonal of a
  top-left aligned lower-triangular mask; ``softmax``; ``p @ v``), evaluated
  in fp32 on the dequantised e4m3 inputs.  This is the accuracy oracle and the
  timed CPU baseline.
* ``attention_reference_fp16`` - the same function with the reference's own
  precision choices (fp16 matmuls, fp32 softmax rounded to fp16), used to pin
  this module against fixtures produced by the reference's function itself.
* ``attention_quantised_p`` - a model of what an FP8 kernel computes: the
  online softmax of csrc/flash_attention.cu:233-273 walked in key blocks,
  unnormalised P = exp(scale*(S - m)) rounded to e4m3 round-to-nearest-even /
  saturating (csrc/flash_attention.cu:163-179, :524), the row sum taken from
  the fp32 P (:239-240, :264-271), fp32 accumulation of P.V, final division
  with the zero/NaN guard (:542-554).
* ``e4m3_decode`` / ``e4m3_encode`` - the e4m3 ("fn": no infinities, max 448)
  number format of cuda_fp8.h's __nv_fp8x2_e4m3 conversions used at
  csrc/flash_attention.cu:166-175.

Parity pin: the reference ships no golden vectors and no CPU implementation
(its only check is test.py:87 on a GPU).  The pin used here is
tests/golden/*.npz, produced by tests/golden/make_golden.py by calling the
reference's own ``self_attention`` (test.py:25-33) on CPU.
"""
from __future__ import annotations

import math

import numpy as np
import torch

E4M3_MAX = 448.0
LOG2E = 1.4426950408889634


def _build_decode_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if (b & 0x80) else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = (m / 8.0) * 2.0 ** (-6)
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = sign * v
    return t


_DECODE = _build_decode_table()


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn bit patterns -> float32."""
    return _DECODE[np.asarray(bits, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> uint8 e4m3fn bit patterns, round-to-nearest-even, saturating to
    +-448 (cvt.rn.satfinite semantics); NaN -> 0x7f."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, E4M3_MAX)
    # exponent of the binade, clamped to the subnormal binade
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)                 # spacing of representable values in the binade
    q = np.rint(a / step)                 # numpy rint = round half to even
    val = q * step                        # may round up into the next binade (still exact)
    val = np.minimum(val, E4M3_MAX)
    # re-derive fields from the rounded value
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0)))
    e2 = np.clip(e2, -6, 8)
    is_sub = val < 2.0 ** (-6)
    mant = np.where(is_sub, np.rint(val / 2.0 ** (-9)), np.rint((val / 2.0 ** e2 - 1.0) * 8.0))
    expf = np.where(is_sub, 0, e2 + 7)
    bits = (expf.astype(np.uint8) << 3) | mant.astype(np.uint8)
    bits = np.where(nan, np.uint8(0x7F), bits).astype(np.uint8)
    return (bits | sign).astype(np.uint8)


E5M2_MAX = 57344.0


def _e5m2_decode_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if (b & 0x80) else 1.0
        e = (b >> 2) & 0x1F
        m = b & 0x3
        if e == 0x1F:
            v = float("inf") if m == 0 else float("nan")
        elif e == 0:
            v = (m / 4.0) * 2.0 ** (-14)
        else:
            v = (1.0 + m / 4.0) * 2.0 ** (e - 15)
        t[b] = sign * v
    return t


_DECODE_E5M2 = _e5m2_decode_table()


def e5m2_decode(bits: np.ndarray) -> np.ndarray:
    """uint8 e5m2 bit patterns -> float32."""
    return _DECODE_E5M2[np.asarray(bits, dtype=np.uint8)]


def e5m2_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest e5m2 VALUE (as float32), round-to-nearest-even, saturating to +-57344
    (cvt.rn.satfinite.e5m2x2.f32 semantics); used for P of the e5m2 path."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), E5M2_MAX)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -14, 15)
    step = 2.0 ** (e - 2)
    val = np.minimum(np.rint(a / step) * step, E5M2_MAX)
    return (np.sign(x) * val).astype(np.float32)


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """fp32 tensor -> nearest e4m3 VALUE (fp32), round-to-nearest-even, saturating to +-448:
    what cvt.rn.satfinite.e4m3x2.f32 gives.  Uses torch's cast after the clamp (the cast alone
    turns values beyond the range into NaN); same result as e4m3_decode(e4m3_encode(x)), which
    tests/test_oracle_cpu.py checks, at a fraction of the time."""
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).to(torch.float32)


def _as_f32(x8) -> torch.Tensor:
    """Accepts uint8 bit patterns (numpy / torch) or a float8_e4m3fn tensor."""
    if isinstance(x8, np.ndarray):
        return torch.from_numpy(e4m3_decode(x8))
    if x8.dtype == torch.uint8:
        return torch.from_numpy(e4m3_decode(x8.cpu().numpy()))
    return x8.detach().cpu().to(torch.float32)


def causal_mask(seqlen: int) -> torch.Tensor:
    """True where a query row may see a key column: col <= row (test.py:27,30)."""
    return torch.ones(seqlen, seqlen, dtype=torch.bool).tril()


def attention_fp32(q8, k8, v8, causal: bool, softmax_scale: float,
                   dq: float = 1.0, dk: float = 1.0, dv: float = 1.0) -> torch.Tensor:
    """fp32 attention on dequantised e4m3 inputs; q8,k8,v8 are [B,H,S,D] (V NOT
    transposed).  d* are per-tensor descales (x_true = d * x8).  Restates
    test.py:25-33 in fp32.  Returns fp32 [B,H,S,D]."""
    q = _as_f32(q8) * dq
    k = _as_f32(k8) * dk
    v = _as_f32(v8) * dv
    B, H, S, D = q.shape
    out = torch.empty(B, H, S, D, dtype=torch.float32)
    mask = causal_mask(S) if causal else None
    for b in range(B):
        for h in range(H):
            p = (q[b, h] @ k[b, h].T) * softmax_scale
            if mask is not None:
                p = p.masked_fill(~mask, float("-inf"))
            p = torch.softmax(p, dim=-1)
            out[b, h] = p @ v[b, h]
    return out


def attention_reference_fp16(q8, k8, v8, causal: bool, softmax_scale: float) -> torch.Tensor:
    """test.py:25-33 with the reference's precisions: fp16 q@k^T, fp16 scale,
    fp32 softmax rounded to fp16, fp16 p@v.  Returns fp16 [B,H,S,D]."""
    q = _as_f32(q8).half()
    k = _as_f32(k8).half()
    v = _as_f32(v8).half()
    S = q.shape[-2]
    p = torch.matmul(q, k.transpose(2, 3)) * softmax_scale
    if causal:
        p[:, :, ~causal_mask(S)] = float("-inf")
    p = torch.softmax(p.float(), dim=-1).half()
    return torch.matmul(p, v)


# Polynomials for 2^f on [-1/2, 1/2] (minimax in relative error: 7.5e-5 and 1.7e-3), the ones
# the sm_100a kernel evaluates on the FMA pipe for part of the exponentials.
EXP2_POLY = {3: (0.99992806, 0.69326097, 0.24261114, 0.055171654),
             2: (1.0004431, 0.703448, 0.23842894)}
EXP2_POLY_LO, EXP2_POLY_HI = -126.0, 9.0


def exp2_poly(x: torch.Tensor, degree: int) -> torch.Tensor:
    """2^x the way the kernel's FMA-pipe path computes it: x clamped to [-126, 9], split into
    n = round-to-nearest(x) and f = x - n, polynomial in f, exponent added exactly."""
    x = x.double().clamp(EXP2_POLY_LO, EXP2_POLY_HI)
    n = torch.round(x)                       # ties to even, like the magic-number addition
    f = (x - n).float().double()
    c = EXP2_POLY[degree]
    r = torch.full_like(f, c[-1])
    for ck in reversed(c[:-1]):
        r = (r * f + ck).float().double()    # one rounding per fused multiply-add
    return (r * torch.exp2(n)).float()


def attention_quantised_p(q8, k8, v8, causal: bool, softmax_scale: float, block_n: int = 128,
                          o_scale: float = 1.0, lazy: bool = False, lazy_limit: float = 256.0,
                          lazy_rows: int = 32, p_format: str = "e4m3", poly_mask: int = 0,
                          poly_degree: int = 3) -> torch.Tensor:
    """Model of an FP8 kernel (see module docstring).  Raw fp8 values are used
    as they are (no descale), like the reference kernel; P is rounded to `p_format`
    ("e4m3", or "e5m2" when the inputs are e5m2, csrc/flash_attention.cu:163-179,631).
    Returns fp32 [B,H,S,D]
    *before* any rounding of O.

    lazy=False is the reference's rule: the running maximum m follows every block
    (csrc/flash_attention.cu:233-273), so P <= 1.  lazy=True models the sm_100a
    kernel: after the first block m is kept until, within a group of `lazy_rows`
    consecutive query rows, some row's block sum of P exceeds `lazy_limit`; only then
    m, l and the accumulator of the whole group are brought up to date.  Both give the
    same O/l up to the rounding of P.

    poly_mask: bit p set = the key columns 2p and 2p+1 of every block (block_n <= 64) take their
    exponential from exp2_poly(., poly_degree) instead of exp, as the kernel does on the FMA
    pipe; the row sum is taken from whatever P was computed, as in the kernel."""
    q = _as_f32(q8)
    k = _as_f32(k8)
    v = _as_f32(v8)
    B, H, S, D = q.shape
    out = torch.empty(B, H, S, D, dtype=torch.float32)
    rows = torch.arange(S).unsqueeze(1)
    for b in range(B):
        for h in range(H):
            m = torch.full((S,), float("-inf"))
            l = torch.zeros(S)
            acc = torch.zeros(S, D)
            for n0 in range(0, S, block_n):
                n1 = min(S, n0 + block_n)
                s = q[b, h] @ k[b, h, n0:n1].T                      # exact products, fp32 sums
                if causal:
                    cols = torch.arange(n0, n1).unsqueeze(0)
                    s = s.masked_fill(cols > rows, float("-inf"))
                m_new = torch.maximum(m, s.max(dim=1).values)
                if lazy and n0 > 0:
                    p_stale = torch.exp(s * softmax_scale - (m * softmax_scale).unsqueeze(1))
                    over = ~(p_stale.sum(dim=1) <= lazy_limit)
                    pad = (-S) % lazy_rows
                    grp = torch.cat([over, torch.zeros(pad, dtype=torch.bool)]).view(-1, lazy_rows).any(dim=1)
                    update = grp.repeat_interleave(lazy_rows)[:S]
                    m_new = torch.where(update, m_new, m)
                alpha = torch.where(torch.isinf(m) & (m < 0), torch.ones_like(m),
                                    torch.exp((m - m_new) * softmax_scale))
                m_eff = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                p = torch.exp(s * softmax_scale - (m_eff * softmax_scale).unsqueeze(1))
                if poly_mask:
                    c_log2 = softmax_scale * LOG2E
                    cols_in = torch.arange(n1 - n0)
                    sel = ((poly_mask >> (cols_in // 2)) & 1).bool()
                    x2 = (s[:, sel] * c_log2 - (m_eff * c_log2).unsqueeze(1))
                    p = p.clone()
                    p[:, sel] = exp2_poly(x2, poly_degree)
                l = l * alpha + p.sum(dim=1)
                p8 = torch.from_numpy(e5m2_round(p.numpy())) if p_format == "e5m2" else e4m3_round(p)
                acc = acc * alpha.unsqueeze(1) + p8 @ v[b, h, n0:n1]
                m = m_new
            inv = torch.where((l == 0) | torch.isnan(l), torch.ones_like(l), 1.0 / l)
            out[b, h] = acc * inv.unsqueeze(1) * o_scale
    return out


def attention_flops(B: int, H: int, S: int, D: int, causal: bool) -> float:
    """4*B*H*S^2*D, halved for causal."""
    f = 4.0 * B * H * S * S * D
    return f / 2 if causal else f


def error_metrics(out: torch.Tensor, ref: torch.Tensor) -> dict:
    out = out.detach().cpu().float()
    ref = ref.detach().cpu().float()
    diff = (out - ref)
    return {
        "max_abs": float(diff.abs().max()),
        "rel_l2": float(diff.norm() / max(ref.norm(), 1e-30)),
        "max_ref": float(ref.abs().max()),
    }


def attention_fp32_rows(q8, k8, v8, rows, causal: bool, softmax_scale: float) -> torch.Tensor:
    """attention_fp32 for ONE slice and a subset of its query rows: q8,k8,v8 are [S,D]
    (V not transposed), `rows` a 1-D index tensor.  Returns fp32 [len(rows), D].  Lets a
    test check a long sequence without the full S x S score matrix."""
    q = _as_f32(q8)[rows]
    k = _as_f32(k8)
    v = _as_f32(v8)
    p = (q @ k.T) * softmax_scale
    if causal:
        cols = torch.arange(k.shape[0]).unsqueeze(0)
        p = p.masked_fill(cols > rows.unsqueeze(1), float("-inf"))
    return torch.softmax(p, dim=-1) @ v
