"""GPU parity tests: the sm_100a kernel, called through the C ABI (ctypes), against the CPU
oracle on the same seeded inputs.

Stated tolerances (fp16 O, e4m3 P inside the kernel):
  * against the fp32 oracle:            rel-L2 <= 3e-2 and max-abs <= 0.05 * max|O_oracle|
  * against the quantised-P model:      rel-L2 <= 2e-3
  * against the reference's fixtures:   max-abs <= 1e-2  (the reference's own test.py:87)
"""
import glob
import math
import os

import numpy as np
import pytest
import torch

from cutlass_flash_atten_fp8_b200 import _lib, check_status, flash_attention_v2_cutlass, synth
from oracle.attention_oracle import (attention_fp32, attention_fp32_rows, attention_quantised_p,
                                     error_metrics)

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn
REL_L2_FP32, MAX_ABS_FRAC_FP32, REL_L2_MODEL = 3e-2, 0.05, 2e-3
# how the sm_100a kernel walks the keys: 64-key sub-blocks, row maximum raised lazily per 32-row warp
KERNEL_MODEL = dict(block_n=64, lazy=True, lazy_limit=448.0, lazy_rows=32)


def dev():
    return torch.device("cuda", 0)


def run_kernel(q8, k8, v8, causal, scale, **kw):
    """q8,k8,v8: float8 [B,H,S,D] on any device, V in natural layout."""
    d = dev()
    vt = v8.to(d).transpose(2, 3).contiguous()
    out = flash_attention_v2_cutlass(q8.to(d).contiguous(), k8.to(d).contiguous(), vt, causal, scale, **kw)[0]
    check_status(d)
    return out


def rand8(*shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(F8)


def assert_close_to_oracles(out, q8, k8, v8, causal, scale):
    o = out.float().cpu()
    assert not torch.isnan(o).any()
    ref = attention_fp32(q8.cpu(), k8.cpu(), v8.cpu(), causal, scale)
    m = error_metrics(o, ref)
    assert m["rel_l2"] <= REL_L2_FP32, m
    assert m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], m
    model = attention_quantised_p(q8.cpu(), k8.cpu(), v8.cpu(), causal, scale, **KERNEL_MODEL)
    mm = error_metrics(o, model)
    assert mm["rel_l2"] <= REL_L2_MODEL, mm


def test_reference_fixtures(golden_dir):
    files = sorted(glob.glob(os.path.join(golden_dir, "ref_self_attention_*.npz")))
    assert len(files) >= 4
    for f in files:
        g = np.load(f)
        q8, k8, v8 = (torch.from_numpy(g[n]).view(F8) for n in ("q", "k", "v"))
        out = run_kernel(q8, k8, v8, bool(g["causal"]), float(g["scale"]))
        diff = (out.float().cpu() - torch.from_numpy(g["out"].astype(np.float32))).abs().max()
        assert float(diff) <= 1e-2, (f, float(diff))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [64, 128, 192, 256, 320, 384, 640, 1024])
def test_random_inputs_against_oracles(D, causal, S):
    B, H = 2, 3
    q8, k8, v8 = (rand8(B, H, S, D, seed=100 * S + D + i) for i in range(3))
    out = run_kernel(q8, k8, v8, causal, 1 / math.sqrt(D))
    assert out.dtype == torch.float16 and tuple(out.shape) == (B, H, S, D)
    assert_close_to_oracles(out, q8, k8, v8, causal, 1 / math.sqrt(D))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [64, 192, 256, 1024, 1360])
def test_natural_v_layout(D, causal, S):
    """V passed as [B,H,S,D] (no transpose by the caller): bitwise the same O as with the
    reference's transposed V, and close to the oracles."""
    d = dev()
    q8, k8, v8 = (rand8(2, 3, S, D, seed=31 * S + D + i).to(d) for i in range(3))
    scale = 1 / math.sqrt(D)
    nat = flash_attention_v2_cutlass(q8, k8, v8.contiguous(), causal, scale, v_layout="natural")[0]
    check_status(d)
    tr = run_kernel(q8, k8, v8, causal, scale)
    assert torch.equal(nat, tr)
    assert_close_to_oracles(nat, q8, k8, v8, causal, scale)


@pytest.mark.parametrize("S", [16, 48, 144, 272])
def test_ragged_sequence_lengths(S):
    # not multiples of the 128-row tile (the reference needs multiples of 64, csrc/flash_attention.cu:594-597)
    for D, causal in ((64, True), (128, False), (128, True)):
        q8, k8, v8 = (rand8(1, 2, S, D, seed=7 * S + D + i) for i in range(3))
        out = run_kernel(q8, k8, v8, causal, 1 / math.sqrt(D))
        assert_close_to_oracles(out, q8, k8, v8, causal, 1 / math.sqrt(D))


@pytest.mark.parametrize("Sq,Sk", [(100, 100), (77, 333), (1, 64), (130, 17), (257, 1000)])
@pytest.mark.parametrize("causal", [False, True])
def test_any_sequence_length_with_natural_v(Sq, Sk, causal):
    """Only V^T has the sequence as its contiguous axis (rows of seqlen_k bytes, which the copy
    engine wants in multiples of 16): with V in its natural layout every length is accepted."""
    d = dev()
    for D in (64, 128):
        q8 = rand8(2, 2, Sq, D, seed=Sq + D)
        k8, v8 = rand8(2, 2, Sk, D, seed=Sk + D + 1), rand8(2, 2, Sk, D, seed=Sk + D + 2)
        scale = 1 / math.sqrt(D)
        guard = torch.full((2 * 2 * Sq * D + 64,), float("nan"), dtype=torch.float16, device=d)
        out = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v8.to(d), causal, scale, v_layout="natural",
                                         out=guard[:2 * 2 * Sq * D].view(2, 2, Sq, D))[0]
        check_status(d)
        assert bool(torch.isnan(guard[2 * 2 * Sq * D:]).all())
        s = torch.matmul(q8.float(), k8.float().transpose(2, 3)) * scale
        if causal:
            s = s.masked_fill(torch.arange(Sk).unsqueeze(0) > torch.arange(Sq).unsqueeze(1), float("-inf"))
        ref = torch.softmax(s, dim=-1) @ v8.float()
        m = error_metrics(out, ref)
        assert m["rel_l2"] <= REL_L2_FP32 and m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], (D, m)
    with pytest.raises(RuntimeError, match="unsupported"):     # transposed V still needs a multiple of 16
        x = torch.zeros(1, 1, 100, 64, device=d).to(F8)
        flash_attention_v2_cutlass(x, x, x.transpose(2, 3).contiguous(), False, 0.125)


def test_tiny_config_with_per_tensor_scales():
    # B1 H2 S128 D64 non-causal, N(0,1) amax-scaled to e4m3; descales folded by the caller
    w = synth.WORKLOADS["tiny"]
    q8, k8, v8, (dq, dk, dv) = synth.make_qkv(w, "cpu", transpose_v=False)
    q8, k8, v8 = (t.view(w.batch, w.heads, w.seqlen, w.head_dim) for t in (q8, k8, v8))
    out = run_kernel(q8, k8, v8, False, w.softmax_scale * dq * dk, o_scale=dv)
    ref = attention_fp32(q8, k8, v8, False, w.softmax_scale, dq, dk, dv)
    m = error_metrics(out, ref)
    assert m["rel_l2"] <= REL_L2_FP32 and m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], m


@pytest.mark.parametrize("causal", [False, True])
def test_log_sum_exp_output(causal):
    # lse_i = log(sum_j exp(scale * s_ij)); the scores are exact fp32 sums of e4m3 products
    d = dev()
    B, H, S, D = 2, 2, 704, 128
    q8, k8, v8 = (rand8(B, H, S, D, seed=900 + i) for i in range(3))
    scale = 1 / math.sqrt(D)
    out, lse = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v8.to(d), causal, scale, v_layout="natural",
                                          return_lse=True)
    check_status(d)
    s = torch.matmul(q8.float(), k8.float().transpose(2, 3)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    want = torch.logsumexp(s, dim=-1)
    assert tuple(lse.shape) == (B, H, S) and lse.dtype == torch.float32
    assert float((lse.cpu() - want).abs().max()) <= 2e-3
    assert torch.equal(out, run_kernel(q8, k8, v8, causal, scale))


@pytest.mark.parametrize("Hk", [1, 2])
@pytest.mark.parametrize("causal", [False, True])
def test_grouped_query_attention(Hk, causal):
    # 4 query heads share Hk key/value heads: same as expanding K and V
    d = dev()
    B, H, S, D = 2, 4, 640, 128
    q8 = rand8(B, H, S, D, seed=70)
    k8, v8 = rand8(B, Hk, S, D, seed=71), rand8(B, Hk, S, D, seed=72)
    scale = 1 / math.sqrt(D)
    got = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v8.to(d).transpose(2, 3).contiguous(), causal, scale)[0]
    check_status(d)
    rep = H // Hk
    want = run_kernel(q8, k8.repeat_interleave(rep, dim=1), v8.repeat_interleave(rep, dim=1), causal, scale)
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError, match="heads_kv"):
        flash_attention_v2_cutlass(q8.to(d), rand8(B, 3, S, D, seed=73).to(d), v8.to(d), causal, scale)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_e5m2_inputs(D, causal):
    """Q, K, V in e5m2 (the reference's other element type, csrc/flash_attention.cu:308,631); P is
    rounded to e5m2 too, which has one mantissa bit less: tolerance against fp32 is 6e-2."""
    E5 = torch.float8_e5m2
    B, H, S = 2, 2, 576
    g = torch.Generator().manual_seed(55 + D)
    q8, k8, v8 = (torch.randn(B, H, S, D, generator=g).to(E5) for _ in range(3))
    scale = 1 / math.sqrt(D)
    d = dev()
    out = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v8.to(d).transpose(2, 3).contiguous(), causal, scale)[0]
    check_status(d)
    ref = attention_fp32(q8, k8, v8, causal, scale)
    m = error_metrics(out, ref)
    assert m["rel_l2"] <= 6e-2 and m["max_abs"] <= 0.1 * m["max_ref"], m
    model = attention_quantised_p(q8, k8, v8, causal, scale, p_format="e5m2", **KERNEL_MODEL)
    assert error_metrics(out, model)["rel_l2"] <= REL_L2_MODEL
    with pytest.raises(RuntimeError, match="like q"):
        flash_attention_v2_cutlass(q8.to(d), k8.to(d).to(torch.float8_e4m3fn), v8.to(d), causal, scale)


@pytest.mark.parametrize("Sq,Sk", [(128, 1024), (1024, 320), (400, 640), (16, 2048)])
@pytest.mark.parametrize("causal", [False, True])
def test_different_query_and_key_lengths(Sq, Sk, causal):
    d = dev()
    B, H, D = 2, 2, 128
    q8 = rand8(B, H, Sq, D, seed=Sq)
    k8, v8 = rand8(B, H, Sk, D, seed=Sk + 1), rand8(B, H, Sk, D, seed=Sk + 2)
    scale = 1 / math.sqrt(D)
    out, lse = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v8.to(d), causal, scale, v_layout="natural",
                                          return_lse=True)
    check_status(d)
    s = torch.matmul(q8.float(), k8.float().transpose(2, 3)) * scale
    if causal:      # top-left aligned: key index <= query index
        s = s.masked_fill(torch.arange(Sk).unsqueeze(0) > torch.arange(Sq).unsqueeze(1), float("-inf"))
    ref = torch.softmax(s, dim=-1) @ v8.float()
    m = error_metrics(out, ref)
    assert tuple(out.shape) == (B, H, Sq, D)
    assert m["rel_l2"] <= REL_L2_FP32 and m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], m
    assert float((lse.cpu() - torch.logsumexp(s, dim=-1)).abs().max()) <= 2e-3


@pytest.mark.parametrize("D", [32, 96, 160, 192, 224, 256])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("layout", ["transposed", "natural"])
def test_other_head_dims_of_the_reference_switch(D, causal, layout):
    """The reference's head-dim buckets (csrc/static_switch.h:50-77) besides 64 and 128: 256 has
    a kernel of its own (one query tile per CTA), the rest run zero-padded on the next one up."""
    d = dev()
    B, H, S = 1, 3, 640
    q8, k8, v8 = rand8(B, H, S, D, seed=D), rand8(B, H, S, D, seed=D + 1), rand8(B, H, S, D, seed=D + 2)
    scale = 1 / math.sqrt(D)
    v_arg = v8.to(d) if layout == "natural" else v8.to(d).transpose(2, 3).contiguous()
    guard = torch.full((B * H * S * D + 64,), float("nan"), dtype=torch.float16, device=d)
    out_buf = guard[:B * H * S * D].view(B, H, S, D)
    out = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v_arg, causal, scale, v_layout=layout, out=out_buf)[0]
    check_status(d)
    assert tuple(out.shape) == (B, H, S, D)
    assert bool(torch.isnan(guard[B * H * S * D:]).all())        # nothing written past the last row
    assert_close_to_oracles(out, q8, k8, v8, causal, scale)


def test_known_answers():
    S, D = 512, 128
    q8, k8 = rand8(1, 2, S, D, seed=1), rand8(1, 2, S, D, seed=2)
    # uniform V rows: every output row equals that row, whatever P is
    row = rand8(1, 2, 1, D, seed=3).float()
    v8 = row.expand(1, 2, S, D).contiguous().to(F8)
    out = run_kernel(q8, k8, v8, True, 0.1).float().cpu()
    assert torch.allclose(out, row.expand_as(out), rtol=0, atol=0.04 * float(row.abs().max()))
    # causal: row 0 sees key 0 only -> exactly V[0]
    v8 = rand8(1, 2, S, D, seed=4)
    out = run_kernel(q8, k8, v8, True, 0.1).float().cpu()
    assert torch.equal(out[:, :, 0], v8[:, :, 0].float())
    # Q = 0: uniform probabilities -> column means of V (P = 1.0 is exact in e4m3)
    out = run_kernel(torch.zeros(1, 2, S, D).to(F8), k8, v8, False, 0.1).float().cpu()
    assert torch.allclose(out, v8.float().mean(dim=2, keepdim=True).expand_as(out), rtol=0, atol=2e-3)


def test_large_scores_and_saturated_inputs():
    # +-448 everywhere in Q and K: scores of +-448^2*D, exp underflows for all but the maxima
    S, D = 256, 64
    g = torch.Generator().manual_seed(5)
    sign = lambda: torch.where(torch.rand(1, 1, S, D, generator=g) < 0.5, -448.0, 448.0).to(F8)
    q8, k8, v8 = sign(), sign(), rand8(1, 1, S, D, seed=6)
    out = run_kernel(q8, k8, v8, False, 1e-4)
    assert_close_to_oracles(out, q8, k8, v8, False, 1e-4)


def test_bitwise_deterministic_and_reuses_out():
    q8, k8, v8 = (rand8(2, 4, 1024, 128, seed=20 + i) for i in range(3))
    a = run_kernel(q8, k8, v8, True, 0.09)
    buf = torch.full_like(a, float("nan"))
    b = run_kernel(q8, k8, v8, True, 0.09, out=buf)
    assert b.data_ptr() == buf.data_ptr()
    assert torch.equal(a, b)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [192, 640, 1024, 1360])
def test_work_plans_agree_bitwise(D, causal, S):
    """A launch of a few slices is cut into finer work items than a launch that fills the GPU
    (fa8_work_plan).  The same slices computed either way are bitwise identical, log-sum-exp
    included, and the GPU-filling launch (the plan the full-size configurations run with) is
    checked against the oracles on ragged and whole tile counts alike."""
    sms = torch.cuda.get_device_properties(dev()).multi_processor_count
    H, few = 80, 2
    big_plan = _lib.work_plan(H, S, D, causal, sms)
    small_plan = _lib.work_plan(few, S, D, causal, sms)
    assert big_plan["rows_per_item"] == (128 if D > 128 else 256) and big_plan["paired"] == causal
    if S > 128 and (D <= 128 or causal):      # one query tile per CTA above 128: only unpairing is finer
        assert (small_plan["rows_per_item"], small_plan["paired"]) != (big_plan["rows_per_item"], big_plan["paired"])
    q8, k8, v8 = (rand8(1, H, S, D, seed=300 + i) for i in range(3))
    scale = 1.0 / math.sqrt(D)
    d = dev()
    qd, kd, vtd = q8.to(d), k8.to(d), v8.to(d).transpose(2, 3).contiguous()
    o_big, lse_big = flash_attention_v2_cutlass(qd, kd, vtd, causal, scale, return_lse=True)
    o_few, lse_few = flash_attention_v2_cutlass(qd[:, :few].contiguous(), kd[:, :few].contiguous(),
                                                vtd[:, :few].contiguous(), causal, scale, return_lse=True)
    check_status(d)
    assert torch.equal(o_big[:, :few], o_few)
    assert torch.equal(lse_big[:, :few], lse_few)
    sel = [0, H - 1]
    assert_close_to_oracles(o_big[:, sel], q8[:, sel], k8[:, sel], v8[:, sel], causal, scale)


def test_same_addresses_with_other_shapes_and_other_addresses_with_the_same_shape():
    """The library keeps the tensor maps of a thread's previous call and reuses them when
    addresses, extents and layout all match: calls that differ in any one of them must not
    see the earlier maps."""
    d = dev()
    q8, k8, v8 = (rand8(1, 4, 512, 64, seed=400 + i).to(d) for i in range(3))
    scale = 0.125

    def both(q, k, v, causal):
        vt = v.transpose(2, 3).contiguous()
        a = flash_attention_v2_cutlass(q, k, vt, causal, scale)[0]
        b = flash_attention_v2_cutlass(q, k, vt, causal, scale)[0]      # same addresses except O
        buf = torch.empty_like(a)
        c = flash_attention_v2_cutlass(q, k, vt, causal, scale, out=buf)[0]
        e = flash_attention_v2_cutlass(q, k, vt, causal, scale, out=buf)[0]   # every address the same
        check_status(d)
        assert torch.equal(a, b) and torch.equal(a, c) and torch.equal(a, e)
        assert_close_to_oracles(a, q, k, v, causal, scale)

    both(q8, k8, v8, False)
    both(q8, k8, v8, True)
    # the same storage read as eight slices of 256 rows: same addresses, other extents
    both(q8.view(1, 8, 256, 64), k8.view(1, 8, 256, 64), v8.view(1, 8, 256, 64), False)
    # same shape as the first call, other addresses
    q2, k2, v2 = (rand8(1, 4, 512, 64, seed=410 + i).to(d) for i in range(3))
    both(q2, k2, v2, False)
    both(q8, k8, v8, False)


def test_operator_argument_errors_on_gpu():
    d = dev()
    q = torch.zeros(1, 1, 128, 64, device=d).to(F8)
    vt = torch.zeros(1, 1, 64, 128, device=d).to(F8)
    with pytest.raises(RuntimeError, match="must be contiguous"):       # include/attention_api.cuh:14-15
        flash_attention_v2_cutlass(q.transpose(2, 3), q, vt, False, 0.125)
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        flash_attention_v2_cutlass(q.float(), q, vt, False, 0.125)
    with pytest.raises(RuntimeError, match="v must be"):
        flash_attention_v2_cutlass(q, q, q, False, 0.125)               # V not transposed
    for bad_d in (48, 288):
        qb = torch.zeros(1, 1, 128, bad_d, device=d).to(F8)
        with pytest.raises(RuntimeError, match="unsupported"):
            flash_attention_v2_cutlass(qb, qb, qb.transpose(2, 3).contiguous(), False, 0.125)
    with pytest.raises(RuntimeError, match="bad argument"):
        flash_attention_v2_cutlass(q, q, vt, False, 0.0)
    out = flash_attention_v2_cutlass(q, q, vt)                            # defaults: non-causal, scale 1
    assert isinstance(out, list) and len(out) == 1
    check_status(d)


def _sampled_rows_check(q8, k8, vt8, out, slices, causal, scale, dv=1.0, n_rows=256):
    """q8,k8 [N,S,D], vt8 [N,D,S] on the GPU; compares sampled query rows of some slices."""
    S = q8.shape[1]
    g = torch.Generator().manual_seed(0)
    for s in slices:
        rows = torch.sort(torch.randperm(S, generator=g)[:n_rows]).values
        rows[0], rows[-1] = 0, S - 1
        ref = attention_fp32_rows(q8[s].cpu(), k8[s].cpu(), vt8[s].t().contiguous().cpu(), rows, causal, scale) * dv
        m = error_metrics(out[s].float().cpu()[rows], ref)
        assert m["rel_l2"] <= REL_L2_FP32, (s, m)
        assert m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], (s, m)


def _whole_slice_check(q8, k8, vt8, out, s, causal, scale, dv):
    """Every row of slice `s` against the fp32 oracle and against the kernel model (the tight
    one: it is what would catch a wrong rescale when the lazily raised maximum fires)."""
    S, D = q8.shape[1], q8.shape[2]
    q, k = q8[s].cpu().view(1, 1, S, D), k8[s].cpu().view(1, 1, S, D)
    v = vt8[s].t().contiguous().cpu().view(1, 1, S, D)
    o = out[s].float().cpu().view(1, 1, S, D)
    m = error_metrics(o, attention_fp32(q, k, v, causal, scale) * dv)
    assert m["rel_l2"] <= REL_L2_FP32 and m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], (s, m)
    model = attention_quantised_p(q, k, v, causal, scale, o_scale=dv, **KERNEL_MODEL)
    mm = error_metrics(o, model)
    assert mm["rel_l2"] <= REL_L2_MODEL, (s, mm)


@pytest.mark.parametrize("name", ["prefill_s1024_d64", "mid_s4096_d128", "mid_s4096_d128_causal",
                                  "long_s16384_d128_causal"])
def test_full_size_configs(name):
    """Full-size BASELINE configs on their own synthetic data (per-tensor scales, the +-8 sigma
    outliers of the mid-length config included): one whole slice, all rows, against the fp32
    oracle and the kernel model; sampled rows of three more slices against the fp32 oracle;
    shard invariance (a sub-range of slices computed alone is bitwise the same)."""
    w = synth.WORKLOADS[name]
    d = dev()
    q8, k8, vt8, (dq, dk, dv) = synth.make_qkv(w, d)
    n = w.n_slices
    scale = w.softmax_scale * dq * dk
    as4 = lambda t: t.view(1, *t.shape)
    out = flash_attention_v2_cutlass(as4(q8), as4(k8), as4(vt8), w.causal, scale, o_scale=dv)[0][0]
    check_status(d)
    assert not torch.isnan(out).any()
    _whole_slice_check(q8, k8, vt8, out, n // 3, w.causal, scale, dv)
    _sampled_rows_check(q8, k8, vt8, out, [0, n // 2, n - 1], w.causal, scale, dv)
    lo, hi = n // 4, n // 4 + max(1, n // 8)
    part = flash_attention_v2_cutlass(as4(q8[lo:hi]), as4(k8[lo:hi]), as4(vt8[lo:hi]), w.causal, scale, o_scale=dv)[0][0]
    check_status(d)
    assert torch.equal(part, out[lo:hi])


def test_box_scale_config_shape():
    """B64 H32 S8192 D128 causal (2048 slices, the largest grid and tensors beyond 2^31 bytes) on
    the workload's own data - iid N(0,1), per-tensor amax scaling, descales folded the way the
    benchmark folds them: one whole slice against both oracles, sampled rows of the first, a
    middle and the last slice, and a shard of 256 slices (one rank of eight) bitwise equal."""
    w = synth.WORKLOADS["box_s8192_d128_causal"]
    d = dev()
    n, S, D = w.n_slices, w.seqlen, w.head_dim
    q8, k8, vt8, (dq, dk, dv) = synth.make_qkv(w, d)
    scale = w.softmax_scale * dq * dk
    out = flash_attention_v2_cutlass(q8.view(1, n, S, D), k8.view(1, n, S, D), vt8.view(1, n, D, S), True, scale,
                                     o_scale=dv)[0][0]
    check_status(d)
    _whole_slice_check(q8, k8, vt8, out, 777, True, scale, dv)
    _sampled_rows_check(q8, k8, vt8, out, [0, 1023, n - 1], True, scale, dv, n_rows=128)
    lo, hi = 3 * 256, 4 * 256
    part = flash_attention_v2_cutlass(q8[lo:hi].view(1, 256, S, D), k8[lo:hi].view(1, 256, S, D),
                                      vt8[lo:hi].view(1, 256, D, S), True, scale, o_scale=dv)[0][0]
    check_status(d)
    assert torch.equal(part, out[lo:hi])


@pytest.mark.parametrize("Hk,layout,lse", [(6, "transposed", False), (6, "natural", True), (2, "natural", False)])
def test_host_runner_pipelines_groups_of_slices(Hk, layout, lse):
    """Host tensors in, host tensor out: upload, kernel and download of slice groups overlap on three
    streams; the result is bitwise the one the operator gives on device tensors."""
    from cutlass_flash_atten_fp8_b200 import HostRunner
    d = dev()
    B, H, S, D = 3, 6, 384, 64
    q8, k8, v8 = rand8(B, H, S, D, seed=1), rand8(B, Hk, S, D, seed=2), rand8(B, Hk, S, D, seed=3)
    v_host = (v8 if layout == "natural" else v8.transpose(2, 3).contiguous())
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
    runner = HostRunner(d, chunks=4)
    got = runner(pin(q8), pin(k8), pin(v_host), True, 0.125, v_layout=layout, return_lse=lse)
    want = flash_attention_v2_cutlass(q8.to(d), k8.to(d), v_host.to(d), True, 0.125, v_layout=layout, return_lse=lse)
    check_status(d)
    assert got[0].device.type == "cpu" and torch.equal(got[0], want[0].cpu())
    if lse:
        assert torch.equal(got[1], want[1].cpu())
    again = runner(pin(q8), pin(k8), pin(v_host), True, 0.125, v_layout=layout)[0]     # buffers reused
    assert torch.equal(again, want[0].cpu())


@pytest.mark.parametrize("causal", [False, True])
def test_very_long_sequence(causal):
    """One head of 65 536 positions (256 tile pairs, 1 024 sub-blocks per work item): sampled rows."""
    d = dev()
    S, D = 65536, 128
    g = torch.Generator(device=d).manual_seed(9)
    q8, k8 = (torch.randn(2, S, D, generator=g, device=d).to(F8) for _ in range(2))
    vt8 = torch.randn(2, D, S, generator=g, device=d).to(F8)
    scale = 1 / math.sqrt(D)
    out = flash_attention_v2_cutlass(q8.view(1, 2, S, D), k8.view(1, 2, S, D), vt8.view(1, 2, D, S), causal, scale)[0][0]
    check_status(d)
    assert not torch.isnan(out).any()
    _sampled_rows_check(q8, k8, vt8, out, [1], causal, scale, n_rows=96)


def test_many_short_slices():
    """8 192 (batch, head) slices of one tile each: the unit index runs far past the grid size."""
    d = dev()
    n, S, D = 8192, 128, 64
    g = torch.Generator(device=d).manual_seed(10)
    q8, k8, v8 = (torch.randn(n, S, D, generator=g, device=d).to(F8) for _ in range(3))
    out = flash_attention_v2_cutlass(q8.view(64, 128, S, D), k8.view(64, 128, S, D), v8.view(64, 128, S, D), True, 0.125,
                                     v_layout="natural")[0].view(n, S, D)
    check_status(d)
    for s in (0, 4097, n - 1):
        ref = attention_fp32(q8[s].cpu().view(1, 1, S, D), k8[s].cpu().view(1, 1, S, D), v8[s].cpu().view(1, 1, S, D), True, 0.125)[0, 0]
        m = error_metrics(out[s], ref)
        assert m["rel_l2"] <= REL_L2_FP32 and m["max_abs"] <= MAX_ABS_FRAC_FP32 * m["max_ref"], (s, m)
