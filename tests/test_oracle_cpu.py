"""CPU tests of the oracle itself: pinned against fixtures produced by the reference's
own self_attention (test.py:25-33), plus known-answer cases."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle.attention_oracle import (attention_fp32, attention_quantised_p, attention_reference_fp16,
                                     e4m3_decode, e4m3_encode, error_metrics)

F8 = torch.float8_e4m3fn


def _golden(golden_dir):
    files = sorted(glob.glob(os.path.join(golden_dir, "ref_self_attention_*.npz")))
    assert len(files) >= 4
    return files


def test_e4m3_codec_matches_torch():
    bits = np.arange(256, dtype=np.uint8)
    t = torch.from_numpy(bits).view(F8).float().numpy()
    d = e4m3_decode(bits)
    assert np.array_equal(np.isnan(t), np.isnan(d))
    assert np.array_equal(t[~np.isnan(t)], d[~np.isnan(d)])
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 1e-2, 0.1, 1, 10, 100)])
    fin = d[~np.isnan(d)]
    x = np.concatenate([x, fin, ((np.sort(fin)[:-1] + np.sort(fin)[1:]) / 2).astype(np.float32)])
    x = x[np.abs(x) <= 448]
    ours = e4m3_encode(x)
    theirs = torch.from_numpy(x).to(F8).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)
    # saturation and NaN, the cvt.rn.satfinite semantics of csrc/flash_attention.cu:163-179
    assert list(e4m3_encode(np.array([1e9, -1e9, 449, 464, np.nan], dtype=np.float32))) == [126, 254, 126, 126, 127]


def test_e5m2_codec_matches_torch():
    from oracle.attention_oracle import e5m2_decode, e5m2_round
    bits = np.arange(256, dtype=np.uint8)
    t = torch.from_numpy(bits).view(torch.float8_e5m2).float().numpy()
    d = e5m2_decode(bits)
    assert np.array_equal(np.isnan(t), np.isnan(d))
    assert np.array_equal(t[~np.isnan(t)], d[~np.isnan(d)])
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-5, 1e-3, 0.1, 1, 100, 3e4)])
    x = x[np.abs(x) <= 57344]
    theirs = torch.from_numpy(x).to(torch.float8_e5m2).float().numpy()
    assert np.array_equal(e5m2_round(x), theirs)
    assert list(e5m2_round(np.array([1e9, -1e9, 60000.0], dtype=np.float32))) == [57344.0, -57344.0, 57344.0]


def test_restatement_is_bit_exact_on_reference_fixtures(golden_dir):
    for f in _golden(golden_dir):
        g = np.load(f)
        out = attention_reference_fp16(g["q"], g["k"], g["v"], bool(g["causal"]), float(g["scale"]))
        assert np.array_equal(out.numpy(), g["out"]), f


def test_fp32_oracle_agrees_with_reference_fixtures(golden_dir):
    for f in _golden(golden_dir):
        g = np.load(f)
        out = attention_fp32(g["q"], g["k"], g["v"], bool(g["causal"]), float(g["scale"]))
        # fp16 rounding of p and of the output in the reference's function
        assert np.abs(out.numpy() - g["out"].astype(np.float32)).max() < 2e-3, f


def test_quantised_p_model_within_reference_tolerance(golden_dir):
    # the reference's own acceptance test is atol=1e-2 (test.py:87)
    for f in _golden(golden_dir):
        g = np.load(f)
        out = attention_quantised_p(g["q"], g["k"], g["v"], bool(g["causal"]), float(g["scale"]))
        assert np.abs(out.numpy() - g["out"].astype(np.float32)).max() < 1e-2, f


def _rand8(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(F8)


@pytest.mark.parametrize("fn", [attention_fp32, attention_quantised_p])
def test_uniform_v_rows_give_that_row(fn):
    q, k = _rand8(1, 2, 256, 64, seed=1), _rand8(1, 2, 256, 64, seed=2)
    row = _rand8(1, 2, 1, 64, seed=3).float()
    v = row.expand(1, 2, 256, 64).contiguous().to(F8)
    out = fn(q, k, v, True, 0.125)
    assert torch.allclose(out, row.expand_as(out), rtol=0, atol=0.04 * float(row.abs().max()))


@pytest.mark.parametrize("fn", [attention_fp32, attention_quantised_p])
def test_causal_first_row_is_v0(fn):
    q, k, v = _rand8(1, 1, 128, 64, seed=4), _rand8(1, 1, 128, 64, seed=5), _rand8(1, 1, 128, 64, seed=6)
    out = fn(q, k, v, True, 0.125)
    assert torch.equal(out[0, 0, 0], v[0, 0, 0].float())


def test_one_hot_scores_select_rows():
    S, D = 128, 64
    q = torch.zeros(1, 1, S, D)
    k = torch.zeros(1, 1, S, D)
    perm = torch.randperm(D, generator=torch.Generator().manual_seed(7))
    for r in range(S):
        q[0, 0, r, perm[r % D]] = 16.0
    for c in range(D):
        k[0, 0, c, c] = 16.0          # keys D..S-1 are zero rows
    v = _rand8(1, 1, S, D, seed=8)
    out = attention_quantised_p(q.to(F8), k.to(F8), v, False, 1.0)   # score 256 vs 0 -> one-hot
    for r in range(S):
        assert torch.equal(out[0, 0, r], v[0, 0, perm[r % D]].float())


def test_block_size_does_not_change_the_model_much():
    q, k, v = _rand8(1, 1, 512, 128, seed=9), _rand8(1, 1, 512, 128, seed=10), _rand8(1, 1, 512, 128, seed=11)
    a = attention_quantised_p(q, k, v, True, 1 / math.sqrt(128), block_n=128)
    b = attention_quantised_p(q, k, v, True, 1 / math.sqrt(128), block_n=64)   # the reference's tile
    ref = attention_fp32(q, k, v, True, 1 / math.sqrt(128))
    assert error_metrics(a, ref)["rel_l2"] < 3e-2
    assert error_metrics(b, ref)["rel_l2"] < 3e-2
    assert error_metrics(a, b)["rel_l2"] < 3e-2


def test_descales_fold_into_scale_and_output():
    q, k, v = _rand8(1, 1, 128, 64, seed=12), _rand8(1, 1, 128, 64, seed=13), _rand8(1, 1, 128, 64, seed=14)
    dq, dk, dv = 0.01, 0.02, 0.03
    a = attention_fp32(q, k, v, False, 0.125, dq, dk, dv)
    b = attention_fp32(q, k, v, False, 0.125 * dq * dk) * dv
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-6)


def test_fast_e4m3_rounding_equals_the_bit_level_one():
    from oracle.attention_oracle import e4m3_decode, e4m3_encode, e4m3_round
    g = torch.Generator().manual_seed(21)
    x = torch.cat([torch.randn(200000, generator=g) * s for s in (1e-3, 0.05, 1.0, 30.0, 400.0)])
    x = torch.cat([x, torch.tensor([0.0, 448.0, 449.0, 464.0, 480.0, 1e6, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10,
                                    2.0 ** -10 * 0.999, 0.0078125 + 0.0009765625])])
    want = torch.from_numpy(e4m3_decode(e4m3_encode(x.numpy())))
    assert torch.equal(e4m3_round(x), want)


def test_polynomial_exponential_model():
    from oracle.attention_oracle import exp2_poly
    x = torch.linspace(-140.0, 12.0, 50001)
    t = torch.exp2(x.double().clamp(-126.0, 9.0))
    for deg, tol in ((3, 8e-5), (2, 1.8e-3)):
        r = exp2_poly(x, deg).double()
        assert float(((r - t) / t).abs().max()) <= tol
    # on part of the columns it moves the model by far less than its distance to the fp32 oracle
    q, k, v = _rand8(1, 1, 512, 128, seed=30), _rand8(1, 1, 512, 128, seed=31), _rand8(1, 1, 512, 128, seed=32)
    sc = 1 / math.sqrt(128)
    a = attention_quantised_p(q, k, v, True, sc, block_n=64, lazy=True, lazy_limit=448.0)
    b = attention_quantised_p(q, k, v, True, sc, block_n=64, lazy=True, lazy_limit=448.0, poly_mask=0x11111111,
                              poly_degree=2)
    ref = attention_fp32(q, k, v, True, sc)
    assert error_metrics(a, b)["rel_l2"] < 1e-2
    assert abs(error_metrics(a, ref)["rel_l2"] - error_metrics(b, ref)["rel_l2"]) < 2e-3
