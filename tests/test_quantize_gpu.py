"""GPU tests of the fp16/bf16 -> e4m3 per-tensor quantisation pre-pass (through the C ABI) and of
the device-side descales of the attention operator."""
import math

import pytest
import torch

from cutlass_flash_atten_fp8_b200 import check_status, flash_attention_v2_cutlass, quantize_e4m3
from oracle.attention_oracle import attention_fp32, error_metrics

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


def _torch_quantize(x):
    amax = x.float().abs().max()
    scale = torch.tensor(448.0, device=x.device) / amax
    return (x.float() * scale).to(F8), amax / 448.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [8, 1000003, 16 * 32 * 1024 * 64 + 5])
def test_bit_exact_against_torch(dtype, n):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(n % 1000)
    x = (torch.randn(n, generator=g, device=dev) * 3.0).to(dtype)
    x[n // 2] = 37.5                                     # the maximum, exactly representable
    x8, descale = quantize_e4m3(x)
    want8, want_d = _torch_quantize(x)
    assert torch.equal(x8.view(torch.uint8), want8.view(torch.uint8))
    assert float(descale) == pytest.approx(float(want_d), rel=1e-6)
    assert float(x8.float().abs().max()) == 448.0


def test_all_zero_and_argument_errors():
    dev = torch.device("cuda", 0)
    x8, d = quantize_e4m3(torch.zeros(4096, dtype=torch.float16, device=dev))
    assert float(x8.float().abs().max()) == 0.0 and float(d) == 1.0
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        quantize_e4m3(torch.zeros(16, device=dev))
    with pytest.raises(RuntimeError, match="contiguous"):
        quantize_e4m3(torch.zeros(16, 16, dtype=torch.float16, device=dev).t())


@pytest.mark.parametrize("causal", [False, True])
def test_half_precision_to_attention_without_leaving_the_stream(causal):
    # fp16 Q/K/V -> e4m3 + device descales -> attention; nothing is read back in between
    dev = torch.device("cuda", 0)
    B, H, S, D = 2, 4, 1024, 128
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v = (torch.randn(B, H, S, D, generator=g, device=dev).half() * s for s in (1.0, 2.0, 0.5))
    (q8, dq), (k8, dk), (v8, dv) = quantize_e4m3(q), quantize_e4m3(k), quantize_e4m3(v)
    scale = 1 / math.sqrt(D)
    out, lse = flash_attention_v2_cutlass(q8, k8, v8, causal, scale, v_layout="natural", descale_q=dq,
                                          descale_k=dk, descale_v=dv, return_lse=True)
    check_status(dev)
    # same as folding the descales on the host
    host = flash_attention_v2_cutlass(q8, k8, v8, causal, scale * float(dq) * float(dk), v_layout="natural",
                                      o_scale=float(dv))[0]
    check_status(dev)
    assert float((out.float() - host.float()).abs().max()) <= 2e-3 * float(host.float().abs().max())
    ref = attention_fp32(q8.cpu(), k8.cpu(), v8.cpu(), causal, scale, float(dq), float(dk), float(dv))
    m = error_metrics(out, ref)
    assert m["rel_l2"] <= 3e-2 and m["max_abs"] <= 0.05 * m["max_ref"], m
    # and close to attention on the unquantised fp16 inputs (adds the e4m3 rounding of Q, K, V)
    full = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
    assert error_metrics(out, full)["rel_l2"] <= 8e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_per_head_quantisation_is_bit_exact_against_torch(dtype):
    dev = torch.device("cuda", 0)
    B, H, S, D = 3, 5, 200, 64
    g = torch.Generator(device=dev).manual_seed(11)
    gain = torch.rand(B, H, 1, 1, generator=g, device=dev) * 10 + 0.1      # heads of very different size
    x = (torch.randn(B, H, S, D, generator=g, device=dev) * gain).to(dtype)
    x8, descale = quantize_e4m3(x, per_head=True)
    assert tuple(descale.shape) == (B * H,)
    for b in range(B):
        for h in range(H):
            want8, want_d = _torch_quantize(x[b, h])
            assert torch.equal(x8[b, h].view(torch.uint8), want8.view(torch.uint8))
            assert float(descale[b * H + h]) == pytest.approx(float(want_d), rel=1e-6)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Hk", [6, 2])
def test_per_head_descales(causal, Hk):
    # heads whose magnitudes differ by orders: one scale per (batch, head), applied in the kernel
    dev = torch.device("cuda", 0)
    B, H, S, D = 2, 6, 512, 128
    g = torch.Generator(device=dev).manual_seed(17)
    gains = [torch.rand(B, n, 1, 1, generator=g, device=dev) * 20 + 0.05 for n in (H, Hk, Hk)]
    q, k, v = ((torch.randn(B, n, S, D, generator=g, device=dev) * gn).half() for n, gn in zip((H, Hk, Hk), gains))
    (q8, dq), (k8, dk), (v8, dv) = (quantize_e4m3(t, per_head=True) for t in (q, k, v))
    scale = 1 / math.sqrt(D)
    out, lse = flash_attention_v2_cutlass(q8, k8, v8, causal, scale, v_layout="natural", descale_q=dq,
                                          descale_k=dk, descale_v=dv, return_lse=True)
    check_status(dev)
    rep = H // Hk
    deq = lambda x8, d, n: x8.float() * d.view(B, n, 1, 1)
    qf, kf, vf = deq(q8, dq, H), deq(k8, dk, Hk).repeat_interleave(rep, 1), deq(v8, dv, Hk).repeat_interleave(rep, 1)
    s = torch.matmul(qf, kf.transpose(2, 3)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=dev).triu(1), float("-inf"))
    ref = torch.softmax(s, dim=-1) @ vf
    m = error_metrics(out.float().cpu(), ref.cpu())
    assert m["rel_l2"] <= 3e-2, m
    assert float((lse - torch.logsumexp(s, dim=-1)).abs().max()) <= 2e-3
    # per head, the same as the per-tensor path run on that head alone with its own scalars
    b, h = 1, 4
    hk = h // rep
    one = flash_attention_v2_cutlass(q8[b:b + 1, h:h + 1].contiguous(), k8[b:b + 1, hk:hk + 1].contiguous(),
                                     v8[b:b + 1, hk:hk + 1].contiguous(), causal, scale, v_layout="natural",
                                     descale_q=dq[b * H + h:b * H + h + 1].clone(),
                                     descale_k=dk[b * Hk + hk:b * Hk + hk + 1].clone(),
                                     descale_v=dv[b * Hk + hk:b * Hk + hk + 1].clone())[0]
    check_status(dev)
    assert torch.equal(one[0, 0], out[b, h])
    with pytest.raises(RuntimeError, match="one per"):
        flash_attention_v2_cutlass(q8, k8, v8, causal, scale, v_layout="natural", descale_q=dq, descale_k=dk[:1],
                                   descale_v=dv)
