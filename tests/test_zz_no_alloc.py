"""The quantiser entry point for callers that cannot allocate device memory,
fa8_quantize_e4m3_segments_noalloc, against the ordinary one.

Who needs it: code that runs where asking for device memory is forbidden or fails - a plug-in under
a framework that has frozen its memory plan, a serving callback whose allocator is off limits, a
stream that is being captured into a graph.  fa8_quantize_e4m3_segments makes such a caller bring a
buffer for the per-segment maxima; the variant keeps them in an array inside the library and
allocates nothing.  Everything here goes through the C ABI (ctypes); the only allocations are the
test's own tensors, made before the calls.

This file sorts after the other test files on purpose: a run that stops at the first failure has
then run every other test before it gets here.  It needs nothing from them and passes alone in a
fresh process as well.
"""
import ctypes

import pytest
import torch

from cutlass_flash_atten_fp8_b200 import _lib

pytestmark = pytest.mark.gpu


def _both(lib, x, n_seg, stream):
    """Quantises x ([n_seg, seg_len] fp16/bf16 on the GPU) through both entry points; returns
    (bytes, descales) of each."""
    dt = _lib.FA8_DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.FA8_DTYPE_FP16
    seg_len = x.numel() // n_seg
    ref8 = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    ref_amax = torch.empty(n_seg, dtype=torch.float32, device=x.device)
    ref_descale = torch.empty(n_seg, dtype=torch.float32, device=x.device)
    new8 = torch.full(x.shape, 0xAA, dtype=torch.uint8, device=x.device)
    new_descale = torch.full((n_seg,), -1.0, dtype=torch.float32, device=x.device)
    assert lib.fa8_quantize_e4m3_segments(x.data_ptr(), dt, ref8.data_ptr(), seg_len, n_seg, ref_amax.data_ptr(),
                                          ref_descale.data_ptr(), stream) == _lib.FA8_OK
    assert lib.fa8_quantize_e4m3_segments_noalloc(x.data_ptr(), dt, new8.data_ptr(), seg_len, n_seg,
                                                  new_descale.data_ptr(), stream) == _lib.FA8_OK
    torch.cuda.synchronize()
    return (ref8, ref_descale), (new8, new_descale)


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    g = torch.Generator(device=dev).manual_seed(41)
    # first call: 48 segments of large values.  Second call: fewer segments of values a thousand
    # times smaller - maxima left over from the first call would scale them all to zero, so this
    # also shows that the shared array is cleared where it has to start from zero.
    big = (torch.randn(48, 8 * 1024, generator=g, device=dev) * 300.0).half()
    small = (torch.randn(5, 64 * 1024, generator=g, device=dev) * 0.25).bfloat16()
    for x in (big, small):
        (ref8, ref_d), (new8, new_d) = _both(lib, x, x.shape[0], stream)
        # the quantiser tests of this library are bit-exact; so is this one
        assert torch.equal(new8, ref8)
        assert torch.equal(new_d, ref_d)
        assert bool((new_d > 0).all())
    # and the result is what the cast means: e4m3(x * 448 / amax) per segment
    amax = small.float().abs().amax(dim=1, keepdim=True)
    want = (small.float() * (448.0 / amax)).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(new8, want)
    assert torch.allclose(new_d, (amax / 448.0).flatten(), rtol=1e-6, atol=0)


def test_limits_and_argument_checks():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    x = torch.zeros(8 * 16, dtype=torch.float16, device=dev)
    out = torch.empty(8 * 16, dtype=torch.uint8, device=dev)
    d = torch.empty(_lib.FA8_NOALLOC_MAX_SEGMENTS + 1, dtype=torch.float32, device=dev)
    too_many = _lib.FA8_NOALLOC_MAX_SEGMENTS + 1
    rc = lib.fa8_quantize_e4m3_segments_noalloc(x.data_ptr(), _lib.FA8_DTYPE_FP16, out.data_ptr(), 8, too_many,
                                                d.data_ptr(), None)
    assert rc == _lib.FA8_ERR_UNSUPPORTED
    detail = lib.fa8_last_error_detail().decode()
    assert str(too_many) in detail and str(_lib.FA8_NOALLOC_MAX_SEGMENTS) in detail
    # the descales are the only way the scales come out: they are not optional here
    assert lib.fa8_quantize_e4m3_segments_noalloc(x.data_ptr(), _lib.FA8_DTYPE_FP16, out.data_ptr(), 8, 16, None,
                                                  None) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_quantize_e4m3_segments_noalloc(x.data_ptr(), _lib.FA8_DTYPE_FP16, out.data_ptr(), 12, 2,
                                                  d.data_ptr(), None) == _lib.FA8_ERR_BAD_ARG
    # the largest count the scratch holds works
    n = _lib.FA8_NOALLOC_MAX_SEGMENTS
    xs = torch.ones(n * 8, dtype=torch.float16, device=dev)
    outs = torch.empty(n * 8, dtype=torch.uint8, device=dev)
    assert lib.fa8_quantize_e4m3_segments_noalloc(xs.data_ptr(), _lib.FA8_DTYPE_FP16, outs.data_ptr(), 8, n,
                                                  d.data_ptr(), None) == _lib.FA8_OK
    torch.cuda.synchronize()
    assert bool((outs == 0x7E).all())          # 1.0 * 448 / 1.0 = 448 = 0x7e in e4m3
