"""Failure detection without faulting the GPU: a wait that runs out inside a kernel becomes a
status code the host reads, and the context stays usable."""
import ctypes
import math

import pytest
import torch

from cutlass_flash_atten_fp8_b200 import _lib, check_status, flash_attention_v2_cutlass
from cutlass_flash_atten_fp8_b200.api import status_word

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


def test_expired_wait_is_reported_and_context_survives():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    word = status_word(dev)
    word.zero_()
    stream = torch.cuda.current_stream(dev).cuda_stream
    # a barrier nobody completes; the wait gives up after 2 ms
    assert lib.fa8_selftest_expired_wait(word.data_ptr(), 2000, stream) == _lib.FA8_OK
    code = ctypes.c_int32(0)
    rc = lib.fa8_check_status(word.data_ptr(), stream, ctypes.byref(code))
    assert rc == _lib.FA8_ERR_DEVICE_TIMEOUT and code.value == 0x7E57

    # fa8_check_status has reported it, so the library's host-side flag is clear again; the
    # caller's word is the caller's to clear.  While it stays non-zero every attention CTA
    # returns at once, output untouched - and that launch is reported too.
    q = torch.randn(1, 2, 256, 64, device=dev).to(F8)
    vt = torch.randn(1, 2, 64, 256, device=dev).to(F8)
    out = torch.full((1, 2, 256, 64), 7.0, dtype=torch.float16, device=dev)
    flash_attention_v2_cutlass(q, q, vt, False, 0.125, out=out)
    with pytest.raises(RuntimeError, match="bounded wait"):
        check_status(dev)                      # raises and clears the word
    assert bool((out == 7.0).all())

    # the context is still usable and the next call computes normally
    res = flash_attention_v2_cutlass(q, q, vt, False, 1 / math.sqrt(64), out=out)[0]
    check_status(dev)
    assert not bool((res == 7.0).all()) and not torch.isnan(res).any()


def test_failed_launch_surfaces_at_the_next_call_without_check_status():
    """A caller that never asks for the status (the reference's test.py:72-73 does not) still
    hears of a failed launch: the next call on the device refuses to run and says why, and the
    one after it starts clean.  Uses the library's own status word (status_word = NULL)."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.fa8_check_status(None, stream, None) == _lib.FA8_OK
    assert lib.fa8_selftest_expired_wait(None, 2000, stream) == _lib.FA8_OK
    torch.cuda.synchronize()                   # only so that the failing kernel has ended
    q = torch.randn(1, 2, 256, 64, device=dev).to(F8)
    vt = torch.randn(1, 2, 64, 256, device=dev).to(F8)
    out = torch.full((1, 2, 256, 64), 7.0, dtype=torch.float16, device=dev)
    p = _lib.Fa8FwdParams(q=q.data_ptr(), k=q.data_ptr(), v=vt.data_ptr(), o=out.data_ptr(), batch=1, heads=2,
                          seqlen=256, head_dim=64, softmax_scale=0.125, is_causal=0, v_layout=0, o_scale=1.0,
                          status_word=None)
    assert lib.fa8_fwd(ctypes.byref(p), stream) == _lib.FA8_ERR_DEVICE_TIMEOUT
    assert b"0x7e57" in lib.fa8_last_error_detail()
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())            # nothing was enqueued
    assert lib.fa8_fwd(ctypes.byref(p), stream) == _lib.FA8_OK
    assert lib.fa8_check_status(None, stream, None) == _lib.FA8_OK
    assert not bool((out == 7.0).all()) and not torch.isnan(out).any()
    # the operator raises the same way
    assert lib.fa8_selftest_expired_wait(None, 2000, stream) == _lib.FA8_OK
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="earlier launch"):
        flash_attention_v2_cutlass(q, q, vt, False, 0.125, out=out)
    flash_attention_v2_cutlass(q, q, vt, False, 0.125, out=out)
    check_status(dev)


def test_host_runner_returns_a_tensor_of_its_own_per_call():
    from cutlass_flash_atten_fp8_b200 import HostRunner
    dev = torch.device("cuda", 0)
    runner = HostRunner(dev, chunks=2)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 4, 256, 64, generator=g).to(F8)
    q2 = torch.randn(1, 4, 256, 64, generator=g).to(F8)
    vt = torch.randn(1, 4, 64, 256, generator=g).to(F8)
    first = runner(q, q, vt, False, 0.125)[0]
    keep = first.clone()
    second = runner(q2, q2, vt, False, 0.125)[0]
    assert first.data_ptr() != second.data_ptr()
    assert torch.equal(first, keep) and not torch.equal(first, second)
    mine = torch.empty(first.shape, dtype=torch.float16, pin_memory=True)
    third = runner(q, q, vt, False, 0.125, out=mine)[0]
    assert third.data_ptr() == mine.data_ptr() and torch.equal(third, first)


def test_selftest_argument_checks():
    lib = _lib.load()
    word = status_word(torch.device("cuda", 0))
    assert lib.fa8_selftest_expired_wait(word.data_ptr(), 0, None) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_selftest_expired_wait(word.data_ptr(), 2_000_000, None) == _lib.FA8_ERR_BAD_ARG
