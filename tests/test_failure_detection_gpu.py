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

    # while the status word is non-zero every attention CTA returns at once, output untouched
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


def test_selftest_argument_checks():
    lib = _lib.load()
    assert lib.fa8_selftest_expired_wait(None, 1000, None) == _lib.FA8_ERR_BAD_ARG
    word = status_word(torch.device("cuda", 0))
    assert lib.fa8_selftest_expired_wait(word.data_ptr(), 0, None) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_selftest_expired_wait(word.data_ptr(), 2_000_000, None) == _lib.FA8_ERR_BAD_ARG
