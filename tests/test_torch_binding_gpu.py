"""The compiled torch binding (module attention_cutlass_fp8, as the reference names its
extension: setup.py:45, csrc/attention_api.cpp:6-10) against the ctypes operator: same library,
same kernel, so the outputs must be bitwise equal; and against the reference's own fixtures with
the reference's tolerance (test.py:87)."""
import glob
import importlib.util
import math
import os

import numpy as np
import pytest
import torch

from cutlass_flash_atten_fp8_b200 import check_status, flash_attention_v2_cutlass
from cutlass_flash_atten_fp8_b200.build import binding_is_stale, binding_path

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def binding():
    path = binding_path()
    assert os.path.exists(path) and not binding_is_stale(), \
        "build the module first: python -m cutlass_flash_atten_fp8_b200.build --binding"
    spec = importlib.util.spec_from_file_location("attention_cutlass_fp8", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_fixtures_through_the_compiled_module(binding, golden_dir):
    dev = torch.device("cuda", 0)
    files = sorted(glob.glob(os.path.join(golden_dir, "ref_self_attention_*.npz")))
    assert len(files) >= 4
    for f in files:
        g = np.load(f)
        q8, k8, v8 = (torch.from_numpy(g[n]).view(F8).to(dev) for n in ("q", "k", "v"))
        vt = v8.transpose(2, 3).contiguous()
        causal, scale = bool(g["causal"]), float(g["scale"])
        got = binding.flash_attention_v2_cutlass(q8, k8, vt, causal, scale)        # the reference's call, test.py:72-73
        assert isinstance(got, list) and len(got) == 1 and got[0].dtype == torch.float16
        binding.check_status()
        want = flash_attention_v2_cutlass(q8, k8, vt, causal, scale)[0]
        check_status(dev)
        assert torch.equal(got[0].view(torch.int16), want.view(torch.int16)), f
        diff = (got[0].float().cpu() - torch.from_numpy(g["out"].astype(np.float32))).abs().max()
        assert float(diff) <= 1e-2, (f, float(diff))


def test_defaults_layouts_formats_and_streams(binding):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, 4, 320, 128, generator=g).to(F8).to(dev)
    k = torch.randn(2, 2, 448, 128, generator=g).to(F8).to(dev)          # grouped heads, longer keys
    v = torch.randn(2, 2, 448, 128, generator=g).to(F8).to(dev)
    vt = v.transpose(2, 3).contiguous()
    # defaults are the reference's: is_causal = false, softmax_scale = 1 (include/attention_api.h:10-11)
    a = binding.flash_attention_v2_cutlass(q, k, vt)[0]
    b = flash_attention_v2_cutlass(q, k, vt)[0]
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    sc = 1 / math.sqrt(128)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):                                          # the module follows torch's current stream
        c = binding.flash_attention_v2_cutlass(q, k, v, True, sc, v_layout="natural", o_scale=0.5)[0]
        binding.check_status()
    d = flash_attention_v2_cutlass(q, k, vt, True, sc, o_scale=0.5)[0]
    check_status(dev)
    assert torch.equal(c.view(torch.int16), d.view(torch.int16))
    q5, k5, v5 = (t.float().to(torch.float8_e5m2) for t in (q, k, vt))
    e = binding.flash_attention_v2_cutlass(q5, k5, v5, False, sc)[0]
    f = flash_attention_v2_cutlass(q5, k5, v5, False, sc)[0]
    binding.check_status()
    assert torch.equal(e.view(torch.int16), f.view(torch.int16))
    with pytest.raises(RuntimeError, match="must be contiguous"):         # CHECK_CONTIGUOUS, include/attention_api.cuh:14-15
        binding.flash_attention_v2_cutlass(q, k, v.transpose(2, 3), False, sc)
    with pytest.raises(RuntimeError, match="fa8 error"):                  # head_dim 48: rejected by the C ABI
        x = torch.zeros(1, 1, 64, 48, device=dev).to(F8)
        binding.flash_attention_v2_cutlass(x, x, x.transpose(2, 3).contiguous(), False, sc)
