"""Generates tests/golden/ref_self_attention_*.npz by calling the REFERENCE's own
oracle function, ``self_attention`` of the reference's test.py (lines 25-33), on
CPU.  Run once in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

test.py imports two GPU-only extensions at module level and allocates its mask
with device="cuda".  Neither is touched in the reference tree: the two imports
are satisfied by empty stand-in modules, and torch.ones is wrapped for the
duration of the call so that the mask is allocated on the CPU.  Inputs follow
test.py:12-23 (seed 180, N(0, 0.5^2) fp16, clamp to +-0.1, cast to e4m3), shapes
are small enough to commit.
"""
import importlib.util
import math
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA8_REFERENCE_DIR", "")
if not os.path.isfile(os.path.join(REF, "test.py")):
    sys.exit("usage: make_golden.py REFERENCE_DIR (a checkout of weishengying/cutlass_flash_atten_fp8)")
HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_test_module():
    for name, attrs in (("attention_cutlass_fp8", {"flash_attention_v2_cutlass": None}),
                        ("vllm_flash_attn", {"flash_attn_func": None})):
        mod = types.ModuleType(name)
        for k, v in attrs.items():
            setattr(mod, k, v)
        sys.modules[name] = mod
    spec = importlib.util.spec_from_file_location("reference_test", os.path.join(REF, "test.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)          # guarded by __main__, only defines functions
    return mod


def on_cpu(fn, *args, **kwargs):
    real_ones = torch.ones

    def ones_cpu(*a, **k):
        k.pop("device", None)
        return real_ones(*a, **k)

    torch.ones = ones_cpu
    try:
        return fn(*args, **kwargs)
    finally:
        torch.ones = real_ones


def make_inputs(B, H, S, D):
    # test.py:12-23 on CPU
    def one():
        x = torch.empty((B, H, S, D), dtype=torch.float16).normal_(mean=0.0, std=0.5)
        return x.clamp(-0.1, 0.1).to(torch.float8_e4m3fn)
    return one(), one(), one()


def main():
    ref = load_reference_test_module()
    torch.manual_seed(180)
    cases = [
        ("b1h2s128d64_causal", 1, 2, 128, 64, True, 1.0 / math.sqrt(128)),      # test.py:57 scale = 1/sqrt(S)
        ("b1h2s128d64_full", 1, 2, 128, 64, False, 1.0 / math.sqrt(64)),
        ("b2h2s256d128_causal", 2, 2, 256, 128, True, 1.0 / math.sqrt(256)),
        ("b1h1s384d128_full", 1, 1, 384, 128, False, 1.0 / math.sqrt(128)),
    ]
    for name, B, H, S, D, causal, scale in cases:
        q8, k8, v8 = make_inputs(B, H, S, D)
        out = on_cpu(ref.self_attention, q8.to(torch.float16), k8.to(torch.float16),
                     v8.to(torch.float16), causal=causal, sm_scale=scale)
        np.savez_compressed(
            os.path.join(HERE, f"ref_self_attention_{name}.npz"),
            q=q8.view(torch.uint8).numpy(), k=k8.view(torch.uint8).numpy(),
            v=v8.view(torch.uint8).numpy(), out=out.numpy().astype(np.float16),
            causal=np.array(causal), scale=np.array(scale, dtype=np.float64))
        print(name, tuple(out.shape), float(out.abs().max()))


if __name__ == "__main__":
    main()
