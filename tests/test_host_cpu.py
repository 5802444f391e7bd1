"""Host-side logic that needs no GPU: operator argument checks, sharding, synthetic data."""
import pytest
import torch

from cutlass_flash_atten_fp8_b200 import flash_attention_v2_cutlass, synth
from cutlass_flash_atten_fp8_b200.shard import all_ranges, shard_range

F8 = torch.float8_e4m3fn


def test_operator_rejects_host_tensors_like_the_reference():
    # CHECK_CUDA of include/attention_api.cuh:12-13 -> RuntimeError through TORCH_CHECK
    q = torch.zeros(1, 1, 128, 64).to(F8)
    with pytest.raises(RuntimeError, match="q must be a CUDA tensor"):
        flash_attention_v2_cutlass(q, q, q.transpose(2, 3).contiguous(), False, 0.125)


def test_drop_in_module_name():
    # the reference's module name (setup.py:45, test.py:3): the compiled torch binding when it
    # has been built (an extension module is found ahead of a .py of the same name), else the
    # ctypes operator re-exported by attention_cutlass_fp8.py
    import attention_cutlass_fp8
    fn = attention_cutlass_fp8.flash_attention_v2_cutlass
    if attention_cutlass_fp8.__file__.endswith(".py"):
        assert fn is flash_attention_v2_cutlass
    else:
        assert "is_causal: bool = False" in fn.__doc__ and "softmax_scale" in fn.__doc__


def test_compiled_binding_builds_and_checks_its_inputs_like_the_reference():
    import importlib.util

    from cutlass_flash_atten_fp8_b200 import _lib
    from cutlass_flash_atten_fp8_b200.build import build_binding
    path = build_binding()
    spec = importlib.util.spec_from_file_location("attention_cutlass_fp8", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.abi_version() == _lib.load().fa8_version()
    q = torch.zeros(1, 1, 128, 64).to(F8)
    with pytest.raises(RuntimeError, match="q must be a CUDA tensor"):      # CHECK_CUDA, include/attention_api.cuh:12-13
        mod.flash_attention_v2_cutlass(q, q, q.transpose(2, 3).contiguous(), False, 0.125)


def test_quantize_per_head_wants_three_dimensions_before_anything_else():
    from cutlass_flash_atten_fp8_b200 import api
    x = torch.zeros(8, dtype=torch.float16)
    with pytest.raises(RuntimeError):          # a host tensor: CHECK_INPUT fires first, never an IndexError
        api.quantize_e4m3(x, per_head=True)


@pytest.mark.parametrize("n,world", [(2048, 8), (512, 4), (7, 3), (3, 8), (0, 2), (64, 1)])
def test_shard_ranges_partition_the_slices(n, world):
    r = all_ranges(n, world)
    assert r[0][0] == 0 and r[-1][1] == n
    for (a, b), (c, d) in zip(r, r[1:]):
        assert b == c and a <= b and c <= d
    sizes = [b - a for a, b in r]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(n, world, world)


def test_synthetic_slices_do_not_depend_on_the_shard():
    w = synth.Workload("t", 2, 3, 128, 64, True, outliers=True, seed=77)
    q, k, v, d = synth.make_qkv(w, "cpu")
    # same global amax -> identical bytes for a sub-range once the scale is shared
    assert q.shape == (6, 128, 64) and v.shape == (6, 64, 128)
    q2, k2, v2, d2 = synth.make_qkv(w, "cpu", 0, 6, transpose_v=False)
    assert torch.equal(v2.view(torch.uint8).transpose(1, 2), v.view(torch.uint8))
    assert float(q.float().abs().max()) == 448.0
    # outliers: 8 sigma entries present, so the bulk sits well below the maximum
    assert float(q.float().abs().median()) < 60.0
    assert all(x > 0 for x in d)


def test_workload_arithmetic():
    w = synth.WORKLOADS["mid_s4096_d128"]
    assert w.flops() == pytest.approx(4.398e12, rel=1e-3)
    assert w.hbm_bytes() == pytest.approx(1.342e9, rel=1e-3)
    assert synth.WORKLOADS["mid_s4096_d128_causal"].flops() == pytest.approx(2.199e12, rel=1e-3)
    assert synth.WORKLOADS["box_s8192_d128_causal"].flops() == pytest.approx(3.518e13, rel=1e-3)


@pytest.mark.parametrize("n,parts", [(512, 16), (18, 4), (3, 16), (1, 8), (7, 7)])
def test_host_runner_groups_partition_the_slices(n, parts):
    from cutlass_flash_atten_fp8_b200 import HostRunner
    g = HostRunner._groups(n, parts)
    assert len(g) == min(n, parts) and g[0][0] == 0 and g[-1][1] == n
    assert all(b == c for (_, b), (c, _) in zip(g, g[1:])) and all(b > a for a, b in g)
    for taper in (0.5, 2.0 / 3.0, 0.9):
        t = HostRunner._groups(n, parts, taper)
        assert t[0][0] == 0 and t[-1][1] == n
        assert all(b == c for (_, b), (c, _) in zip(t, t[1:])) and all(b > a for a, b in t)
        assert t[:max(0, len(g) - 2)] == g[:max(0, len(g) - 2)]   # only the last two groups are cut again
        sizes = [b - a for a, b in t[max(0, len(g) - 2):]]
        if len(g) >= 2:
            assert all(x >= y or y <= 2 for x, y in zip(sizes, sizes[1:]))   # ever smaller towards the end
    assert [b - a for a, b in HostRunner._groups(512, 8, 2.0 / 3.0)] == [64] * 6 + [43, 28, 19, 13, 8, 6, 4, 2, 2, 2, 1]
