"""The C-ABI library loads without a GPU and exports what include/fa8_b200.h declares.
No compute call is made here."""
import ctypes
import os
import re

from cutlass_flash_atten_fp8_b200 import _lib
from cutlass_flash_atten_fp8_b200.build import LIB_PATH, REPO_DIR, build


def _declared_functions():
    text = open(os.path.join(REPO_DIR, "include", "fa8_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa8_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_and_loads():
    build()
    assert os.path.exists(LIB_PATH)
    lib = _lib.load()
    assert lib.fa8_version() == 109


def test_every_declared_symbol_is_exported():
    raw = ctypes.CDLL(LIB_PATH)
    declared = _declared_functions()
    assert set(declared) == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(raw, name), name


def test_error_strings_and_support_query():
    lib = _lib.load()
    for code in (0, -1, -2, -3, -4):
        assert len(lib.fa8_error_string(code)) > 0
    assert lib.fa8_error_string(-99) == b"unknown fa8 status"
    assert lib.fa8_supported(4096, 128, _lib.FA8_V_TRANSPOSED) == _lib.FA8_OK
    assert lib.fa8_supported(128, 64, _lib.FA8_V_TRANSPOSED) == _lib.FA8_OK
    assert lib.fa8_supported(128, 96, _lib.FA8_V_TRANSPOSED) == _lib.FA8_OK
    assert lib.fa8_supported(128, 32, _lib.FA8_V_NATURAL) == _lib.FA8_OK
    assert lib.fa8_supported(128, 256, _lib.FA8_V_NATURAL) == _lib.FA8_OK
    assert lib.fa8_supported(128, 48, _lib.FA8_V_TRANSPOSED) == _lib.FA8_ERR_UNSUPPORTED
    assert lib.fa8_supported(128, 288, _lib.FA8_V_TRANSPOSED) == _lib.FA8_ERR_UNSUPPORTED
    # only V^T has the sequence as its contiguous axis (row strides of 16 bytes for the copy engine)
    assert lib.fa8_supported(100, 64, _lib.FA8_V_TRANSPOSED) == _lib.FA8_ERR_UNSUPPORTED
    assert lib.fa8_supported(100, 64, _lib.FA8_V_NATURAL) == _lib.FA8_OK
    assert lib.fa8_supported(1, 128, _lib.FA8_V_NATURAL) == _lib.FA8_OK
    assert b"multiple of 32" in lib.fa8_error_string(_lib.FA8_ERR_UNSUPPORTED)
    assert lib.fa8_supported(0, 64, _lib.FA8_V_TRANSPOSED) == _lib.FA8_ERR_UNSUPPORTED


def test_work_plan_large_problems_keep_the_two_tile_items():
    """The steady-state plan (items of two query tiles, causal ones paired) is what every
    problem that fills the GPU gets; the baseline configurations are such problems."""
    wp = _lib.work_plan
    assert wp(512, 4096, 128, False, 148) == {"rows_per_item": 256, "paired": False, "items_per_slice": 16, "units": 8192}
    assert wp(512, 4096, 128, True, 148) == {"rows_per_item": 256, "paired": True, "items_per_slice": 16, "units": 4096}
    assert wp(512, 1024, 64, False, 148) == {"rows_per_item": 256, "paired": False, "items_per_slice": 4, "units": 2048}
    assert wp(32, 16384, 128, True, 148) == {"rows_per_item": 256, "paired": True, "items_per_slice": 64, "units": 1024}
    assert wp(256, 8192, 128, True, 148)["rows_per_item"] == 256
    # one query tile per CTA at head dims above 128
    assert wp(64, 4096, 256, False, 148) == {"rows_per_item": 128, "paired": False, "items_per_slice": 32, "units": 2048}
    # between half a wave and a wave of two-tile items nothing finer fits one wave
    assert wp(36, 1024, 128, False, 148)["rows_per_item"] == 256
    assert wp(64, 1024, 64, True, 148) == {"rows_per_item": 256, "paired": True, "items_per_slice": 4, "units": 128}


def test_work_plan_small_problems_are_cut_finer():
    """Fewer units than half the SMs: one-tile items and/or unpaired causal items, as long as
    they fit one wave of the grid; every query row is covered exactly once either way."""
    wp = _lib.work_plan
    assert wp(16, 1024, 128, False, 148) == {"rows_per_item": 128, "paired": False, "items_per_slice": 8, "units": 128}
    assert wp(16, 1024, 64, True, 148) == {"rows_per_item": 128, "paired": False, "items_per_slice": 8, "units": 128}
    p = wp(32, 1024, 128, True, 148)
    assert p["units"] <= 148 and (p["rows_per_item"], p["paired"]) in ((128, True), (256, False))
    assert wp(2, 128, 64, False, 148) == {"rows_per_item": 128, "paired": False, "items_per_slice": 1, "units": 2}
    for slices in (1, 3, 16, 40, 75, 200):
        for seqlen in (1, 100, 128, 129, 640, 1000, 4096):
            for causal in (False, True):
                for d in (32, 64, 128, 192, 256):
                    p = wp(slices, seqlen, d, causal, 148)
                    assert p["rows_per_item"] in (128, 256)
                    assert p["items_per_slice"] == -(-seqlen // p["rows_per_item"])
                    per_slice = (p["items_per_slice"] + 1) // 2 if p["paired"] else p["items_per_slice"]
                    assert p["units"] == slices * per_slice
                    assert not (p["paired"] and not causal)
                    if d > 128:
                        assert p["rows_per_item"] == 128
    lib = _lib.load()
    out = (ctypes.c_int32 * 4)()
    assert lib.fa8_work_plan(0, 128, 0, 64, 0, 148, ctypes.byref(out)) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_work_plan(1, 128, 0, 64, 0, 0, ctypes.byref(out)) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_work_plan(1, 128, 0, 48, 0, 148, ctypes.byref(out)) == _lib.FA8_ERR_UNSUPPORTED
    assert lib.fa8_work_plan(1, 128, 0, 64, 0, 148, None) == _lib.FA8_ERR_BAD_ARG


def test_argument_validation_needs_no_gpu():
    lib = _lib.load()
    assert lib.fa8_fwd(None, None) == _lib.FA8_ERR_BAD_ARG
    p = _lib.Fa8FwdParams()          # all zero: null pointers
    assert lib.fa8_fwd(ctypes.byref(p), None) == _lib.FA8_ERR_BAD_ARG
    fake = 0x1000                    # never dereferenced: validation fails first
    p = _lib.Fa8FwdParams(q=fake, k=fake, v=fake, o=fake, batch=1, heads=1, seqlen=128, head_dim=64,
                          softmax_scale=0.0, is_causal=0, v_layout=0, o_scale=1.0, status_word=None)
    assert lib.fa8_fwd(ctypes.byref(p), None) == _lib.FA8_ERR_BAD_ARG          # scale must be > 0
    p.softmax_scale = 0.125
    p.q = fake + 8
    assert lib.fa8_fwd(ctypes.byref(p), None) == _lib.FA8_ERR_BAD_ARG          # 16-byte alignment
    p.q = fake
    p.head_dim = 48
    assert lib.fa8_fwd(ctypes.byref(p), None) == _lib.FA8_ERR_UNSUPPORTED
    p.head_dim = 64
    p.v_layout = 7
    assert lib.fa8_fwd(ctypes.byref(p), None) == _lib.FA8_ERR_BAD_ARG
    # without a device there is no library-owned status word to fall back on
    assert lib.fa8_check_status(None, None, None) == _lib.FA8_ERR_BAD_ARG
    assert lib.fa8_selftest_expired_wait(None, 1000, None) == _lib.FA8_ERR_BAD_ARG


def test_stale_library_is_not_loaded_silently(tmp_path, monkeypatch):
    from cutlass_flash_atten_fp8_b200 import build as b
    build()
    assert not b.is_stale()
    monkeypatch.setattr(b, "source_digest", lambda: "0" * 64)
    assert b.is_stale()
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "is_stale", b.is_stale)
    try:
        _lib.load()
    except ImportError as e:
        assert "older than its sources" in str(e)
    else:
        raise AssertionError("a stale library was loaded")
