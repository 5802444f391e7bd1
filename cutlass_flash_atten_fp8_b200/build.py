"""Builds libfa8_b200.so (the C-ABI library with the sm_100a kernel) in-tree.

    python -m cutlass_flash_atten_fp8_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library sits next to this
file so that it travels with a snapshot of the source tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfa8_b200.so")
# Digest of the sources the library was built from, written next to it: a copy of the tree keeps
# file contents but not necessarily modification times, so staleness is decided by content.
HASH_PATH = os.path.join(PKG_DIR, "libfa8_b200.srchash")
SOURCES = ["fa8_fwd_sm100.cu", "fa8_quant.cu", "fa8_capi.cu"]
HEADERS = ["fa8_kernel.h", "ptx_sm100.cuh", os.path.join(REPO_DIR, "include", "fa8_b200.h")]


def nvcc_path() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def source_digest() -> str:
    h = hashlib.sha256()
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [h_ if os.path.isabs(h_) else os.path.join(CSRC, h_) for h_ in HEADERS]
    for d in deps:
        h.update(os.path.basename(d).encode() + b"\0")
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones present."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(HASH_PATH):
        return True
    try:
        now = source_digest()
    except FileNotFoundError:
        return False          # an installed copy without its sources cannot go stale
    with open(HASH_PATH) as f:
        return f.read().strip() != now


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    if os.path.exists(HASH_PATH):
        os.remove(HASH_PATH)
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-I" + os.path.join(REPO_DIR, "include"), "-I" + CSRC,
           "-Xcompiler", "-fPIC", "-shared", "-o", LIB_PATH]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfa8_b200.so")
    with open(HASH_PATH, "w") as f:
        f.write(source_digest() + "\n")
    return LIB_PATH


# The compiled torch binding: a pybind11 module with the reference's module name, built at the
# root of the tree (where `import attention_cutlass_fp8` finds it ahead of the ctypes shim of
# the same name) and linked against libfa8_b200.so through an $ORIGIN-relative run path.
BINDING_NAME = "attention_cutlass_fp8"
BINDING_SRC = os.path.join(CSRC, "torch_binding.cpp")


def binding_path() -> str:
    import sysconfig
    return os.path.join(REPO_DIR, BINDING_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def binding_is_stale() -> bool:
    out = binding_path()
    hp = out + ".srchash"
    if not os.path.exists(out) or not os.path.exists(hp):
        return True
    with open(hp) as f:
        return f.read().strip() != _binding_digest()


def _binding_digest() -> str:
    h = hashlib.sha256()
    for d in (BINDING_SRC, os.path.join(REPO_DIR, "include", "fa8_b200.h")):
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build_binding(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/torch_binding.cpp into attention_cutlass_fp8.<abi>.so (host compiler only:
    the CUDA code lives in libfa8_b200.so, which is built first if need be)."""
    build(force=False, verbose=verbose)
    out = binding_path()
    if not force and not binding_is_stale():
        return out
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"),
                                os.path.join(REPO_DIR, "include")]
    lib_dirs = ce.library_paths() + [os.path.join(cuda_home, "lib64"), PKG_DIR]
    # The module must share the C++ runtime (libstdc++.so) with torch, whose streams, strings and
    # exceptions cross into it: a compiler set-up that links libstdc++ statically gives the module
    # a private, uninitialised copy that crashes on the first formatted error message.  So the
    # system g++ is used unless FA8_CXX names another one, and the result is checked.
    cxx = os.environ.get("FA8_CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=" + BINDING_NAME,
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cmd += ["-I" + i for i in inc] + [BINDING_SRC, "-o", out]
    cmd += ["-L" + d for d in lib_dirs]
    cmd += ["-lfa8_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    cmd += ["-Wl,-rpath,$ORIGIN/" + os.path.basename(PKG_DIR)] + ["-Wl,-rpath," + d for d in ce.library_paths()]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("building the torch binding failed")
    with open(out, "rb") as f:
        if b"libstdc++.so" not in f.read():
            os.remove(out)
            raise RuntimeError(f"{cxx} linked libstdc++ statically into the torch binding; set FA8_CXX to a "
                               "g++ that links it dynamically")
    with open(out + ".srchash", "w") as f:
        f.write(_binding_digest() + "\n")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--binding" in sys.argv:
        print(build_binding(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
