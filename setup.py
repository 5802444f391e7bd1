"""Install recipe.  The reference's setup.py (:42-113) builds one CUDAExtension called
attention_cutlass_fp8; here the CUDA code is a plain shared library with a C ABI
(libfa8_b200.so, built by nvcc for sm_100a) and the module of that name is a thin torch
binding linked against it, so the build step runs the two recipes of
cutlass_flash_atten_fp8_b200/build.py instead of torch's CUDAExtension machinery.

    python setup.py build_ext --inplace        # build in the source tree (what build() does)
    pip install --no-build-isolation .         # install the package, the library and the module

Needs nvcc (CUDA_HOME, default /usr/local/cuda), a host C++17 compiler and the torch the
module is to be used with.
"""
import importlib.util
import os
import shutil

from setuptools import Extension, setup
from setuptools.command.build_ext import build_ext

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = "cutlass_flash_atten_fp8_b200"


def _recipes():
    # build.py is loaded by path: importing the package would need the library it is about to build
    spec = importlib.util.spec_from_file_location("_fa8_build", os.path.join(ROOT, PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildNative(build_ext):
    """Builds libfa8_b200.so and the attention_cutlass_fp8 module in the tree, then copies them
    to where the command's mode wants them."""

    def run(self):
        b = _recipes()
        lib = b.build()
        module = b.build_binding()
        if self.inplace:
            return
        dst_pkg = os.path.join(self.build_lib, PKG)
        os.makedirs(dst_pkg, exist_ok=True)
        shutil.copy2(lib, dst_pkg)
        shutil.copy2(b.HASH_PATH, dst_pkg)
        shutil.copy2(module, self.build_lib)


setup(
    name="cutlass_flash_atten_fp8_b200",
    version="0.2.0",
    description="FP8 flash-attention forward for B200 (sm_100a) behind the operator interface of "
                "weishengying/cutlass_flash_atten_fp8",
    packages=[PKG],
    package_data={PKG: ["csrc/*", "*.so", "*.srchash"]},
    data_files=[("include", ["include/fa8_b200.h"])],
    # one placeholder so that build_ext runs; BuildNative.run does the work
    ext_modules=[Extension("attention_cutlass_fp8", sources=[])],
    cmdclass={"build_ext": BuildNative},
    python_requires=">=3.9",
    install_requires=["torch"],
)
