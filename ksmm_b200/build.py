"""Builds libksmm_cu.so in-tree with nvcc for sm_100a (`python -m ksmm_b200.build`)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")


def build_library(jobs=None, verbose=False):
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", CSRC, f"-j{jobs}"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building libksmm_cu.so failed")
    lib = os.path.join(HERE, "libksmm_cu.so")
    if not os.path.exists(lib):
        raise RuntimeError(f"{lib} was not produced")
    return lib


def build_torch_extension(verbose=False):
    """Compiles csrc/torch_ext.cpp into ksmm_b200/ksmm_torch_ext*.so: the module the reference
    builds from kernel.cpp + kernel.cu (src/ksmm_py/layer/kronecker_sparse/kernel.cpp:25-50), here
    a binding layer over libksmm_cu.so with no kernel code of its own."""
    import sysconfig

    from torch.utils import cpp_extension as ce

    build_library(verbose=verbose)
    out = os.path.join(HERE, "ksmm_torch_ext" + sysconfig.get_config_var("EXT_SUFFIX"))
    src = os.path.join(CSRC, "torch_ext.cpp")
    deps = [src, os.path.join(HERE, "..", "include", "ksmm_cu.h")]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    import torch

    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=ksmm_torch_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}"]
    for inc in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", out, f"-L{HERE}", "-lksmm_cu", "-Wl,-rpath,$ORIGIN"]
    for lp in ce.library_paths("cuda"):
        cmd += [f"-L{lp}", f"-Wl,-rpath,{lp}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building the torch extension failed")
    return out


def load_torch_extension():
    """Imports the extension module, building it first when it is missing."""
    import importlib

    import torch  # noqa: F401  (libtorch must be loaded before the module)

    build_torch_extension()
    return importlib.import_module("ksmm_b200.ksmm_torch_ext")


if __name__ == "__main__":
    print(build_library(verbose=True))
    print(build_torch_extension(verbose=True))
