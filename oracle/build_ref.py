"""Build recipe for the reference's own CUDA extensions (test infrastructure).

Compiles the reference's two torch extensions straight from its source tree,
unmodified, for sm_100a, and writes only the resulting shared objects to
``oracle/_ref/``:

  _bitpack_cuda.<abi>.so      from bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu
                              and bitsmoe/quant/bitpack/bitpack_cuda_binding.cpp
  _mlp_forward_cuda.<abi>.so  from bitsmoe/algorithms/cpp/mlp_forward.cu
                              and bitsmoe/algorithms/cpp/mlp_forward_binding.cpp

The flags are those of the reference's setup.py:46-50 (``-O3 --use_fast_math
-lineinfo``; fast math is part of the reference's numerics) with only the
``-gencode`` list replaced (setup.py:38-44 lists sm_80/86/89 only).  No
reference source is copied anywhere.  The objects are used by the GPU parity
tests as the checker ("the reference's own implementation on the same seeded
inputs") and by nothing on the product path.

Usage:  python oracle/build_ref.py [--reference DIR] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

EXTS = {
    "_bitpack_cuda": [
        "bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu",
        "bitsmoe/quant/bitpack/bitpack_cuda_binding.cpp",
    ],
    "_mlp_forward_cuda": [
        "bitsmoe/algorithms/cpp/mlp_forward.cu",
        "bitsmoe/algorithms/cpp/mlp_forward_binding.cpp",
    ],
}


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    return inc, lib


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def ext_path(name: str) -> str:
    return os.path.join(OUT, name + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference: str, force: bool = False) -> None:
    os.makedirs(OUT, exist_ok=True)
    inc, torch_lib = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incflags = [f"-I{p}" for p in inc] + [f"-I{pyinc}", f"-I{cuda_home}/include"]
    jobs = []
    for name, srcs in EXTS.items():
        target = ext_path(name)
        srcs_abs = [os.path.join(reference, s) for s in srcs]
        if not force and os.path.exists(target) and all(
            os.path.getmtime(target) >= os.path.getmtime(s) for s in srcs_abs
        ):
            print(f"up to date: {target}")
            continue
        common = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  "-D_GLIBCXX_USE_CXX11_ABI=1", "-std=c++17"]
        objs = []
        for s in srcs_abs:
            obj = os.path.join(OUT, name + "_" + os.path.basename(s) + ".o")
            objs.append(obj)
            if s.endswith(".cu"):
                cmd = [os.path.join(cuda_home, "bin", "nvcc"), "-c", s, "-o", obj,
                       "-O3", "--use_fast_math", "-lineinfo",
                       "-gencode", "arch=compute_100a,code=sm_100a",
                       "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
                       "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                       "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
                       ] + common + incflags
            else:
                cmd = ["g++", "-c", s, "-o", obj, "-O3", "-fPIC"] + common + incflags
            jobs.append((name, cmd))
        link = ["g++", "-shared", "-o", target] + objs + [
            f"-L{torch_lib}", f"-L{cuda_home}/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
            f"-Wl,-rpath,{torch_lib}"]
        jobs.append((name + ":link", link))
    compile_jobs = [c for n, c in jobs if not n.endswith(":link")]
    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(_run, compile_jobs))
    for n, c in jobs:
        if n.endswith(":link"):
            _run(c)
    for name in EXTS:
        for f in os.listdir(OUT):
            if f.startswith(name + "_") and f.endswith(".o"):
                os.remove(os.path.join(OUT, f))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a BitsMoE source tree")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.reference):
        print(f"reference tree not found at {a.reference}; nothing built", file=sys.stderr)
        sys.exit(0)
    build(a.reference, a.force)
