"""Compile the reference project's CPU sources for this path into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The sources are compiled where they lie (they are
never copied into this repository); the output is a Python extension
``oracle/_ref/ts_ref_cpu*.so`` used as value oracle and as the timed CPU
baseline.  Files compiled (paths inside the reference project):

  torchsparse/backend/convolution/convolution_gather_scatter_cpu.cpp
  torchsparse/backend/hash/hash_cpu.cpp
  torchsparse/backend/others/count_cpu.cpp
  torchsparse/backend/voxelize/voxelize_cpu.cpp
  torchsparse/backend/devoxelize/devoxelize_cpu.cpp

``query_cpu.cpp`` / ``hashmap_cpu.*`` need google/dense_hash_map (sparsehash),
which is not installed, and are left out.

Usage:  python oracle/build_ref.py [path-to-reference-root]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ts_ref_cpu"

SOURCES = [
    "convolution/convolution_gather_scatter_cpu.cpp",
    "hash/hash_cpu.cpp",
    "others/count_cpu.cpp",
    "voxelize/voxelize_cpu.cpp",
    "devoxelize/devoxelize_cpu.cpp",
]


def so_path() -> str:
    return os.path.join(OUT, NAME + ".so")


def build(ref_root: str = "/root/reference", force: bool = False) -> str:
    backend = os.path.join(ref_root, "torchsparse", "backend")
    target = so_path()
    if os.path.exists(target) and not force:
        return target
    if not os.path.isdir(backend):
        raise FileNotFoundError(f"reference sources not found under {backend}")
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{backend}"]
    cflags = ["-O3", "-fopenmp", "-fPIC", "-std=c++17", f"-DTORCH_EXTENSION_NAME={NAME}",
              "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
              "-w"]
    srcs = [os.path.join(backend, s) for s in SOURCES] + [os.path.join(HERE, "ref_binding.cpp")]
    objs = [os.path.join(OUT, os.path.basename(s).replace(".cpp", ".o")) for s in srcs]

    def cc(pair):
        s, o = pair
        subprocess.check_call(["g++", *cflags, *inc, "-c", s, "-o", o])

    with ThreadPoolExecutor(max_workers=min(6, os.cpu_count() or 1)) as ex:
        list(ex.map(cc, zip(srcs, objs)))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    gomp_dir = "/usr/lib/gcc/x86_64-linux-gnu/13"
    link = ["g++", "-shared", *objs, "-o", target, f"-L{libdir}", f"-Wl,-rpath,{libdir}",
            "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    if os.path.isdir(gomp_dir):
        link += [f"-L{gomp_dir}"]
    link += ["-lgomp"]
    subprocess.check_call(link)
    for o in objs:
        os.remove(o)
    return target


def load():
    """Import the built module (raises if it has not been built)."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)

    path = so_path()
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print(build(root, force=True))
