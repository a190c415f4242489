"""Build ``aihwkit_b200/csrc/libaihwkit_b200.so`` in-tree with nvcc for sm_100a.

    python -m aihwkit_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library links cudart statically and has no torch
dependency; ``libcuda`` entry points (tensor maps) are resolved at run time.
"""

from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "libaihwkit_b200.so")
OBJ = os.path.join(CSRC, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(
        glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
        + glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    )
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    logs = {}

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            logs[src] = res.stderr
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(OUT, objs):
        # A C-ABI library keeps its runtimes to itself: the CUDA runtime and the C++ runtime are
        # linked statically and hidden (-Bsymbolic, --exclude-libs), so that a process which also
        # holds other copies (torch exports its own instantiations of std::string and
        # std::ostringstream members, and loads the shared CUDA runtime) cannot have this
        # library's calls bound to them. Without this, loading the library as a dependency of a
        # torch extension crashed in its error path (the message is built with std::ostringstream).
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-cudart", "static", "-ldl", "-lpthread",
                                                     "-Xcompiler", "-static-libstdc++",
                                                     "-Xlinker", "-Bsymbolic", "-Xlinker", "--exclude-libs=ALL"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        for src, log in logs.items():
            print(f"== {os.path.basename(src)}\n{log}")
    with open(os.path.join(OBJ, "ptxas.log"), "a", encoding="utf-8") as f:
        for src, log in logs.items():
            f.write(f"== {os.path.basename(src)}\n{log}\n")
    return OUT


def build_pybind(verbose: bool = False):
    """Compile ``csrc/pybind_module.cpp`` - the pybind11 / torch binding over the C ABI that a
    maintainer of the reference would link in place of its own tile classes - in-tree
    (``csrc/build_pybind/ab200_pybind.so``) and return the imported module.  The binding sees the
    library through ``include/aihwkit_b200.h`` and the linker only."""
    from torch.utils.cpp_extension import load

    build()
    out_dir = os.path.join(HERE, "csrc", "build_pybind")
    os.makedirs(out_dir, exist_ok=True)
    return load(
        name="ab200_pybind",
        sources=[os.path.join(HERE, "csrc", "pybind_module.cpp")],
        extra_include_paths=[os.path.join(os.path.dirname(HERE), "include")],
        extra_cflags=["-O2"],
        extra_ldflags=[f"-L{os.path.join(HERE, 'csrc')}", "-laihwkit_b200",
                       f"-Wl,-rpath,{os.path.join(HERE, 'csrc')}"],
        build_directory=out_dir,
        with_cuda=True,
        verbose=verbose,
    )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
