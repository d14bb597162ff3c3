"""In-tree build of the CUDA extension ``tinyllmforge_b200/_C*.so`` for sm_100a.

Kernels (``csrc/**/*.cu``) are compiled with nvcc directly (they do not include torch headers, so a file
rebuilds in seconds); ``csrc/host/bindings.cpp`` is the only translation unit that sees torch.  Objects are
cached under ``build/`` by content hash of the source, its headers and the flags.  nvcc cross-compiles without
a GPU, so this runs on a CPU-only machine.

    python -m tinyllmforge_b200.build_ext [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(ROOT, "build", "ext")
PKG = os.path.join(ROOT, "tinyllmforge_b200")
EXT_NAME = "_C"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def ext_path() -> str:
    return os.path.join(PKG, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd, verbose, log_path=None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stdout + r.stderr)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what changed and link; returns the path of the shared object."""
    import torch
    from torch.utils import cpp_extension

    os.makedirs(BUILD, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "include", "*"))
    cu_files = sorted(glob.glob(os.path.join(CSRC, "**", "*.cu"), recursive=True))
    cpp_files = [os.path.join(CSRC, "host", "bindings.cpp")]
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include") if os.path.sep in _nvcc() else "/usr/local/cuda/include"

    jobs, objs = [], []
    for src in cu_files:
        tag = _digest([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD, os.path.basename(src) + "." + tag + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append(([_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj], obj + ".log"))
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=" + EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
                 f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    incs = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_inc}"]
    for src in cpp_files:
        tag = _digest([src], " ".join(cxx_flags) + torch.__version__)
        obj = os.path.join(BUILD, os.path.basename(src) + "." + tag + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((["g++"] + cxx_flags + incs + ["-c", src, "-o", obj], obj + ".log"))

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _run(j[0], verbose, j[1]), jobs))

    out = ext_path()
    stamp = os.path.join(BUILD, "link.stamp")
    link_tag = _digest(objs, "link")
    if force or jobs or not os.path.exists(out) or not os.path.exists(stamp) or open(stamp).read() != link_tag:
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_lib = os.path.join(os.path.dirname(cuda_inc), "lib64")
        cmd = ["g++", "-shared", "-o", out] + objs + [
            f"-L{torch_lib}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-lcudart", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"]
        _run(cmd, verbose)
        with open(stamp, "w") as f:
            f.write(link_tag)
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the cached compile logs."""
    lines = []
    for log in sorted(glob.glob(os.path.join(BUILD, "*.cu.*.o.log"))):
        with open(log) as f:
            txt = f.read()
        for ln in txt.splitlines():
            if "Compiling entry function" in ln or "Used " in ln or "spill" in ln:
                lines.append(ln.strip())
    return "\n".join(lines)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    if "--report" in sys.argv:
        print(ptxas_report())
