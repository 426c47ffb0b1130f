"""Builds ``libxn_attn.so`` (hand-written CUDA for sm_100a + the C ABI) in-tree with nvcc."""
from __future__ import annotations

import glob
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libxn_attn.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the attention library cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    return any(os.path.getmtime(p) > built for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source of the package into one shared library beside this file."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-o", LIB_PATH, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    # nvcc needs a host compiler with OpenMP-free defaults; the system g++ is used
    env = dict(os.environ)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


def build_host_tool(name: str, force: bool = False) -> str:
    """Compiles host/<name>.cpp (a C++ program over the host mirror and the C ABI) beside the
    library and returns the path of the executable."""
    src = os.path.join(HERE, "host", name + ".cpp")
    exe = os.path.join(HERE, name)
    build_library()
    deps = [src, os.path.join(HERE, "host", "xor_net_attn.hpp"), os.path.join(INCLUDE, "xn_attn.h")]
    if force or not os.path.exists(exe) or any(os.path.getmtime(p) > os.path.getmtime(exe) for p in deps):
        cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-I", INCLUDE, "-I", os.path.join(HERE, "host"), src,
               "-o", exe, "-L", HERE, "-lxn_attn", f"-Wl,-rpath,{HERE}"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return exe


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
