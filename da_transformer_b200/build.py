"""Builds the CUDA kernels and the C ABI into ``da_transformer_b200/libdat_b200.so``.

    python -m da_transformer_b200.build [--verbose] [--force]

nvcc cross-compiles for sm_100a without a GPU.  The shared object is built in-tree,
next to this file, and is loaded with ctypes by ``_native.py``.  The benchmark's
measurement probes (``csrc/bench_probe``) go into a library of their own,
``libdat_bench_probe.so``, which the operator path never loads.
"""
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdat_b200.so")
PROBE_LIB = os.path.join(HERE, "libdat_bench_probe.so")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def probe_sources():
    return sorted(glob.glob(os.path.join(CSRC, "bench_probe", "*.cu")))


def _deps():
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [
        os.path.join(os.path.dirname(HERE), "include", "dat_b200.h")]


def up_to_date():
    if not os.path.exists(LIB) or not os.path.exists(PROBE_LIB):
        return False
    t = os.path.getmtime(LIB)
    tp = os.path.getmtime(PROBE_LIB)
    return (all(os.path.getmtime(p) <= t for p in _deps())
            and all(os.path.getmtime(p) <= tp for p in probe_sources()))


def nvcc_path():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libdat_b200.so")
    return nvcc


def _link(out, srcs, verbose):
    cmd = [nvcc_path(), *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-o", out + ".tmp"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += srcs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed building {os.path.basename(out)}")
    os.replace(out + ".tmp", out)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    _link(LIB, sources(), verbose)
    _link(PROBE_LIB, probe_sources(), verbose)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
