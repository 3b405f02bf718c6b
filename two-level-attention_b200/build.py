"""Build the CUDA library in-tree with nvcc for sm_100a.

The result, ``libloda_b200.so`` next to this file, is a plain C-ABI shared
library (no torch, no Python symbols) that ``_capi.py`` loads with ctypes.
Every source is compiled to an object under ``build/`` (in parallel, only when
it or a header changed) and the objects are linked into the library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SOURCES = ["loda_append.cu", "loda_l1.cu", "loda_l2.cu", "loda_select_fused.cu", "loda_attn.cu", "loda_attn_mla.cu", "loda_tia.cu",
           "loda_tls.cu", "loda_shard.cu", "loda_capi.cu"]
LIB = os.path.join(HERE, "libloda_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _headers():
    csrc = os.path.join(HERE, "csrc")
    hs = [os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "loda_b200.h"))
    return hs


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(HERE, "csrc", s))]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def needs_build():
    deps = [os.path.join(HERE, "csrc", s) for s in _sources()] + _headers()
    return _stale(LIB, deps)


def build(force=False, verbose=False):
    if not force and not verbose and not needs_build():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc, headers = nvcc_path(), _headers()
    flags = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]
    if verbose:
        flags += ["-Xptxas", "-v"]
    jobs = []
    for s in _sources():
        src = os.path.join(HERE, "csrc", s)
        obj = os.path.join(OBJ_DIR, s[:-3] + ".o")
        if force or verbose or _stale(obj, [src] + headers):
            jobs.append((s, [nvcc] + flags + ["-c", src, "-o", obj]))

    def run(job):
        name, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return name, res

    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4) or 1) as pool:
        for name, res in pool.map(run, jobs):
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}:\n" + res.stdout + res.stderr)
            if verbose:
                print(res.stderr)
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in _sources()]
    res = subprocess.run([nvcc] + ARCH + ["-shared", "-o", LIB] + objs, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
