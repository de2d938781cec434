"""Build libvoxb200.so (the C-ABI library declared in include/vb_api.h) in-tree with nvcc for sm_100a.

    python -m vox_serve_b200.build [--force]

nvcc cross-compiles without a GPU.  Objects are cached under vox_serve_b200/lib/obj and rebuilt when a
source or header is newer.  The .so is git-ignored but travels to the GPU box with the tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "libvoxb200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

SOURCES = ["api.cu", "elementwise.cu", "attn.cu", "prefill_attn.cu", "prefill_attn_tc.cu", "kvcopy.cu", "encoder.cu", "gemm.cu", "sampler.cu", "snac.cu", "snac_mma.cu",
           "multicodebook.cu", "mimi.cu", "codec.cu", "norm_linear.cu", "window_attn.cu", "linear_attn.cu", "gated_recurrence.cu", "moe.cu", "short_conv.cu", "sigmoid_attn.cu", "selective_scan.cu"]
# subsets of the sources that serve one family of models: a first run that only needs that family compiles only these
# (into lib/libvoxb200_<profile>.so; entry points of the other sources are absent from it)
_TEXT = ["api.cu", "elementwise.cu", "gemm.cu", "sampler.cu", "norm_linear.cu", "window_attn.cu"]
PROFILES = {"text": _TEXT + ["linear_attn.cu", "moe.cu"],           # attention + decay attention + mixtures of experts
            "text_gated": _TEXT + ["gated_recurrence.cu"],           # attention + element-wise gated recurrence, dense feed-forward
            # attention + short convolutions + pooled-window sigmoid attention + selective scan + mixtures of experts
            "text_conv": _TEXT + ["moe.cu", "short_conv.cu", "sigmoid_attn.cu", "selective_scan.cu"]}
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return cand


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def lib_path(profile: str = None) -> str:
    return LIB if profile is None else os.path.join(LIBDIR, f"libvoxb200_{profile}.so")


def build(force: bool = False, verbose: bool = False, profile: str = None) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    sources, lib = (SOURCES, LIB) if profile is None else (PROFILES[profile], lib_path(profile))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE, "vb_api.h"))
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr:
            print(r.stderr)
        return o

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJDIR, s.replace(".cu", ".o")) for s in sources]
    if force or jobs or _stale(lib, objs):
        # (linked under a temporary name and renamed: another process may be loading the library meanwhile)
        tmp = f"{lib}.{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "--cudart", "static",
               "-o", tmp, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    prof = next((a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--profile=")), None)
    print(build(force="--force" in sys.argv, verbose=True, profile=prof))
