"""Builds the C-ABI shared library ``libb200attn.so`` in-tree with nvcc for
sm_100a.  No torch headers are involved: the library speaks raw pointers.

    python -m auto_infer_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libb200attn.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)

SOURCES = [
    "host_util.cu",
    "decode_plan.cu",
    "reshape_and_cache.cu",
    "paged_decode_gqa.cu",
    "paged_prefill_gqa.cu",
    "mla_decode.cu",
    "lse_combine.cu",
    "cp_exchange.cu",
    "copy_blocks.cu",
    "rope_cache.cu", "paged_mha.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build " + LIB_NAME)
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source for sm_100a and link the shared library.  Returns
    its path.  Objects are rebuilt only when a source or header changed."""
    nvcc = _nvcc()
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "b200_attention.h"))
    objects = []
    logs = []
    for src in SOURCES:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objects.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src_path, "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            logs.append(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}")
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if force or _stale(LIB_PATH, objects):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objects]
        res = subprocess.run(cmd, capture_output=True, text=True)
        logs.append(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}")
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if logs:
        with open(os.path.join(obj_dir, "build.log"), "w") as fh:
            fh.write("\n".join(logs))
    if verbose:
        print("\n".join(logs))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
