"""Builds ``libtritium_b200.so`` in-tree with nvcc for sm_100a (no JIT cache, no other arch)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
LIB = os.path.join(OUT_DIR, "libtritium_b200.so")

CU_SOURCES = ["tb_api.cu", "kernels_exact.cu", "kernels_decode.cu", "kernels_prefill.cu", "kernels_comm.cu"]
CPP_SOURCES = ["tb_format.cpp"]
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "tritium_b200.h"))
    nvcc = _nvcc()
    objects = []
    for src in CU_SOURCES + CPP_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OUT_DIR, src.rsplit(".", 1)[0] + ".o")
        objects.append(obj)
        if not (force or _stale(obj, [path] + headers)):
            continue
        cmd = [nvcc, "-c", path, "-o", obj, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
               "-Xcompiler", "-ffp-contract=off"] + GENCODE
        if src == "kernels_exact.cu":
            cmd += ["--fmad=false"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += os.environ.get("TB_NVCC_FLAGS", "").split()
        subprocess.check_call(cmd)
    if force or _stale(LIB, objects):
        subprocess.check_call([nvcc, "-shared", "-o", LIB] + objects + ["-cudart", "static"] + GENCODE)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
