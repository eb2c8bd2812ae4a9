"""Compiles csrc/ into libvioletto_b200.so for sm_100a with nvcc (no GPU needed to build)."""
from __future__ import annotations

import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libvioletto_b200.so"
SOURCES = ["abi.cc", "generator.cc", "router.cc", "engine.cu", "k_small.cu", "k_matmul.cu", "k_attn.cu", "k_gemm.cu", "k_spec.cu", "k_draft.cu", "k_prefill.cu", "k_block.cu", "k_limite.cu", "k_limite_attn.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-x", "cu",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [src, HERE.parent / "include" / "violetto.h"])
    return obj.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    # Objects compiled with other extra flags (VLT_NVCC_FLAGS: the developer probes) are not reused.
    extra, stamp = os.environ.get("VLT_NVCC_FLAGS", ""), objdir / "flags.txt"
    if not stamp.exists() or stamp.read_text() != extra:
        force = True
        stamp.write_text(extra)
    jobs = []
    for name in SOURCES:
        src, obj = CSRC / name, objdir / (name + ".o")
        if force or _stale(obj, src):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([NVCC, *FLAGS, *os.environ.get("VLT_NVCC_FLAGS", "").split(), "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
        (objdir / (src.name + ".log")).write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [str(objdir / (n + ".o")) for n in SOURCES]
    if jobs or not LIB.exists():
        r = subprocess.run([NVCC, "-shared", "-o", str(LIB), *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
