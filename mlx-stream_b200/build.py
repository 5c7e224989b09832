"""Builds libmlxs_moe.so (the C-ABI library) in-tree with nvcc for sm_100a.  No torch involved."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libmlxs_moe.so"
SOURCES = ["api.cu", "router.cu", "dispatch.cu", "exl3.cu", "shared_combine.cu", "exl3_static.cu", "exl3_probe.cu", "fp4_native_probe.cu", "fp4.cu", "ep.cu", "exl3_prefill.cu", "fp4_prefill.cu", "fp4_native.cu", "dense_gemm.cu", "front.cu", "manifest.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v", "--expt-relaxed-constexpr"]
# extra compiler flags for a measurement build (e.g. MLXS_NVCC_EXTRA=-DMLXS_LANE_COUNTERS; rebuild with --force, and
# again without the variable afterwards)
FLAGS += os.environ.get("MLXS_NVCC_EXTRA", "").split()


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [src] +
                 list((HERE.parent / "include").glob("*.h")))
    return obj.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    bdir = HERE / "build"
    bdir.mkdir(exist_ok=True)
    jobs = []
    for s in SOURCES:
        src, obj = CSRC / s, bdir / (s + ".o")
        if force or _stale(obj, src):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([NVCC, *FLAGS, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
        (bdir / (src.name + ".log")).write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr[-4000:]}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        logs = list(ex.map(compile_one, jobs))
    if verbose:
        for lg in logs:
            print(lg)
    objs = [str(bdir / (s + ".o")) for s in SOURCES]
    if jobs or not OUT.exists():
        r = subprocess.run([NVCC, "-shared", "-o", str(OUT), *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
