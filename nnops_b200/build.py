"""Compile the CUDA sources of libnnb200 for sm_100a with nvcc, in-tree.

    python -m nnops_b200.build [--force] [--verbose]

Output: nnops_b200/lib/libnnb200.so (git-ignored; shipped to GPU machines as a built file).
nvcc cross-compiles without a GPU.  -fmad=false keeps every f32 multiply and add separately
rounded unless a kernel asks for an fma explicitly -- the int8 requantisation must match the
CPU arithmetic bit for bit.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libnnb200.so"
NVCC = os.environ.get("NNB200_NVCC", "/usr/local/cuda/bin/nvcc")

SOURCES = ["capi.cu", "gemm_i8_umma.cu", "gemm_i8_simt.cu", "gemm_i8_decode.cu", "gemm_i8_skinny.cu", "q4_1_gemv.cu", "q4_1_gemv_mma.cu", "q4_1_gemv_dsq.cu", "q4_1_gemm_umma.cu", "gemm_f16_umma.cu", "shard_gather.cu", "quant_linear.cu", "prepack.cu", "static_scratch.cu", "mma_peak.cu", "conv2d_i8.cu"]
HEADERS = ["ptx.cuh", "ptx_pair.cuh", "epilogue.cuh", "internal.cuh", "q4_1_common.cuh", "../../include/nnb200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo", "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    headers = [CSRC / h for h in HEADERS]
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(name: str) -> Path:
        src = CSRC / name
        obj = obj_dir / (name + ".o")
        if force or _stale(obj, [src, *headers]):
            r = subprocess.run([NVCC, *flags, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _stale(LIB, objs):
        r = subprocess.run([NVCC, "-shared", "-o", str(LIB), *map(str, objs)],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
