"""Build the CPU checkers (test infrastructure, never part of the shipped path).

  python -m oracle.build          # builds oracle/_build/libnnops_oracle.so (plain-C restatement)
                                  # and, when the reference tree is present, oracle/_ref/*.so

The reference route is compiled from the reference's own source files where they lie
(REFERENCE_ROOT: the directory NNOPS_REFERENCE_ROOT names, else the default below) with plain g++ -- its build system is not run --
plus oracle/ref_shim.cpp.  Outputs go only into oracle/_ref/ (git-ignored).  Two ISA variants
are produced because the int8 micro-kernel needs vpdpbusd: AVX-VNNI (the reference's default
flags) and AVX512-VNNI+VL; the loader picks the one the host CPU supports.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
# The nnops source tree: NNOPS_REFERENCE_ROOT, or a checkout named "reference" beside this repository.
REFERENCE_ROOT = Path(os.environ.get("NNOPS_REFERENCE_ROOT", str(HERE.parent.parent / "reference")))
CXX = os.environ.get("NNOPS_ORACLE_CXX", "/usr/bin/g++")
CC = os.environ.get("NNOPS_ORACLE_CC", "/usr/bin/gcc")

# The translation units the Linear/MatMul CPU route needs (reference src/CMakeLists.txt lists
# ~130; these close the link for ops/linear.cpp, ops/matmul.cpp, ops/quant_linear.cpp and ops/conv2d.cpp).
REF_SOURCES = [
    "ops/linear.cpp",
    "ops/matmul.cpp",
    "detail/cpu_features.cpp",
    "backend/cpu/common/memory_pool.cpp",
    "backend/cpu/matmul/matmul.cpp",
    "backend/cpu/matmul/matmul_i8.cpp",
    "backend/cpu/matmul/matmul_helper_i8.cpp",
    "backend/cpu/matmul/matmul_helper.cpp",
    "backend/cpu/matmul/matmul_small.cpp",
    "backend/cpu/matmul/matmul_qblock_fused.cpp",
    "backend/cpu/matmul/linear.cpp",
    "ops/quant_linear.cpp",
    "backend/cpu/quant_linear.cpp",
    # Conv2D's CPU route (the int8 convolution is checked against it): seven more units close the link.
    "ops/conv2d.cpp",
    "ops/depthwise_conv.cpp",
    "backend/cpu/conv/conv2d_implicit_gemm.cpp",
    "backend/cpu/conv/conv2d_implicit_gemm_i8.cpp",
    "backend/cpu/conv/conv2d_winograd.cpp",
    "backend/cpu/conv/depthwise_conv.cpp",
    "backend/cpu/conv/depthwise_conv_i8.cpp",
]

ISA_VARIANTS = {
    # name -> extra flags (the first is the reference's own CMake flag set)
    "avxvnni": ["-mavx2", "-mfma", "-mf16c", "-mavxvnni"],
    "avx512vnni": ["-mavx2", "-mfma", "-mf16c", "-mavx512f", "-mavx512bw", "-mavx512vl", "-mavx512vnni",
                   "-mprefer-vector-width=256"],
}


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build_port(force: bool = False) -> Path:
    """Compile the plain-C restatement.  -ffp-contract=off keeps every f32 step separately
    rounded, which the requant arithmetic depends on."""
    out_dir = HERE / "_build"
    out_dir.mkdir(exist_ok=True)
    out = out_dir / "libnnops_oracle.so"
    src = HERE / "nnops_oracle.c"
    if force or _stale(out, [src]):
        _run([CC, "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
              "-o", str(out), str(src), "-lm"])
    return out


def build_ref(force: bool = False) -> list[Path]:
    """Compile the reference CPU route + shim, one .so per ISA variant.  No-op (returns the
    prebuilt files, possibly none) when the reference tree is absent."""
    out_dir = HERE / "_ref"
    if not (REFERENCE_ROOT / "src" / "ops" / "linear.cpp").exists():
        return sorted(out_dir.glob("libnnops_ref_*.so")) if out_dir.exists() else []
    out_dir.mkdir(exist_ok=True)
    outs = []
    shim = HERE / "ref_shim.cpp"
    for name, isa in ISA_VARIANTS.items():
        out = out_dir / f"libnnops_ref_{name}.so"
        outs.append(out)
        srcs = [REFERENCE_ROOT / "src" / s for s in REF_SOURCES] + [shim]
        if not (force or _stale(out, srcs)):
            continue
        obj_dir = out_dir / f"obj_{name}"
        obj_dir.mkdir(exist_ok=True)
        # -include limits: two reference headers use std::numeric_limits without <limits> (GCC 13).
        flags = ["-std=c++23", "-O3", "-fPIC", "-fopenmp", "-include", "limits", "-DNDEBUG",
                 f"-I{REFERENCE_ROOT / 'include'}", f"-I{REFERENCE_ROOT / 'src'}"] + isa
        objs = []
        jobs = []
        for s in srcs:
            o = obj_dir / (str(s).replace("/", "_") + ".o")
            objs.append(o)
            jobs.append([CXX, *flags, "-c", str(s), "-o", str(o)])
        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            list(ex.map(_run, jobs))
        _run([CXX, "-shared", "-fopenmp", "-o", str(out), *map(str, objs)])
        for o in objs:
            o.unlink()
        obj_dir.rmdir()
    return outs


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_port(force))
    for p in build_ref(force):
        print(p)
