"""Build the C++23 host side: the operator front end + CUDA backend glue, and the C++ test
programs.

    python -m nnops_b200.host.build

Outputs (all git-ignored, shipped as built files):
  nnops_b200/lib/libnnb200_host.so      operator front end + backend glue against the stand-alone API mirror
  tests/cpp/_bin/test_ops_standalone    operator tests against that library
and, only where the nnops source tree is present (the directory NNOPS_REFERENCE_ROOT names, else the default below):
  nnops_b200/lib/libnnops_b200_dropin.so   nnops' own front end (src/ops/linear.cpp, matmul.cpp, quant_linear.cpp, conv2d.cpp) and CPU route,
                                           compiled in place with NNOPS_HAS_CUDA, linked against THIS backend
  tests/cpp/_bin/test_ops_dropin           the same tests through the real nnops API, CUDA vs nnops' CPU route
"""
from __future__ import annotations

import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from .. import build as lib_build

HOST = Path(__file__).resolve().parent
ROOT = HOST.parent.parent
LIB_DIR = HOST.parent / "lib"
BIN_DIR = ROOT / "tests" / "cpp" / "_bin"
# The nnops source tree: NNOPS_REFERENCE_ROOT, or a checkout named "reference" beside this repository.
REFERENCE_ROOT = Path(os.environ.get("NNOPS_REFERENCE_ROOT", str(ROOT.parent / "reference")))
CXX = os.environ.get("NNB200_CXX", "/usr/bin/g++")
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

# The reference translation units behind Linear/MatMul on the CPU (same list as oracle/build.py).
REF_SOURCES = [
    "ops/linear.cpp", "ops/matmul.cpp", "detail/cpu_features.cpp", "backend/cpu/common/memory_pool.cpp",
    "backend/cpu/matmul/matmul.cpp", "backend/cpu/matmul/matmul_i8.cpp", "backend/cpu/matmul/matmul_helper_i8.cpp",
    "backend/cpu/matmul/matmul_helper.cpp", "backend/cpu/matmul/matmul_small.cpp",
    "backend/cpu/matmul/matmul_qblock_fused.cpp", "backend/cpu/matmul/linear.cpp",
    "ops/quant_linear.cpp", "backend/cpu/quant_linear.cpp",
    # Conv2D's front end and the CPU route its tests compare with.
    "ops/conv2d.cpp", "ops/depthwise_conv.cpp", "backend/cpu/conv/conv2d_implicit_gemm.cpp",
    "backend/cpu/conv/conv2d_implicit_gemm_i8.cpp", "backend/cpu/conv/conv2d_winograd.cpp",
    "backend/cpu/conv/depthwise_conv.cpp", "backend/cpu/conv/depthwise_conv_i8.cpp",
]
COMMON = ["-std=c++23", "-O2", "-fPIC", "-Wall", f"-I{ROOT / 'include'}"]


def _run(cmd):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def _stale(out: Path, deps) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(d).exists() and Path(d).stat().st_mtime > t for d in deps)


def _rpath(*dirs):
    return ["-Wl,-rpath," + ":".join(str(d) for d in dirs)]


def build_standalone(force=False) -> Path:
    lib = lib_build.build()
    out = LIB_DIR / "libnnb200_host.so"
    srcs = [HOST / "cuda_backend.cpp", HOST / "quant_backend.cpp", HOST / "conv_backend.cpp", HOST / "ops_frontend.cpp"]
    deps = srcs + [HOST / "staging.hpp", ROOT / "include" / "nnops_b200" / "nnops_api.hpp", ROOT / "include" / "nnb200.h", lib]
    if force or _stale(out, deps):
        _run([CXX, *COMMON, "-shared", "-o", out, *srcs, f"-L{LIB_DIR}", "-lnnb200", *_rpath("$ORIGIN")])
    return out


def build_dropin(force=False) -> Path | None:
    """nnops' front end + CPU route + this backend in one library.  None without the source tree."""
    if not (REFERENCE_ROOT / "src" / "ops" / "linear.cpp").exists():
        p = LIB_DIR / "libnnops_b200_dropin.so"
        return p if p.exists() else None
    lib = lib_build.build()
    out = LIB_DIR / "libnnops_b200_dropin.so"
    glue = [HOST / "cuda_backend.cpp", HOST / "quant_backend.cpp", HOST / "conv_backend.cpp", HOST / "not_implemented.cpp"]
    srcs = [REFERENCE_ROOT / "src" / s for s in REF_SOURCES]
    if not (force or _stale(out, [*glue, HOST / "staging.hpp", lib, ROOT / "include" / "nnb200.h", *srcs])):
        return out
    obj_dir = LIB_DIR / "obj_dropin"
    obj_dir.mkdir(exist_ok=True)
    # NNOPS_HAS_CUDA for every unit: nnops derives an inline constant from it, so a per-file
    # define would be an ODR hazard.  -include limits: two nnops headers miss <limits> (GCC 13).
    flags = ["-std=c++23", "-O3", "-fPIC", "-fopenmp", "-DNDEBUG", "-DNNOPS_HAS_CUDA=1", "-include", "limits",
             "-mavx2", "-mfma", "-mf16c", "-mavxvnni",
             f"-I{REFERENCE_ROOT / 'include'}", f"-I{REFERENCE_ROOT / 'src'}", f"-I{ROOT / 'include'}"]
    jobs, objs = [], []
    for s in srcs:
        o = obj_dir / (str(s.relative_to(REFERENCE_ROOT)).replace("/", "_") + ".o")
        objs.append(o)
        jobs.append([CXX, *flags, "-c", s, "-o", o])
    for g in glue:
        o = obj_dir / (g.stem + ".o")
        objs.append(o)
        jobs.append([CXX, *flags, "-DNNB200_USE_NNOPS_HEADERS=1", "-c", g, "-o", o])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        list(ex.map(_run, jobs))
    _run([CXX, "-shared", "-fopenmp", "-o", out, *objs, f"-L{LIB_DIR}", "-lnnb200", *_rpath("$ORIGIN")])
    for o in objs:
        o.unlink()
    obj_dir.rmdir()
    return out


def build_tests(force=False) -> list[Path]:
    from oracle import build as oracle_build
    oracle_lib = oracle_build.build_port()
    BIN_DIR.mkdir(parents=True, exist_ok=True)
    src = ROOT / "tests" / "cpp" / "test_ops.cpp"
    cuda = [f"-I{CUDA_HOME / 'include'}", f"-L{CUDA_HOME / 'lib64'}", "-lcudart"]
    outs = []
    host_lib = build_standalone(force)
    out = BIN_DIR / "test_ops_standalone"
    if force or _stale(out, [src, host_lib, oracle_lib]):
        _run([CXX, *COMMON, "-o", out, src, f"-L{LIB_DIR}", "-lnnb200_host", "-lnnb200", f"-L{oracle_lib.parent}",
              "-lnnops_oracle", *cuda, *_rpath(LIB_DIR, oracle_lib.parent, CUDA_HOME / "lib64")])
    outs.append(out)
    # The C++ sharded layer (header-only over the C ABI) and its forked-ranks test.
    shard_src = ROOT / "tests" / "cpp" / "test_sharded.cpp"
    out = BIN_DIR / "test_sharded"
    if force or _stale(out, [shard_src, ROOT / "include" / "nnops_b200" / "sharded_linear.hpp", lib_build.LIB]):
        _run([CXX, *COMMON, "-o", out, shard_src, f"-L{LIB_DIR}", "-lnnb200", *cuda, "-lrt", "-pthread",
              *_rpath(LIB_DIR, CUDA_HOME / "lib64")])
    outs.append(out)
    bench_src = ROOT / "tests" / "cpp" / "bench_linear_op.cpp"
    out = BIN_DIR / "bench_linear_op_standalone"
    if force or _stale(out, [bench_src, host_lib]):
        _run([CXX, *COMMON, "-o", out, bench_src, f"-L{LIB_DIR}", "-lnnb200_host", "-lnnb200", *cuda,
              *_rpath(LIB_DIR, CUDA_HOME / "lib64")])
    outs.append(out)
    dropin = build_dropin(force)
    if dropin is not None and (REFERENCE_ROOT / "include").exists():
        out = BIN_DIR / "test_ops_dropin"
        if force or _stale(out, [src, dropin, oracle_lib]):
            _run([CXX, "-std=c++23", "-O2", "-include", "limits", "-DNNB200_USE_NNOPS_HEADERS=1", "-DNNOPS_HAS_CUDA=1",
                  f"-I{REFERENCE_ROOT / 'include'}", f"-I{ROOT / 'include'}", "-o", out, src, f"-L{LIB_DIR}",
                  "-lnnops_b200_dropin", "-lnnb200", f"-L{oracle_lib.parent}", "-lnnops_oracle", "-fopenmp", *cuda,
                  *_rpath(LIB_DIR, oracle_lib.parent, CUDA_HOME / "lib64")])
        outs.append(out)
        out = BIN_DIR / "bench_linear_op_dropin"
        if force or _stale(out, [bench_src, dropin]):
            _run([CXX, "-std=c++23", "-O2", "-include", "limits", "-DNNB200_USE_NNOPS_HEADERS=1", "-DNNOPS_HAS_CUDA=1",
                  f"-I{REFERENCE_ROOT / 'include'}", f"-I{ROOT / 'include'}", "-o", out, bench_src, f"-L{LIB_DIR}",
                  "-lnnops_b200_dropin", "-lnnb200", "-fopenmp", *cuda, *_rpath(LIB_DIR, CUDA_HOME / "lib64")])
        outs.append(out)
    else:
        for name in ("test_ops_dropin", "bench_linear_op_dropin"):
            if (BIN_DIR / name).exists():
                outs.append(BIN_DIR / name)
    return outs


if __name__ == "__main__":
    for p in build_tests():
        print(p)
