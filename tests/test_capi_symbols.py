"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every symbol that
include/nnb200.h declares.  No compute call is made here."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_header_symbols_exported(nnb200_lib):
    header = (ROOT / "include" / "nnb200.h").read_text()
    declared = set(re.findall(r"\b(nnb200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    from nnops_b200 import capi
    bound = {name for name, _, _ in capi.SYMBOLS}
    assert declared == bound, f"header/binding drift: {declared ^ bound}"
    for name in declared:
        assert getattr(nnb200_lib, name) is not None


def test_struct_sizes_match_header(nnb200_lib):
    # The argument blocks are plain C structs; ctypes and nvcc must agree on their layout.
    from nnops_b200 import capi
    assert C.sizeof(capi.GemmI8Args) % 8 == 0
    assert C.sizeof(capi.Q41Args) % 8 == 0
    assert nnb200_lib.nnb200_version().startswith(b"nnb200")


def test_argument_validation_without_gpu(nnb200_lib):
    from nnops_b200 import capi
    args = capi.GemmI8Args()
    args.m, args.n, args.k, args.batch = 4, 4, -1, 1
    assert nnb200_lib.nnb200_gemm_i8(C.byref(args), None) == capi.INVALID_ARGUMENT
    args.k = 4
    args.out_kind = 9
    assert nnb200_lib.nnb200_gemm_i8(C.byref(args), None) == capi.INVALID_ARGUMENT
    # Empty output: nothing to do, ok (reference matmul.cu:108-110).
    args.out_kind = 0
    args.m = 0
    assert nnb200_lib.nnb200_gemm_i8(C.byref(args), None) == capi.OK
    q = capi.Q41Args()
    q.m, q.n, q.k = 1, 4, 64
    assert nnb200_lib.nnb200_linear_q4_1(C.byref(q), None) == capi.INVALID_ARGUMENT  # null pointers
