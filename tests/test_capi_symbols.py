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


def test_misaligned_pointers_are_refused_before_any_launch(nnb200_lib):
    """Arrays read as 4-byte words (bias, scales, zero points, row sums), f16 bias and the
    16-byte workspace: a misaligned pointer is INVALID_ARGUMENT, not a device fault."""
    from nnops_b200 import capi
    base = 0x7000_0000_1000            # never dereferenced: validation comes first

    def block():
        a = capi.GemmI8Args()
        a.a, a.w, a.out = base, base + 0x1000, base + 0x2000
        a.m, a.n, a.k, a.batch = 4, 4, 16, 1
        a.a_stride_m, a.a_stride_k, a.w_stride_n, a.w_stride_k, a.ldc = 16, 1, 16, 1, 4
        a.scale_a_scalar = a.scale_w_scalar = a.out_scale = 1.0
        return a

    before = nnb200_lib.nnb200_launch_count()
    for field, off in [("bias", 2), ("scale_a", 1), ("scale_w", 2), ("zp_a", 3), ("zp_w", 2), ("r_w", 1),
                       ("workspace", 8), ("out", 2)]:
        a = block()
        setattr(a, field, base + 0x3000 + off)
        assert nnb200_lib.nnb200_gemm_i8(C.byref(a), None) == capi.INVALID_ARGUMENT, field
        if field != "workspace":       # the allocation-free entry ignores the caller's workspace
            assert nnb200_lib.nnb200_gemm_i8_static_scratch(C.byref(a), None) == capi.INVALID_ARGUMENT, field
    a = block()
    a.out_kind = capi.OUT_KINDS["f16"]
    a.bias = base + 0x3001             # f16 bias: 2-byte alignment
    assert nnb200_lib.nnb200_gemm_i8(C.byref(a), None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_launch_count() == before


def test_knobs_round_trip(nnb200_lib):
    from nnops_b200 import capi
    assert nnb200_lib.nnb200_get_knob(capi.KNOBS["i8_bn"]) == -1
    assert capi.set_knob("i8_bn", 192) == -1
    assert nnb200_lib.nnb200_get_knob(capi.KNOBS["i8_bn"]) == 192
    assert capi.set_knob("i8_bn", -5) == 192
    assert nnb200_lib.nnb200_get_knob(capi.KNOBS["i8_bn"]) == -1
    assert nnb200_lib.nnb200_set_knob(99, 1) == -(2 ** 31)


def test_conv_arguments_are_checked_before_any_launch(nnb200_lib):
    """nnb200_conv2d_i8 without a GPU: geometry that is no convolution, null or misaligned pointers and a
    missing workspace are refused with a status, nothing is launched."""
    from nnops_b200 import capi
    base = 0x7000_0000_1000            # never dereferenced: validation comes first

    def block(**over):
        a = capi.Conv2dI8Args(input=base, weight=base + 0x10000, out=base + 0x20000, batch=1, ih=8, iw=8, ic=16, oh=8,
                              ow=8, oc=8, kh=3, kw=3, stride_h=1, stride_w=1, dil_h=1, dil_w=1, pad_h=1, pad_w=1,
                              groups=1, in_stride_n=1024, in_stride_h=128, in_stride_w=16, in_stride_c=1,
                              w_stride_kh=384, w_stride_kw=128, w_stride_ic=8, w_stride_oc=1, out_stride_n=512,
                              out_stride_h=64, out_stride_w=8, out_kind=1, scale_x=1.0, scale_w_scalar=1.0, out_scale=1.0)
        for k, v in over.items():
            setattr(a, k, v)
        return a

    before = nnb200_lib.nnb200_launch_count()
    assert nnb200_lib.nnb200_conv2d_i8_workspace_bytes(C.byref(block())) > 0
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block()), None) == capi.INVALID_ARGUMENT            # no workspace given
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(groups=3)), None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(input=None)), None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(out_kind=0)), None) == capi.UNSUPPORTED        # s32 destination
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(bias=base + 2)), None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(scale_w=base + 1)), None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_conv2d_i8(C.byref(block(batch=0)), None) == capi.OK                    # empty output
    assert nnb200_lib.nnb200_conv2d_i8_pack(None, 1, 1, 1, 1, 3, 3, 16, 8, 1, None, None) == capi.INVALID_ARGUMENT
    assert nnb200_lib.nnb200_conv2d_i8_pack_bytes(3, 3, 16, 8) >= 8 * 144 + 8 * 4
    assert nnb200_lib.nnb200_launch_count() == before
