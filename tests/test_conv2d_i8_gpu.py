"""Parity of the int8 Conv2D with the CPU oracle, through the C ABI.

Mirrors the reference's differential test (tests/test_cuda_conv2d.cpp:252-500, `cuda_conv2d_i8`):
the same shape table -- every (activation, destination) pair, the three zero-point isolations,
strides, dilation, groups down to one channel per group, planes of thousands of pixels, reductions
of thousands of taps -- the same seeded value ranges and quantisation parameters, the CPU route as
the expected value.  Integer outputs are compared byte for byte (so are the fp ones: the epilogue
is the matmul's, which is restated operation for operation).  Added here: pitched and offset
activation views, batches, the packed filter, the in-place 1x1 path and refused arguments.
"""
import numpy as np
import pytest
import torch

import oracle
from nnops_b200 import capi, ops

pytestmark = pytest.mark.gpu

S8, U8 = np.int8, np.uint8

# n, ic, ih, iw, oc, kh, kw, sh, sw, dh, dw, ph, pw, groups, act dtype, out kind, bias, relu, zp_x (None = default), symmetric w
CASES = [
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", False, False, 0, True),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", False, False, 128, True),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", False, False, 0, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, None, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", True, False, None, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "u8", True, True, None, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "u8", True, True, None, False),
    (1, 16, 8, 8, 8, 1, 1, 1, 1, 1, 1, 0, 0, 1, U8, "f32", True, True, None, False),
    (1, 16, 8, 8, 8, 1, 1, 1, 1, 1, 1, 0, 0, 1, S8, "f32", False, False, None, False),
    (1, 16, 8, 8, 8, 3, 3, 2, 1, 1, 1, 1, 1, 1, U8, "f16", True, True, None, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 2, 1, 1, 1, 1, S8, "f16", True, True, None, False),
    (1, 16, 8, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 2, U8, "s8", True, True, None, False),
    (1, 16, 16, 16, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, None, False),
    (1, 16, 12, 12, 16, 3, 3, 1, 1, 1, 1, 1, 1, 2, U8, "u8", True, True, None, False),
    (1, 64, 112, 112, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, None, False),
    (1, 32, 224, 224, 32, 1, 1, 1, 1, 1, 1, 0, 0, 1, S8, "f32", False, False, None, False),
    (1, 16, 8, 8, 16, 3, 3, 1, 1, 1, 1, 1, 1, 16, S8, "u8", True, True, None, False),
    (1, 128, 16, 16, 128, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", True, False, 0, True),
    (1, 32, 32, 32, 24, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", True, True, -6, False),
    (1, 32, 16, 16, 32, 3, 3, 1, 1, 1, 1, 1, 1, 2, S8, "s8", True, False, 0, False),
    (1, 64, 56, 56, 128, 1, 1, 1, 1, 1, 1, 0, 0, 1, S8, "s8", True, False, 0, True),
    (1, 256, 14, 14, 256, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", True, True, 0, False),
    (1, 128, 7, 7, 128, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "f32", False, False, 0, False),
    # Beyond the reference's table: batches, odd channel counts (byte-wise gather), rectangular
    # filters with unequal strides / dilations / paddings, a 7x7 stem over three channels.
    (3, 24, 15, 17, 40, 5, 3, 2, 3, 1, 2, 2, 1, 1, U8, "s8", True, True, None, False),
    (2, 3, 33, 31, 32, 7, 7, 2, 2, 1, 1, 3, 3, 1, U8, "s8", True, True, None, False),
    (4, 48, 9, 9, 21, 3, 3, 1, 1, 1, 1, 0, 0, 3, S8, "f16", True, False, None, False),
    (2, 64, 28, 28, 96, 1, 1, 2, 2, 1, 1, 0, 0, 1, U8, "u8", True, True, None, False),
    # Shapes the implicit-GEMM form takes (stride 1, whole 128-channel blocks per group, symmetric
    # weights): zero points against padding (the border correction), dilation, groups, a 1x1 with
    # padding, patches that overhang the image on both axes, every destination.
    (2, 128, 20, 20, 160, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, 128, True),
    (1, 256, 28, 28, 96, 3, 3, 1, 1, 2, 2, 2, 2, 1, S8, "u8", True, True, -6, True),
    (2, 256, 17, 13, 64, 5, 3, 1, 1, 1, 1, 2, 0, 2, U8, "f16", True, True, None, True),
    (1, 128, 30, 30, 40, 1, 1, 1, 1, 1, 1, 1, 1, 1, U8, "f32", True, False, 128, True),
    (3, 128, 9, 40, 256, 3, 3, 1, 1, 1, 1, 1, 1, 1, S8, "s8", True, True, 0, True),
    (1, 384, 56, 56, 128, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, 77, True),
    # Enough 256-wide tiles for the CTA-pair form: an odd number of patches (the last pair's second
    # half is past the batch), and a second column of tiles with a ragged edge.
    (17, 128, 24, 40, 256, 3, 3, 1, 1, 1, 1, 1, 1, 1, U8, "s8", True, True, 128, True),
    (5, 128, 56, 56, 320, 3, 3, 1, 1, 2, 2, 2, 2, 1, S8, "f16", True, True, -6, True),
    # Strides of 2 (the tensor map's element strides): a downsampling 3x3 over an odd plane, a
    # 1x1 projection, unequal strides, and one with enough tiles for CTA pairs.
    (2, 128, 57, 57, 160, 3, 3, 2, 2, 1, 1, 1, 1, 1, U8, "s8", True, True, 128, True),
    (1, 256, 56, 56, 64, 1, 1, 2, 2, 1, 1, 0, 0, 1, S8, "u8", True, True, -6, True),
    (2, 128, 40, 33, 96, 3, 3, 2, 1, 1, 1, 1, 1, 1, U8, "f16", True, True, None, True),
    (22, 128, 56, 56, 256, 3, 3, 2, 2, 1, 1, 1, 1, 1, U8, "s8", True, True, 128, True),
    (2, 128, 41, 45, 64, 3, 5, 2, 2, 2, 2, 2, 4, 1, U8, "s8", True, True, 77, True),     # stride 2 with dilation 2
    (3, 256, 31, 29, 48, 3, 3, 1, 2, 1, 1, 1, 1, 2, S8, "f32", True, False, -6, True),   # stride along w only, two groups
]
IMPLICIT = list(range(len(CASES) - 14, len(CASES)))


def _make(case, seed):
    n, ic, ih, iw, oc, kh, kw, sh, sw, dh, dw, ph, pw, g, adt, odt, bias, relu, zpx, sym = case
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, (n, ih, iw, ic), dtype=np.uint8).view(adt)
    w = rng.integers(-127, 128, (kh, kw, ic // g, oc), dtype=np.int8)
    # The reference test's parameters (tests/test_cuda_conv2d.cpp:327-350).
    s_w = (0.008 + 0.001 * (np.arange(oc) % 5)).astype(np.float32)
    z_w = np.zeros(oc, np.int32) if sym else ((np.arange(oc) % 7) - 3).astype(np.int32)
    zx = zpx if zpx is not None else (128 if adt == U8 else -6)
    int_out = odt in ("s8", "u8")
    b = None
    if bias:
        b = rng.integers(-1000, 1001, oc).astype(np.int32) if int_out else \
            rng.uniform(-0.5, 0.5, oc).astype(np.float32 if odt == "f32" else np.float16)
    kwargs = dict(stride=(sh, sw), dilation=(dh, dw), padding=(ph, pw), groups=g, out_kind=odt, bias=b, relu=relu,
                  scale_x=0.0078125, zp_x=zx, scale_w=s_w, zp_w=z_w, out_scale=0.03, out_zp=110 if odt == "u8" else 0)
    return x, w, kwargs


def _gpu(x_t, w_t, kwargs, **extra):
    kw = dict(kwargs)
    if kw["out_kind"] in ("f32", "f16") and kw["relu"]:
        kw["activation"] = "relu"
    out = ops.conv2d_i8(x_t, w_t, **kw, **extra)
    torch.cuda.synchronize()
    assert capi.take_device_error() == 0
    return out.cpu().numpy()


def _same(got, want):
    assert got.shape == want.shape
    if not np.array_equal(got.view(np.uint8), want.view(np.uint8)):
        bad = np.argwhere(got != want)
        raise AssertionError(f"{len(bad)} mismatches of {got.size}; first {bad[:5].tolist()} "
                             f"got {got[tuple(bad[0])]} want {want[tuple(bad[0])]}")


@pytest.mark.parametrize("idx", range(len(CASES)))
def test_conv2d_i8_matches_cpu_route(cuda_device, idx):
    x, w, kwargs = _make(CASES[idx], 100 + idx)
    want = oracle.conv2d_i8(x, w, impl="ref" if oracle.have_ref() else "port", **kwargs)
    got = _gpu(torch.from_numpy(x).to(cuda_device), torch.from_numpy(w).to(cuda_device), kwargs)
    _same(got, want)


@pytest.mark.parametrize("idx", IMPLICIT + [17])
def test_implicit_form_equals_gather_form(cuda_device, idx, knobs):
    """The implicit-GEMM form (4-D TMA boxes of the activation, zeros outside the image, the zero
    point's share added back for overhanging windows) against the gather pass + GEMM on the same
    bytes, and its workspace: no gathered copy."""
    import ctypes as C
    x, w, kwargs = _make(CASES[idx], 300 + idx)
    x_t, w_t = torch.from_numpy(x).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    lib = capi.lib()

    def scratch():
        n, ih, iw, ic = x.shape
        kh, kw, icg, oc = w.shape
        oh, ow = ops.conv2d_out_hw(ih, iw, kh, kw, kwargs["stride"], kwargs["dilation"], kwargs["padding"])
        a = capi.Conv2dI8Args(input=x_t.data_ptr(), weight=w_t.data_ptr(), out=x_t.data_ptr(), batch=n, ih=ih, iw=iw, ic=ic,
                              oh=oh, ow=ow, oc=oc, kh=kh, kw=kw, stride_h=kwargs["stride"][0], stride_w=kwargs["stride"][1],
                              dil_h=kwargs["dilation"][0],
                              dil_w=kwargs["dilation"][1], pad_h=kwargs["padding"][0], pad_w=kwargs["padding"][1],
                              groups=kwargs["groups"], in_stride_n=ih * iw * ic, in_stride_h=iw * ic, in_stride_w=ic,
                              in_stride_c=1, w_stride_kh=kw * icg * oc, w_stride_kw=icg * oc, w_stride_ic=oc, w_stride_oc=1,
                              out_stride_n=oh * ow * oc, out_stride_h=ow * oc, out_stride_w=oc, out_kind=1,
                              zp_x=kwargs["zp_x"])
        return lib.nnb200_conv2d_i8_workspace_bytes(C.byref(a)), n * oh * ow * kh * kw * icg * kwargs["groups"]

    knobs("conv_form", 2)         # the implicit form wherever it can run, whatever the plane size
    need, col = scratch()
    assert need < col             # no gathered copy in the plan
    implicit = _gpu(x_t, w_t, kwargs)
    knobs("i8_pair", 0)           # one CTA per tile where the default pairs them
    _same(_gpu(x_t, w_t, kwargs), implicit)
    knobs("i8_pair", -1)
    knobs("conv_form", 1)         # never
    need, col = scratch()
    assert need >= col
    _same(_gpu(x_t, w_t, kwargs), implicit)
    _same(implicit, oracle.conv2d_i8(x, w, **kwargs))


@pytest.mark.parametrize("idx", [3, 11, 16, 18, 21, 23, 24] + IMPLICIT[:3])
def test_packed_filter_is_bit_identical(cuda_device, idx):
    """The packed filter holds the bytes the per-call filter pass would write: same output
    (tests/test_cuda_conv2d.cpp:531-650, `cuda_conv2d_i8_packed_filter`)."""
    x, w, kwargs = _make(CASES[idx], 200 + idx)
    x_t, w_t = torch.from_numpy(x).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    raw = _gpu(x_t, w_t, kwargs)
    packed = ops.prepack_conv2d_i8(w_t, groups=kwargs["groups"])
    _same(_gpu(x_t, packed, kwargs), raw)
    _same(raw, oracle.conv2d_i8(x, w, **kwargs))


def test_strided_views_and_canaries(cuda_device):
    """Activation and output as windows of larger buffers (pitched pixels, channel offset); the
    filter as a transposed view.  Bytes outside the output window must survive."""
    case = (2, 32, 13, 11, 48, 3, 3, 1, 2, 1, 1, 1, 1, 2, U8, "s8", True, True, None, False)
    x, w, kwargs = _make(case, 7)
    want = oracle.conv2d_i8(x, w, **kwargs)
    n, ih, iw, ic = x.shape
    big = torch.full((n, ih, iw + 3, ic + 16), 77, dtype=torch.uint8, device=cuda_device)
    big[:, :, :iw, 16:] = torch.from_numpy(x).to(cuda_device)
    x_view = big[:, :, :iw, 16:]
    w_oihw = torch.from_numpy(np.ascontiguousarray(w.transpose(3, 2, 0, 1))).to(cuda_device)   # stored OIHW
    w_view = w_oihw.permute(2, 3, 1, 0)                                                        # viewed HWIO
    oh, ow, oc = want.shape[1:]
    out_big = torch.full((n, oh, ow, oc + 16), -99, dtype=torch.int8, device=cuda_device)
    out_view = out_big[:, :, :, :oc]
    got = _gpu(x_view, w_view, kwargs, out=out_view)
    _same(got, want)
    assert bool((out_big[:, :, :, oc:] == -99).all().item())


def test_pointwise_runs_in_place(cuda_device):
    """1x1 / stride 1 / unpadded over a dense activation: no gather, so the workspace holds only
    the filter pass and the GEMM's scratch."""
    import ctypes as C
    case = (2, 64, 20, 20, 128, 1, 1, 1, 1, 1, 1, 0, 0, 1, S8, "s8", True, True, 0, True)
    x, w, kwargs = _make(case, 9)
    x_t, w_t = torch.from_numpy(x).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    _same(_gpu(x_t, w_t, kwargs), oracle.conv2d_i8(x, w, **kwargs))
    lib = capi.lib()
    args = capi.Conv2dI8Args(input=x_t.data_ptr(), weight=w_t.data_ptr(), out=x_t.data_ptr(), batch=2, ih=20, iw=20,
                             ic=64, oh=20, ow=20, oc=128, kh=1, kw=1, stride_h=1, stride_w=1, dil_h=1, dil_w=1,
                             pad_h=0, pad_w=0, groups=1, in_stride_n=20 * 20 * 64, in_stride_h=20 * 64, in_stride_w=64,
                             in_stride_c=1, w_stride_kh=64 * 128, w_stride_kw=64 * 128, w_stride_ic=128, w_stride_oc=1,
                             out_stride_n=20 * 20 * 128, out_stride_h=20 * 128, out_stride_w=128, out_kind=1)
    in_place = lib.nnb200_conv2d_i8_workspace_bytes(C.byref(args))
    args.pad_h = args.pad_w = 1
    args.kh = args.kw = 3
    args.w_stride_kh, args.w_stride_kw = 3 * 64 * 128, 64 * 128
    gathered = lib.nnb200_conv2d_i8_workspace_bytes(C.byref(args))
    assert in_place < 2 * 20 * 20 * 64 and gathered >= 2 * 20 * 20 * 9 * 64


def test_refusals_launch_nothing(cuda_device):
    import ctypes as C
    lib = capi.lib()
    x = torch.zeros((1, 8, 8, 16), dtype=torch.int8, device=cuda_device)
    w = torch.zeros((3, 3, 16, 8), dtype=torch.int8, device=cuda_device)
    out = torch.zeros((1, 8, 8, 8), dtype=torch.int32, device=cuda_device)
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device=cuda_device)

    def args(**over):
        a = capi.Conv2dI8Args(input=x.data_ptr(), weight=w.data_ptr(), out=out.data_ptr(), batch=1, ih=8, iw=8, ic=16,
                              oh=8, ow=8, oc=8, kh=3, kw=3, stride_h=1, stride_w=1, dil_h=1, dil_w=1, pad_h=1, pad_w=1,
                              groups=1, in_stride_n=1024, in_stride_h=128, in_stride_w=16, in_stride_c=1,
                              w_stride_kh=384, w_stride_kw=128, w_stride_ic=8, w_stride_oc=1, out_stride_n=512,
                              out_stride_h=64, out_stride_w=8, out_kind=1, scale_x=1.0, scale_w_scalar=1.0,
                              out_scale=1.0, workspace=ws.data_ptr(), workspace_bytes=ws.numel())
        for k, v in over.items():
            setattr(a, k, v)
        return a

    before = lib.nnb200_launch_count()
    assert lib.nnb200_conv2d_i8(C.byref(args(out_kind=0)), None) == capi.UNSUPPORTED       # s32 destination
    assert lib.nnb200_conv2d_i8(C.byref(args(oh=16)), None) == capi.INVALID_ARGUMENT         # windows start far below the image
    assert lib.nnb200_conv2d_i8(C.byref(args(groups=3)), None) == capi.INVALID_ARGUMENT
    assert lib.nnb200_conv2d_i8(C.byref(args(out_stride_h=80)), None) == capi.UNSUPPORTED    # rows at two pitches
    assert lib.nnb200_conv2d_i8(C.byref(args(workspace_bytes=16)), None) == capi.INVALID_ARGUMENT
    assert lib.nnb200_conv2d_i8(C.byref(args(workspace=ws.data_ptr() + 4)), None) == capi.INVALID_ARGUMENT
    assert lib.nnb200_launch_count() == before
    assert lib.nnb200_conv2d_i8(C.byref(args()), None) == capi.OK
    torch.cuda.synchronize()
