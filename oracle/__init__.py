"""CPU checkers for the quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Two implementations behind one numpy interface:

* ``impl="port"``  -- the plain-C restatement in ``nnops_oracle.c`` (always available);
* ``impl="ref"``   -- the unmodified reference CPU route compiled into ``oracle/_ref`` (available
  when it was prebuilt and the host CPU has the VNNI flavour it needs).

Only tests, ``__graft_entry__.smoke()`` and the bench's CPU-baseline legs may import this
package; the shipped CUDA path never does.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

from . import build as _build

HERE = Path(__file__).resolve().parent
OUT_KINDS = {"s32": 0, "s8": 1, "u8": 2, "f32": 3, "f16": 4}
_OUT_NP = {"s32": np.int32, "s8": np.int8, "u8": np.uint8, "f32": np.float32, "f16": np.float16}
Q4_1_BLOCK_BYTES = 20
Q4_1_BLOCK_ELEMS = 32


class GemmI8Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a_stride_m", C.c_int64), ("a_stride_k", C.c_int64),
        ("w_stride_n", C.c_int64), ("w_stride_k", C.c_int64), ("ldc", C.c_int64),
        ("a_unsigned", C.c_int32), ("out_kind", C.c_int32),
        ("bias", C.c_void_p), ("relu", C.c_int32),
        ("scale_a", C.c_void_p), ("scale_w", C.c_void_p), ("zp_a", C.c_void_p), ("zp_w", C.c_void_p),
        ("scale_a_scalar", C.c_float), ("scale_w_scalar", C.c_float),
        ("zp_a_scalar", C.c_int32), ("zp_w_scalar", C.c_int32),
        ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("min_clip", C.c_float), ("max_clip", C.c_float),
    ]


_port = None
_ref = None
_ref_tried = False


def _cpu_flags() -> set[str]:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def port_lib() -> C.CDLL:
    global _port
    if _port is None:
        _port = C.CDLL(str(_build.build_port()))
        _port.oracle_f16_to_f32.restype = C.c_float
        _port.oracle_f16_to_f32.argtypes = [C.c_uint16]
        _port.oracle_f32_to_f16.restype = C.c_uint16
        _port.oracle_f32_to_f16.argtypes = [C.c_float]
    return _port


def ref_lib() -> C.CDLL | None:
    """The compiled reference route, or None when it is not prebuilt / not runnable here."""
    global _ref, _ref_tried
    if _ref_tried:
        return _ref
    _ref_tried = True
    flags = _cpu_flags()
    need = {"avx2", "fma", "f16c"}
    if not need <= flags:
        return None
    order = []
    if "avx_vnni" in flags:
        order.append("avxvnni")
    if {"avx512_vnni", "avx512vl", "avx512bw", "avx512f"} <= flags:
        order.append("avx512vnni")
    for name in order:
        p = HERE / "_ref" / f"libnnops_ref_{name}.so"
        if p.exists():
            try:
                _ref = C.CDLL(str(p))
                _ref.ref_isa = name
                return _ref
            except OSError:
                continue
    return None


def have_ref() -> bool:
    return ref_lib() is not None


def ref_threads() -> int:
    return int(os.environ.get("NNOPS_ORACLE_THREADS", os.cpu_count() or 1))


def _ptr(x) -> int | None:
    return None if x is None else x.ctypes.data


def gemm_i8(a: np.ndarray, w: np.ndarray, *, out_kind: str = "s32", bias: np.ndarray | None = None,
            relu: bool = False, scale_a=1.0, scale_w=1.0, zp_a=0, zp_w=0, out_scale: float = 1.0,
            out_zp: int = 0, min_clip: float = -np.inf, max_clip: float = np.inf,
            impl: str = "port", threads: int | None = None, use_linear: bool = True) -> np.ndarray:
    """int8 matmul + fused epilogue.  ``a`` is [M,K] s8/u8 (any 2-D strides: a transposed
    numpy view expresses MatMul's transpose_a); ``w`` is given as the LOGICAL [N,K] matrix
    (pass ``w_kn.T`` for a weight stored [K,N]).  scale_*/zp_* are scalars or 1-D arrays
    (per-token for A, per-channel for W)."""
    assert a.ndim == 2 and w.ndim == 2 and a.shape[1] == w.shape[1]
    assert a.dtype in (np.int8, np.uint8) and w.dtype == np.int8
    m, k = a.shape
    n = w.shape[0]
    out = np.zeros((m, n), dtype=_OUT_NP[out_kind])
    keep = []

    def arr(v, dt):
        if np.isscalar(v):
            return None, dt(v)
        v = np.ascontiguousarray(v, dtype=dt)
        keep.append(v)
        return v, dt(1 if dt is np.float32 else 0)

    sa, sa0 = arr(scale_a, np.float32)
    sw, sw0 = arr(scale_w, np.float32)
    za, za0 = arr(zp_a, np.int32)
    zw, zw0 = arr(zp_w, np.int32)
    if bias is not None:
        bdt = np.int32 if out_kind in ("s32", "s8", "u8") else _OUT_NP[out_kind]
        bias = np.ascontiguousarray(bias, dtype=bdt)
    args = GemmI8Args(
        a=a.ctypes.data, w=w.ctypes.data, out=out.ctypes.data, m=m, n=n, k=k,
        a_stride_m=a.strides[0], a_stride_k=a.strides[1] if k > 1 or a.strides[1] == 1 else 1,
        w_stride_n=w.strides[0], w_stride_k=w.strides[1] if k > 1 or w.strides[1] == 1 else 1, ldc=n,
        a_unsigned=int(a.dtype == np.uint8), out_kind=OUT_KINDS[out_kind], bias=_ptr(bias), relu=int(relu),
        scale_a=_ptr(sa), scale_w=_ptr(sw), zp_a=_ptr(za), zp_w=_ptr(zw),
        scale_a_scalar=float(sa0), scale_w_scalar=float(sw0), zp_a_scalar=int(za0), zp_w_scalar=int(zw0),
        out_scale=float(out_scale), out_zp=int(out_zp), min_clip=float(min_clip), max_clip=float(max_clip))
    if impl == "port":
        port_lib().oracle_gemm_i8(C.byref(args))
    else:
        lib = ref_lib()
        if lib is None:
            raise RuntimeError("reference route not available on this host")
        linear = use_linear and a.strides[1] == 1 and w.strides[1] == 1
        st = lib.ref_gemm_i8(C.byref(args), int(linear), int(threads or ref_threads()))
        if st != 0:
            raise RuntimeError(f"reference op returned Status {st}")
    return out


def q4_1_decode(blocks: np.ndarray, count: int, impl: str = "port") -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.zeros(count, dtype=np.float32)
    if impl == "port":
        port_lib().oracle_q4_1_decode_row(C.c_void_p(blocks.ctypes.data), C.c_int64(count),
                                          C.c_void_p(out.ctypes.data))
    else:
        ref_lib().ref_q4_1_decode(C.c_void_p(blocks.ctypes.data), C.c_int64(count), C.c_void_p(out.ctypes.data))
    return out


def q4_1_quantize(src: np.ndarray, impl: str = "port") -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.float32).ravel()
    nblk = (src.size + Q4_1_BLOCK_ELEMS - 1) // Q4_1_BLOCK_ELEMS
    blocks = np.zeros(nblk * Q4_1_BLOCK_BYTES, dtype=np.uint8)
    if impl == "port":
        port_lib().oracle_q4_1_quantize_row(C.c_void_p(src.ctypes.data), C.c_int64(src.size),
                                            C.c_void_p(blocks.ctypes.data))
    else:
        ref_lib().ref_q4_1_quantize(C.c_void_p(src.ctypes.data), C.c_int64(src.size), C.c_void_p(blocks.ctypes.data))
    return blocks


def q4_1_matmul(a: np.ndarray, w_blocks: np.ndarray, k: int, *, out_dtype: str = "f32",
                w_round_f16: bool = False, bias: np.ndarray | None = None, impl: str = "port",
                threads: int | None = None) -> np.ndarray:
    """``a`` [M,K] f16/f32 (C-contiguous), ``w_blocks`` uint8 [N, ceil(K/32)*20].
    port: f64 accumulation, out_dtype free.  ref: the reference Linear op, whose output dtype
    equals the activation dtype (f16 activations x f32 output is not a reference pose)."""
    assert a.ndim == 2 and w_blocks.ndim == 2 and w_blocks.dtype == np.uint8
    a = np.ascontiguousarray(a)
    w_blocks = np.ascontiguousarray(w_blocks)
    m = a.shape[0]
    n = w_blocks.shape[0]
    assert a.shape[1] == k and w_blocks.shape[1] == ((k + 31) // 32) * 20
    a_f16 = a.dtype == np.float16
    out = np.zeros((m, n), dtype=_OUT_NP[out_dtype])
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=_OUT_NP[out_dtype])
    if impl == "port":
        port_lib().oracle_q4_1_matmul(
            C.c_void_p(a.ctypes.data), C.c_int(a_f16), C.c_int64(k),
            C.c_void_p(w_blocks.ctypes.data), C.c_int64(w_blocks.shape[1] // 20),
            C.c_void_p(out.ctypes.data), C.c_int(out_dtype == "f16"), C.c_int64(n),
            C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_int(w_round_f16), C.c_void_p(_ptr(bias)))
    else:
        lib = ref_lib()
        if lib is None:
            raise RuntimeError("reference route not available on this host")
        assert (out_dtype == "f16") == a_f16, "reference pose: output dtype == activation dtype"
        st = lib.ref_linear_q4_1(
            C.c_void_p(a.ctypes.data), C.c_int(a_f16), C.c_int64(m), C.c_int64(k), C.c_int64(a.strides[0]),
            C.c_void_p(w_blocks.ctypes.data), C.c_int64(n), C.c_int64(w_blocks.strides[0]),
            C.c_void_p(_ptr(bias)), C.c_void_p(out.ctypes.data), C.c_int64(out.strides[0]),
            C.c_int(int(threads or ref_threads())))
        if st != 0:
            raise RuntimeError(f"reference op returned Status {st}")
    return out


def quant_decompose(shape, axis: int, param_count: int) -> tuple[int, int, int]:
    """[outer][rows][inner] view of a dense tensor for QuantizeLinear / DequantizeLinear:
    one parameter -> per tensor; axis < 0 -> one per innermost row; else one per index of axis
    (reference resolve_quant_granularity, include/nnops/ops/quant_linear.hpp:38-45)."""
    shape = tuple(int(s) for s in shape)
    numel = int(np.prod(shape)) if shape else 1
    if param_count <= 1:
        return 1, 1, numel
    if axis < 0:
        return 1, numel // shape[-1], shape[-1]
    outer = int(np.prod(shape[:axis])) if axis > 0 else 1
    inner = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
    return outer, shape[axis], inner


def quantize_linear(x: np.ndarray, scale, zero_point, *, axis: int = -1, out_dtype=np.int8, impl: str = "port",
                    threads: int | None = None, tail_fused: bool = True) -> np.ndarray:
    """y = saturate(round_half_even(x / scale + zero_point)) with the reference's arithmetic.
    ``scale`` f32 and ``zero_point`` s8/u8 arrays of equal length (1 = per tensor)."""
    x = np.ascontiguousarray(x)
    assert x.dtype in (np.float32, np.float16)
    scale = np.ascontiguousarray(np.atleast_1d(scale), dtype=np.float32)
    zero_point = np.ascontiguousarray(np.atleast_1d(zero_point))
    assert zero_point.dtype in (np.int8, np.uint8) and zero_point.size == scale.size
    y = np.zeros(x.shape, dtype=out_dtype)
    if x.size == 0:
        return y
    if impl == "port":
        outer, rows, inner = quant_decompose(x.shape, axis, scale.size)
        assert rows == scale.size
        port_lib().oracle_quantize_linear(
            C.c_void_p(x.ctypes.data), C.c_int(x.dtype == np.float16), C.c_int64(outer), C.c_int64(rows),
            C.c_int64(inner), C.c_void_p(scale.ctypes.data), C.c_void_p(zero_point.ctypes.data),
            C.c_int(zero_point.dtype == np.uint8), C.c_void_p(y.ctypes.data), C.c_int(y.dtype == np.uint8),
            C.c_int(int(tail_fused)))
    else:
        shape = (C.c_int64 * x.ndim)(*x.shape)
        st = ref_lib().ref_quantize_linear(
            C.c_void_p(x.ctypes.data), C.c_int(x.dtype == np.float16), shape, C.c_int(x.ndim), C.c_int64(axis),
            C.c_void_p(scale.ctypes.data), C.c_void_p(zero_point.ctypes.data), C.c_int(zero_point.dtype == np.uint8),
            C.c_int64(scale.size), C.c_void_p(y.ctypes.data), C.c_int(y.dtype == np.uint8),
            C.c_int(int(threads or ref_threads())))
        if st != 0:
            raise RuntimeError(f"reference op returned Status {st}")
    return y


def dequantize_linear(x: np.ndarray, scale, zero_point, *, axis: int = -1, out_dtype=np.float32, impl: str = "port",
                      threads: int | None = None) -> np.ndarray:
    """y = (x - zero_point) * scale with the reference's arithmetic (see nnops_oracle.c)."""
    x = np.ascontiguousarray(x)
    assert x.dtype in (np.int8, np.uint8)
    scale = np.ascontiguousarray(np.atleast_1d(scale), dtype=np.float32)
    zero_point = np.ascontiguousarray(np.atleast_1d(zero_point))
    assert zero_point.dtype in (np.int8, np.uint8) and zero_point.size == scale.size
    y = np.zeros(x.shape, dtype=out_dtype)
    if x.size == 0:
        return y
    if impl == "port":
        outer, rows, inner = quant_decompose(x.shape, axis, scale.size)
        assert rows == scale.size
        port_lib().oracle_dequantize_linear(
            C.c_void_p(x.ctypes.data), C.c_int(x.dtype == np.uint8), C.c_int64(outer), C.c_int64(rows),
            C.c_int64(inner), C.c_void_p(scale.ctypes.data), C.c_void_p(zero_point.ctypes.data),
            C.c_int(zero_point.dtype == np.uint8), C.c_void_p(y.ctypes.data), C.c_int(y.dtype == np.float16))
    else:
        shape = (C.c_int64 * x.ndim)(*x.shape)
        st = ref_lib().ref_dequantize_linear(
            C.c_void_p(x.ctypes.data), C.c_int(x.dtype == np.uint8), shape, C.c_int(x.ndim), C.c_int64(axis),
            C.c_void_p(scale.ctypes.data), C.c_void_p(zero_point.ctypes.data), C.c_int(zero_point.dtype == np.uint8),
            C.c_int64(scale.size), C.c_void_p(y.ctypes.data), C.c_int(y.dtype == np.float16),
            C.c_int(int(threads or ref_threads())))
        if st != 0:
            raise RuntimeError(f"reference op returned Status {st}")
    return y


def linear_fp_act(a: np.ndarray, w: np.ndarray, *, scale_a, zp_a=0, act_dtype=np.int8, bias: np.ndarray | None = None,
                  relu: bool = False, scale_w=1.0, zp_w=0, min_clip: float = -np.inf, max_clip: float = np.inf,
                  impl: str = "port", threads: int | None = None) -> np.ndarray:
    """f32/f16 activations carrying quantization parameters x s8 weights [N,K] -> a's dtype:
    quantise A on the fly (QuantizeLinear arithmetic with A's per-tensor / per-token scale and
    int32 zero point), int8 matmul, dequantizing epilogue
    (reference src/backend/cpu/matmul/matmul_i8.cpp:389-464)."""
    assert a.ndim == 2 and a.dtype in (np.float32, np.float16) and w.dtype == np.int8
    a = np.ascontiguousarray(a)
    m, k = a.shape
    out_kind = "f32" if a.dtype == np.float32 else "f16"
    if impl == "port":
        per_token = not (np.isscalar(scale_a) and np.isscalar(zp_a))
        count = m if per_token else 1
        s = np.ascontiguousarray(np.broadcast_to(np.asarray(scale_a, dtype=np.float32), (count,)))
        z = np.ascontiguousarray(np.broadcast_to(np.asarray(zp_a, dtype=np.int32), (count,)))
        aq = np.zeros((m, k), dtype=act_dtype)
        outer, rows, inner = (1, m, k) if per_token else (1, 1, m * k)
        port_lib().oracle_quantize_linear(
            C.c_void_p(a.ctypes.data), C.c_int(a.dtype == np.float16), C.c_int64(outer), C.c_int64(rows),
            C.c_int64(inner), C.c_void_p(s.ctypes.data), C.c_void_p(z.ctypes.data), C.c_int(2),
            C.c_void_p(aq.ctypes.data), C.c_int(aq.dtype == np.uint8), C.c_int(1))
        return gemm_i8(aq, w, out_kind=out_kind, bias=bias, relu=relu, scale_a=scale_a, scale_w=scale_w, zp_a=zp_a,
                       zp_w=zp_w, min_clip=min_clip, max_clip=max_clip)
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("reference route not available on this host")
    assert act_dtype == np.int8, "the reference Linear quantises activations to s8"
    n = w.shape[0]
    out = np.zeros((m, n), dtype=_OUT_NP[out_kind])
    keep = []

    def arr(v, dt):
        if np.isscalar(v):
            return None, dt(v)
        v = np.ascontiguousarray(v, dtype=dt)
        keep.append(v)
        return v, dt(1 if dt is np.float32 else 0)

    sa, sa0 = arr(scale_a, np.float32)
    sw, sw0 = arr(scale_w, np.float32)
    za, za0 = arr(zp_a, np.int32)
    zw, zw0 = arr(zp_w, np.int32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=_OUT_NP[out_kind])
    args = GemmI8Args(
        a=a.ctypes.data, w=w.ctypes.data, out=out.ctypes.data, m=m, n=n, k=k, a_stride_m=k, a_stride_k=1,
        w_stride_n=w.strides[0], w_stride_k=1, ldc=n, a_unsigned=2 if a.dtype == np.float32 else 3,
        out_kind=OUT_KINDS[out_kind], bias=_ptr(bias), relu=int(relu), scale_a=_ptr(sa), scale_w=_ptr(sw),
        zp_a=_ptr(za), zp_w=_ptr(zw), scale_a_scalar=float(sa0), scale_w_scalar=float(sw0), zp_a_scalar=int(za0),
        zp_w_scalar=int(zw0), out_scale=1.0, out_zp=0, min_clip=float(min_clip), max_clip=float(max_clip))
    st = lib.ref_gemm_i8(C.byref(args), 1, int(threads or ref_threads()))
    if st != 0:
        raise RuntimeError(f"reference op returned Status {st}")
    return out


def conv2d_out_hw(ih: int, iw: int, kh: int, kw: int, stride=(1, 1), dilation=(1, 1), padding=(0, 0)) -> tuple[int, int]:
    oh = (ih + 2 * padding[0] - ((kh - 1) * dilation[0] + 1)) // stride[0] + 1
    ow = (iw + 2 * padding[1] - ((kw - 1) * dilation[1] + 1)) // stride[1] + 1
    return oh, ow


def conv2d_i8(x: np.ndarray, w: np.ndarray, *, stride=(1, 1), dilation=(1, 1), padding=(0, 0), groups: int = 1,
              out_kind: str = "s8", bias: np.ndarray | None = None, relu: bool = False, scale_x: float = 1.0,
              zp_x: int = 0, scale_w=1.0, zp_w=0, out_scale: float = 1.0, out_zp: int = 0,
              min_clip: float = -np.inf, max_clip: float = np.inf, impl: str = "port",
              threads: int | None = None) -> np.ndarray:
    """int8 Conv2D: ``x`` [N, IH, IW, IC] u8/s8 (NHWC), ``w`` [KH, KW, IC/G, OC] s8 (HWIO) -> [N, OH, OW, OC].

    ``impl="port"`` restates the reference's definition (src/backend/cuda/conv/conv2d_i8.cu:89-141 gather,
    src/backend/cpu/conv/conv2d_implicit_gemm_i8.cpp:906-980 epilogue): gather the taps of every output
    pixel, k = (kh, kw, c) tap-major, a tap outside the image holding the activation's zero point, then the
    int8 matmul epilogue per group with K = KH*KW*IC/G.  ``impl="ref"`` runs the reference's Conv2D CPU route."""
    assert x.ndim == 4 and w.ndim == 4 and x.dtype in (np.int8, np.uint8) and w.dtype == np.int8
    n, ih, iw, ic = x.shape
    kh, kw, icg, oc = w.shape
    assert ic == icg * groups and oc % groups == 0 and out_kind != "s32"
    oh, ow = conv2d_out_hw(ih, iw, kh, kw, stride, dilation, padding)
    ocg = oc // groups
    if impl == "ref":
        lib = ref_lib()
        if lib is None:
            raise RuntimeError("reference route not available on this host")
        xc = np.ascontiguousarray(x)
        wc = np.ascontiguousarray(w)
        out = np.zeros((n, oh, ow, oc), dtype=_OUT_NP[out_kind])
        sw = None if np.isscalar(scale_w) else np.ascontiguousarray(scale_w, dtype=np.float32)
        zw = None if np.isscalar(zp_w) else np.ascontiguousarray(zp_w, dtype=np.int32)
        if bias is not None:
            bias = np.ascontiguousarray(bias, dtype=np.int32 if out_kind in ("s8", "u8") else _OUT_NP[out_kind])
        geom = (C.c_int64 * 16)(n, ih, iw, ic, oc, kh, kw, stride[0], stride[1], dilation[0], dilation[1],
                                padding[0], padding[1], groups, oh, ow)
        lib.ref_conv2d_i8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                      C.POINTER(C.c_int64), C.c_float, C.c_int32, C.c_void_p, C.c_void_p, C.c_float,
                                      C.c_int32, C.c_float, C.c_int32, C.c_int, C.c_float, C.c_float, C.c_int]
        lib.ref_conv2d_i8.restype = C.c_int
        st = lib.ref_conv2d_i8(xc.ctypes.data, int(x.dtype == np.uint8), wc.ctypes.data, _ptr(bias), out.ctypes.data,
                               OUT_KINDS[out_kind], geom, float(scale_x), int(zp_x), _ptr(sw), _ptr(zw),
                               float(scale_w if sw is None else 1.0), int(zp_w if zw is None else 0),
                               float(out_scale), int(out_zp), int(relu), float(min_clip), float(max_clip),
                               int(threads or ref_threads()))
        if st != 0:
            raise RuntimeError(f"reference op returned Status {st}")
        return out

    # Gather: padded copy filled with the zero point, then one strided slice per tap.
    ph, pw = padding
    xp = np.full((n, ih + 2 * ph, iw + 2 * pw, ic), zp_x, dtype=x.dtype)
    xp[:, ph:ph + ih, pw:pw + iw, :] = x
    out = np.zeros((n, oh, ow, oc), dtype=_OUT_NP[out_kind])
    per_channel = lambda v, g: v if np.isscalar(v) else np.asarray(v)[g * ocg:(g + 1) * ocg]
    for g in range(groups):
        cols = np.empty((n, oh, ow, kh * kw, icg), dtype=x.dtype)
        for a in range(kh):
            for b in range(kw):
                h0, w0 = a * dilation[0], b * dilation[1]
                cols[:, :, :, a * kw + b, :] = xp[:, h0:h0 + (oh - 1) * stride[0] + 1:stride[0],
                                                  w0:w0 + (ow - 1) * stride[1] + 1:stride[1], g * icg:(g + 1) * icg]
        a_mat = cols.reshape(n * oh * ow, kh * kw * icg)
        w_mat = np.ascontiguousarray(w[:, :, :, g * ocg:(g + 1) * ocg].reshape(kh * kw * icg, ocg).T)
        res = gemm_i8(a_mat, w_mat, out_kind=out_kind, bias=None if bias is None else np.asarray(bias)[g * ocg:(g + 1) * ocg],
                      relu=relu, scale_a=float(scale_x), scale_w=per_channel(scale_w, g), zp_a=int(zp_x),
                      zp_w=per_channel(zp_w, g), out_scale=out_scale, out_zp=out_zp, min_clip=min_clip,
                      max_clip=max_clip, impl="port")
        out[..., g * ocg:(g + 1) * ocg] = res.reshape(n, oh, ow, ocg)
    return out
