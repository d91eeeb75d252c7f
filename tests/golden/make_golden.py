"""Generate the golden fixtures of this directory from the compiled reference CPU route.

    python tests/golden/make_golden.py [name-prefix]     (needs oracle/_ref, i.e. the nnops source tree at build time)

Each .npz holds seeded inputs, the reference's output and a JSON `meta` describing the call.
The reference is driven through its public operator API (Linear / MatMul / Conv2D on Backend::CPU, via
oracle/ref_shim.cpp).  tests/test_oracle.py checks the C restatement against these files, and
tests/test_golden_gpu.py checks the CUDA path against them, so parity with the reference stays
pinned on machines where the reference itself cannot be built.
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402
from nnops_b200 import synth  # noqa: E402

HERE = Path(__file__).resolve().parent
ONLY = ""   # optional name prefix given on the command line: regenerate only those fixtures


def save(name, meta, **arrays):
    if not name.startswith(ONLY):
        return
    np.savez_compressed(HERE / f"{name}.npz", meta=np.array(json.dumps(meta)), **arrays)
    print("wrote", name, {k: v.shape for k, v in arrays.items()})


def int8_case(name, m, n, k, out_kind, *, seed, relu=False, a_unsigned=False, per_token=False, per_channel=True,
              zero_points=False, out_scale=1.0, out_zp=0, a_transposed=False, w_kn=False):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8) if a_unsigned else rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    int_out = out_kind in ("s32", "s8", "u8")
    arrays, scalars, kw = {}, {}, []

    def put(key, value):
        kw.append(key)
        if np.isscalar(value):
            scalars[key] = value
        else:
            arrays[key] = value

    put("scale_a", rng.uniform(0.01, 0.03, m).astype(np.float32) if per_token else 0.02)
    put("scale_w", rng.uniform(0.001, 0.02, n).astype(np.float32) if per_channel else 0.01)
    if zero_points:
        put("zp_a", rng.integers(-9, 10, m).astype(np.int32) if per_token else (128 if a_unsigned else 3))
        put("zp_w", rng.integers(-9, 10, n).astype(np.int32) if per_channel else -2)
    put("bias", rng.integers(-1000, 1001, n).astype(np.int32) if int_out
        else (rng.normal(size=n) * 3).astype(np.float32 if out_kind == "f32" else np.float16))
    put("out_scale", float(out_scale))
    put("out_zp", int(out_zp))
    call = {key: (arrays[key] if key in arrays else scalars[key]) for key in kw}
    a_stored = np.ascontiguousarray(a.T) if a_transposed else a        # [K,M] storage for transpose_a
    w_stored = np.ascontiguousarray(w.T) if w_kn else w                # [K,N] storage without transpose_b
    a_view = a_stored.T if a_transposed else a_stored
    w_view = w_stored.T if w_kn else w_stored
    out = oracle.gemm_i8(a_view, w_view, out_kind=out_kind, relu=relu, impl="ref", **call)
    meta = dict(op="gemm_i8", out_kind=out_kind, relu=relu, kw=kw, scalars=scalars, a_transposed=a_transposed, w_kn=w_kn)
    save(name, meta, a=a_stored, w=w_stored, out=out, **arrays)


def q4_case(name, m, n, k, dtype, *, seed):
    rng = np.random.default_rng(seed)
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16 if dtype == "f16" else np.float32)
    out = oracle.q4_1_matmul(a, wb, k, out_dtype=dtype, impl="ref")
    # f16: the reference's own route carries f16 round trips of partial sums at large M; 1e-2.
    save(name, dict(op="q4_1", k=k, out_dtype=dtype, rtol=1e-2 if dtype == "f16" else 2e-3), a=a, w_blocks=wb, out=out)


def fp_act_case(name, m, n, k, fdt, *, seed, per_token, relu):
    """f32/f16 activations with quantization parameters x s8 weights (quantize on the fly)."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    a = (rng.standard_normal((m, k)) * 2).astype(fdt)
    scale_w = rng.uniform(0.001, 0.02, n).astype(np.float32)
    bias = (rng.normal(size=n) * 3).astype(fdt)
    scale_a = rng.uniform(0.01, 0.05, m).astype(np.float32) if per_token else np.float32(0.03)
    zp_a = rng.integers(-9, 10, m).astype(np.int32) if per_token else np.int32(3)
    out = oracle.linear_fp_act(a, w, scale_a=scale_a if per_token else float(scale_a),
                               zp_a=zp_a if per_token else int(zp_a), bias=bias, relu=relu, scale_w=scale_w, impl="ref")
    save(name, dict(op="fp_act", relu=relu, per_token=per_token), a=a, w=w, scale_a=np.atleast_1d(scale_a),
         zp_a=np.atleast_1d(zp_a), scale_w=scale_w, bias=bias, out=out)


def quant_case(name, shape, axis, per, fdt, qdt, *, seed):
    """QuantizeLinear and DequantizeLinear of one tensor.  x carries exact .5 ties (in units of
    its scale), infinities, a NaN and values far outside the 8-bit range."""
    rng = np.random.default_rng(seed)
    count = {"tensor": 1, "token": int(np.prod(shape[:-1])), "channel": shape[axis]}[per]
    scale = rng.uniform(0.05, 3.0, count).astype(np.float32)
    zdt = np.uint8 if qdt == "u8" else np.int8
    zp = (rng.integers(0, 256, count) if qdt == "u8" else rng.integers(-128, 128, count)).astype(zdt)
    x = (rng.standard_normal(shape) * 60).astype(fdt)
    flat = x.reshape(-1)
    flat[::5] = ((rng.integers(-90, 90, flat[::5].size) + 0.5) * scale[0]).astype(fdt)
    flat[:3] = [np.inf, -np.inf, np.nan]
    if fdt == np.float32:
        flat[3:5] = [3e9, -3e9]
    q = oracle.quantize_linear(x, scale, zp, axis=axis, out_dtype=zdt, impl="ref")
    xq = (rng.integers(0, 256, shape) if qdt == "u8" else rng.integers(-128, 128, shape)).astype(zdt)
    dq = oracle.dequantize_linear(xq, scale, zp, axis=axis, out_dtype=fdt, impl="ref")
    save(name, dict(op="quant_linear", axis=axis), x=x, scale=scale, zero_point=zp, quantized=q, xq=xq,
         dequantized=dq)


def conv_case(name, shape, filt, out_kind, *, seed, stride=(1, 1), dilation=(1, 1), padding=(0, 0), groups=1,
              a_unsigned=True, relu=True, zp_x=None):
    """int8 Conv2D through the reference's Conv2D on Backend::CPU: NHWC activation, HWIO filter, per-channel
    filter scales and zero points, the parameters of the reference's own CUDA-vs-CPU test."""
    rng = np.random.default_rng(seed)
    n, ih, iw, ic = shape
    kh, kw, oc = filt
    x = rng.integers(0, 256, shape, dtype=np.uint8).view(np.uint8 if a_unsigned else np.int8)
    w = rng.integers(-127, 128, (kh, kw, ic // groups, oc), dtype=np.int8)
    scale_w = (0.008 + 0.001 * (np.arange(oc) % 5)).astype(np.float32)
    zp_w = ((np.arange(oc) % 7) - 3).astype(np.int32)
    int_out = out_kind in ("s8", "u8")
    bias = rng.integers(-1000, 1001, oc).astype(np.int32) if int_out else \
        rng.uniform(-0.5, 0.5, oc).astype(np.float32 if out_kind == "f32" else np.float16)
    scalars = dict(scale_x=0.0078125, zp_x=int(zp_x if zp_x is not None else (128 if a_unsigned else -6)),
                   out_scale=0.03, out_zp=110 if out_kind == "u8" else 0)
    geom = dict(stride=list(stride), dilation=list(dilation), padding=list(padding), groups=groups)
    out = oracle.conv2d_i8(x, w, out_kind=out_kind, bias=bias, relu=relu, scale_w=scale_w, zp_w=zp_w, impl="ref",
                           stride=stride, dilation=dilation, padding=padding, groups=groups, **scalars)
    save(name, dict(op="conv2d_i8", out_kind=out_kind, relu=relu, scalars=scalars, geom=geom), x=x, w=w, bias=bias,
         scale_w=scale_w, zp_w=zp_w, out=out)


if __name__ == "__main__":
    if not oracle.have_ref():
        raise SystemExit("the compiled reference (oracle/_ref) is not available on this machine")
    ONLY = sys.argv[1] if len(sys.argv) > 1 else ""
    int8_case("i8_s32_bias", 128, 192, 256, "s32", seed=1, per_channel=False)
    int8_case("i8_s8_relu_per_channel", 160, 272, 512, "s8", seed=2, relu=True, out_scale=1.6)
    int8_case("i8_s8_saturating", 64, 128, 1024, "s8", seed=3, relu=True, out_scale=0.05)
    int8_case("i8_u8_per_token_zero_points", 77, 130, 272, "u8", seed=4, per_token=True, zero_points=True,
              out_scale=2.3, out_zp=7)
    int8_case("i8_u8_activations_s32", 50, 96, 160, "s32", seed=5, a_unsigned=True, zero_points=True, per_token=True)
    int8_case("i8_f32_dequant", 96, 144, 320, "f32", seed=6, per_token=True, relu=True)
    int8_case("i8_f16_dequant_zero_points", 40, 100, 256, "f16", seed=7, per_token=True, zero_points=True)
    int8_case("i8_transposed_poses", 70, 90, 200, "s8", seed=8, out_scale=40.0, per_channel=False, a_transposed=True,
              w_kn=True)
    int8_case("i8_decode_m4", 4, 520, 1024, "s8", seed=9, relu=True, out_scale=1.1)
    q4_case("q4_1_gemv_m1_f32", 1, 256, 4096, "f32", seed=10)
    q4_case("q4_1_gemv_m8_f32", 8, 203, 1000, "f32", seed=11)
    q4_case("q4_1_small_m_f16", 4, 128, 1024, "f16", seed=12)
    q4_case("q4_1_gemm_f32", 96, 160, 512, "f32", seed=13)
    q4_case("q4_1_gemm_f16", 160, 192, 512, "f16", seed=14)
    quant_case("qdq_per_tensor_f32_s8", (7, 1003), -1, "tensor", np.float32, "s8", seed=20)
    quant_case("qdq_per_token_f16_u8", (37, 75), -1, "token", np.float16, "u8", seed=21)
    quant_case("qdq_per_channel_f32_u8", (5, 12, 24), 1, "channel", np.float32, "u8", seed=22)
    quant_case("qdq_per_channel_last_axis_f16_s8", (6, 50), 1, "channel", np.float16, "s8", seed=23)
    fp_act_case("fp_act_f32_per_token", 96, 144, 320, np.float32, seed=30, per_token=True, relu=True)
    fp_act_case("fp_act_f16_per_tensor", 40, 100, 256, np.float16, seed=31, per_token=False, relu=False)
    conv_case("conv_i8_3x3_u8_s8", (2, 14, 14, 32), (3, 3, 48), "s8", seed=40, padding=(1, 1))
    conv_case("conv_i8_3x3_groups_stride_u8_u8", (1, 17, 15, 24), (3, 3, 36), "u8", seed=41, padding=(1, 1), stride=(2, 1),
              groups=3)
    conv_case("conv_i8_1x1_s8_f32", (2, 12, 12, 64), (1, 1, 40), "f32", seed=42, a_unsigned=False, relu=False)
    conv_case("conv_i8_5x3_dilated_s8_f16", (1, 16, 18, 16), (5, 3, 24), "f16", seed=43, a_unsigned=False,
              dilation=(1, 2), padding=(2, 2))
    conv_case("conv_i8_7x7_stem_u8_s8", (1, 35, 33, 3), (7, 7, 16), "s8", seed=44, stride=(2, 2), padding=(3, 3))
