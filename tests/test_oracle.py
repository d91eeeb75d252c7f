"""CPU tests of the checkers: the plain-C restatement against the hand-computed vectors of the
reference's own tests (tests/test_matmul_int8.cpp:106-285, tests/test_q4_1.cpp), against the
committed golden fixtures produced by the compiled reference, and -- where the compiled
reference can run on this host -- against it directly."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
IMPLS = ["port"] + (["ref"] if oracle.have_ref() else [])


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_basic_s32(impl):
    a = np.array([[1, -2, 3], [-4, 5, -6]], np.int8)
    b = np.array([[1, 2], [3, 4], [5, 6]], np.int8)  # stored [K,N]
    assert oracle.gemm_i8(a, b.T, impl=impl).ravel().tolist() == [10, 12, -19, -24]


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_zero_points_s32(impl):
    a = np.array([[1, 2, 3], [4, 5, 6]], np.int8)
    w = np.array([[7, 8, 9], [10, 11, 12]], np.int8)
    out = oracle.gemm_i8(a, w, zp_a=np.array([1, 2]), zp_w=np.array([3, 4]), scale_a=np.ones(2),
                         scale_w=np.ones(2), impl=impl)
    assert out.ravel().tolist() == [17, 23, 47, 65]


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_u8_zero_points_s32(impl):
    a = np.array([[130, 128, 3], [200, 255, 0]], np.uint8)
    b = np.array([[1, -4], [2, 5], [3, -6]], np.int8)
    out = oracle.gemm_i8(a, b.T, zp_a=np.array([128, 100]), scale_a=np.ones(2), zp_w=3, impl=impl)
    assert out.ravel().tolist() == [-4, 1111, -355, 510]


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_requant_and_clamp(impl):
    out = oracle.gemm_i8(np.array([[4, 6]], np.int8), np.ones((2, 2), np.int8), out_kind="s8", out_scale=2.0,
                         impl=impl)
    assert out.ravel().tolist() == [5, 5]
    out = oracle.gemm_i8(np.array([[100, 100]], np.int8), np.full((2, 2), 100, np.int8), out_kind="s8", impl=impl)
    assert out.ravel().tolist() == [127, 127]


def test_requant_rounds_half_away_from_zero():
    # acc = +/-1, +/-3 with scale 0.5 -> +/-0.5, +/-1.5 -> +/-1, +/-2 (ties away), not ties-to-even (0, 2).
    a = np.array([[1], [-1], [3], [-3]], np.int8)
    w = np.array([[1]], np.int8)
    out = oracle.gemm_i8(a, w, out_kind="s8", out_scale=2.0)
    assert out.ravel().tolist() == [1, -1, 2, -2]


def test_requant_f32_half_quirk():
    # x = 0.49999997 (largest f32 below 0.5): x + 0.5 rounds to 1.0 in f32, so the result is 1.
    x = np.nextafter(np.float32(0.5), np.float32(0))
    out = oracle.gemm_i8(np.array([[1]], np.int8), np.array([[1]], np.int8), out_kind="s8", scale_a=float(x))
    assert out.item() == 1


def test_f16_conversions_match_numpy():
    lib = oracle.port_lib()
    rng = np.random.default_rng(1)
    for bits in rng.integers(0, 1 << 16, 4000):
        h = np.uint16(bits).view(np.float16)
        if np.isnan(h):
            continue
        assert lib.oracle_f16_to_f32(int(bits)) == float(np.float32(h))
    vals = np.concatenate([rng.normal(size=2000), rng.normal(size=500) * 1e-6, rng.normal(size=500) * 7e4,
                           [0.0, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.99e-8]]).astype(np.float32)
    for v in vals:
        assert lib.oracle_f32_to_f16(float(v)) == int(np.float32(v).astype(np.float16).view(np.uint16))


def test_q4_1_block_layout():
    # d = 0.5, m = -1; byte j = j | ((15-j) << 4): value j -> j*0.5-1, value j+16 -> (15-j)*0.5-1.
    blk = np.zeros(20, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:4] = np.array([-1.0], np.float16).view(np.uint8)
    blk[4:] = [j | ((15 - j) << 4) for j in range(16)]
    out = oracle.q4_1_decode(blk, 32)
    exp = [j * 0.5 - 1 for j in range(16)] + [(15 - j) * 0.5 - 1 for j in range(16)]
    assert out.tolist() == exp
    assert oracle.q4_1_decode(blk, 20).tolist() == exp[:20]  # partial block


def test_q4_1_quantize_round_trip():
    rng = np.random.default_rng(2)
    x = rng.normal(size=96 + 7).astype(np.float32)
    blocks = oracle.q4_1_quantize(x)
    assert blocks.size == 4 * 20
    y = oracle.q4_1_decode(blocks, x.size)
    d = np.repeat(blocks.reshape(4, 20)[:, :2].copy().view(np.float16).astype(np.float32), 32)[: x.size]
    assert np.all(np.abs(x - y) <= 0.5 * d + 2e-3)


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not runnable on this host")
def test_port_matches_reference_random():
    rng = np.random.default_rng(3)
    for (m, n, k) in [(37, 53, 600), (6, 200, 33), (130, 70, 257)]:
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        kw = dict(scale_a=rng.uniform(0.01, 0.03, m).astype(np.float32),
                  scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32),
                  zp_a=rng.integers(-5, 5, m).astype(np.int32), zp_w=rng.integers(-5, 5, n).astype(np.int32))
        for kind in ("s32", "s8", "u8", "f32", "f16"):
            bias = rng.integers(-1000, 1000, n)
            b = bias.astype(np.int32) if kind in ("s32", "s8", "u8") else bias.astype(np.float32) * 0.01
            for relu in (False, True):
                p = oracle.gemm_i8(a, w, out_kind=kind, bias=b, relu=relu, out_scale=1.6,
                                   out_zp=0 if kind == "s32" else 3, impl="port", **kw)
                r = oracle.gemm_i8(a, w, out_kind=kind, bias=b, relu=relu, out_scale=1.6,
                                   out_zp=0 if kind == "s32" else 3, impl="ref", **kw)
                assert np.array_equal(p.view(np.uint8), r.view(np.uint8)), (m, n, k, kind, relu)


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not runnable on this host")
def test_conv_port_matches_reference():
    """The gather + matmul-epilogue restatement of the int8 convolution against the reference's Conv2D CPU route:
    strides, dilation, padding with a non-zero activation zero point, groups down to one channel, all four
    destinations (shapes after tests/test_cuda_conv2d.cpp:268-315)."""
    rng = np.random.default_rng(17)
    table = [  # n, ic, ih, iw, oc, kh, kw, stride, dilation, padding, groups, act, out
        (1, 16, 8, 8, 8, 3, 3, (1, 1), (1, 1), (1, 1), 1, np.uint8, "s8"),
        (1, 16, 8, 8, 8, 3, 3, (2, 1), (1, 1), (1, 1), 1, np.uint8, "f16"),
        (1, 16, 8, 8, 8, 3, 3, (1, 1), (2, 1), (1, 1), 1, np.int8, "f16"),
        (1, 16, 12, 12, 16, 3, 3, (1, 1), (1, 1), (1, 1), 2, np.uint8, "u8"),
        (1, 16, 8, 8, 16, 3, 3, (1, 1), (1, 1), (1, 1), 16, np.int8, "u8"),
        (1, 32, 32, 32, 24, 3, 3, (1, 1), (1, 1), (1, 1), 1, np.int8, "s8"),
        (2, 24, 15, 17, 40, 5, 3, (2, 3), (1, 2), (2, 1), 1, np.uint8, "s8"),
        (1, 3, 33, 31, 32, 7, 7, (2, 2), (1, 1), (3, 3), 1, np.uint8, "s8"),
        (1, 64, 9, 9, 32, 1, 1, (1, 1), (1, 1), (0, 0), 1, np.int8, "f32"),
    ]
    for (n, ic, ih, iw, oc, kh, kw, stride, dilation, padding, groups, adt, kind) in table:
        x = rng.integers(0, 256, (n, ih, iw, ic), dtype=np.uint8).view(adt)
        w = rng.integers(-127, 128, (kh, kw, ic // groups, oc), dtype=np.int8)
        int_out = kind in ("s8", "u8")
        bias = rng.integers(-1000, 1001, oc).astype(np.int32) if int_out else \
            rng.uniform(-0.5, 0.5, oc).astype(np.float32 if kind == "f32" else np.float16)
        kw_ = dict(stride=stride, dilation=dilation, padding=padding, groups=groups, out_kind=kind, bias=bias, relu=True,
                   scale_x=0.0078125, zp_x=128 if adt == np.uint8 else -6,
                   scale_w=(0.008 + 0.001 * (np.arange(oc) % 5)).astype(np.float32),
                   zp_w=((np.arange(oc) % 7) - 3).astype(np.int32), out_scale=0.03, out_zp=110 if kind == "u8" else 0)
        p = oracle.conv2d_i8(x, w, impl="port", **kw_)
        r = oracle.conv2d_i8(x, w, impl="ref", **kw_)
        assert np.array_equal(p.view(np.uint8), r.view(np.uint8)), (n, ic, ih, iw, oc, kh, kw, groups, kind)


def _golden_cases():
    return sorted(GOLDEN.glob("*.npz"))


@pytest.mark.parametrize("path", _golden_cases(), ids=lambda p: p.stem)
def test_port_matches_golden(path):
    """Fixtures written by tests/golden/make_golden.py from the compiled reference."""
    z = np.load(path)
    meta = json.loads(str(z["meta"]))
    if meta["op"] == "gemm_i8":
        kw = {k: (z[k] if k in z.files else meta["scalars"][k]) for k in meta["kw"]}
        a = z["a"].T if meta.get("a_transposed") else z["a"]
        w = z["w"].T if meta.get("w_kn") else z["w"]
        out = oracle.gemm_i8(a, w, out_kind=meta["out_kind"], relu=meta["relu"], **kw)
        assert np.array_equal(out.view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "conv2d_i8":
        g = meta["geom"]
        out = oracle.conv2d_i8(z["x"], z["w"], out_kind=meta["out_kind"], bias=z["bias"], relu=meta["relu"],
                               scale_w=z["scale_w"], zp_w=z["zp_w"], stride=tuple(g["stride"]),
                               dilation=tuple(g["dilation"]), padding=tuple(g["padding"]), groups=g["groups"],
                               **meta["scalars"])
        assert np.array_equal(out.view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "fp_act":
        pt = meta["per_token"]
        out = oracle.linear_fp_act(z["a"], z["w"], scale_a=z["scale_a"] if pt else float(z["scale_a"][0]),
                                   zp_a=z["zp_a"] if pt else int(z["zp_a"][0]), bias=z["bias"], relu=meta["relu"],
                                   scale_w=z["scale_w"])
        assert np.array_equal(out.view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "quant_linear":
        q = oracle.quantize_linear(z["x"], z["scale"], z["zero_point"], axis=meta["axis"],
                                   out_dtype=z["quantized"].dtype)
        assert np.array_equal(q, z["quantized"])
        dq = oracle.dequantize_linear(z["xq"], z["scale"], z["zero_point"], axis=meta["axis"],
                                      out_dtype=z["dequantized"].dtype)
        assert np.array_equal(dq.view(np.uint8), z["dequantized"].view(np.uint8))
    else:
        out = oracle.q4_1_matmul(z["a"], z["w_blocks"], meta["k"], out_dtype=meta["out_dtype"],
                                 w_round_f16=meta["out_dtype"] == "f16")
        ref = z["out"].astype(np.float32)
        tol = meta["rtol"] * np.abs(ref) + meta["rtol"] * float(np.sqrt(np.mean(ref * ref)))
        assert np.all(np.abs(out.astype(np.float32) - ref) <= tol)


# ---- QuantizeLinear / DequantizeLinear ------------------------------------------------------

def test_quantize_known_answers():
    """Round half to even, saturation, and the x86 conversion's out-of-range rule
    (arithmetic: src/backend/cpu/x86_64/quant.hpp:117-165)."""
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 1000.0, -1000.0, np.inf, -np.inf, np.nan, 3e9], dtype=np.float32)
    q = oracle.quantize_linear(x, [1.0], np.array([0], np.int8))
    assert q.tolist() == [0, 2, 2, 0, -2, -2, 127, -128, -128, -128, -128, -128]
    q = oracle.quantize_linear(x, [1.0], np.array([10], np.uint8), out_dtype=np.uint8)
    assert q.tolist() == [10, 12, 12, 10, 8, 8, 255, 0, 0, 0, 0, 0]
    # per channel along axis 0: row r uses scale[r]
    x2 = np.array([[1.0, 2.0], [1.0, 2.0]], dtype=np.float32)
    q2 = oracle.quantize_linear(x2, [0.5, 0.25], np.array([1, -1], np.int8), axis=0)
    assert q2.tolist() == [[3, 5], [3, 7]]


def test_dequantize_known_answers():
    q = np.array([-128, -1, 0, 1, 127], dtype=np.int8)
    y = oracle.dequantize_linear(q, [0.5], np.array([1], np.int8))
    assert y.tolist() == [-64.5, -1.0, -0.5, 0.0, 63.0]
    y16 = oracle.dequantize_linear(q.view(np.uint8), [0.25], np.array([128], np.uint8), out_dtype=np.float16)
    assert y16.dtype == np.float16 and y16.tolist() == [0.0, 31.75, -32.0, -31.75, -0.25]


def test_dequantize_body_and_tail_round_differently():
    """The first inner - inner % 16 elements of a row go through fma(q, s, -zp*s), the rest
    through (q - zp) * s; with a zero point the two forms differ in the last bit for some
    inputs, and the restatement keeps the position rule."""
    rng = np.random.default_rng(5)
    rows = 4000
    q = rng.integers(-128, 128, (rows, 15)).astype(np.int8)
    s = rng.uniform(0.001, 3, rows).astype(np.float32)
    z = rng.integers(-128, 128, rows).astype(np.int8)
    tail = oracle.dequantize_linear(q, s, z)                                     # 15 < 16: all tail
    body = oracle.dequantize_linear(np.concatenate([q, q[:, :1]], axis=1), s, z)[:, :15]   # 16: all body
    assert np.count_nonzero(tail != body) > 0
    want_tail = (q.astype(np.float32) - z[:, None].astype(np.float32)) * s[:, None]
    assert np.array_equal(tail, want_tail.astype(np.float32))


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not runnable on this host")
def test_quant_linear_port_matches_reference():
    rng = np.random.default_rng(9)
    cases = [((70001,), -1, 1), ((37, 75), -1, 37), ((5, 12, 23), 1, 12), ((6, 50), 1, 50), ((4, 100, 64), 0, 4),
             ((3000, 15), -1, 3000)]
    for shape, axis, count in cases:
        scale = rng.uniform(0.05, 3.0, count).astype(np.float32)
        for fdt in (np.float32, np.float16):
            x = (rng.standard_normal(shape) * 40).astype(fdt)
            flat = x.reshape(-1)
            flat[::7] = ((rng.integers(-300, 300, flat[::7].size) + 0.5) * scale[0]).astype(fdt)
            flat[:3] = [np.inf, -np.inf, np.nan]
            for qdt in (np.int8, np.uint8):
                zp = (rng.integers(-20, 20, count) if qdt == np.int8 else rng.integers(0, 255, count)).astype(qdt)
                assert np.array_equal(oracle.quantize_linear(x, scale, zp, axis=axis, out_dtype=qdt),
                                      oracle.quantize_linear(x, scale, zp, axis=axis, out_dtype=qdt, impl="ref"))
                xq = (rng.integers(-128, 128, shape) if qdt == np.int8 else rng.integers(0, 256, shape)).astype(qdt)
                p = oracle.dequantize_linear(xq, scale, zp, axis=axis, out_dtype=fdt)
                r = oracle.dequantize_linear(xq, scale, zp, axis=axis, out_dtype=fdt, impl="ref")
                assert np.array_equal(p.view(np.uint8), r.view(np.uint8)), (shape, axis, fdt, qdt)


# Known-answer cases of the reference's own operator test (tests/test_quant_linear.cpp:35-300 for
# QuantizeLinear, :361-500 for DequantizeLinear): (x, scale, zero point, axis, expected).
_REF_QUANTIZE_KATS = [
    ([0.0, 1.0, 2.0], [1.0], np.array([0], np.int8), -1, [0, 1, 2]),
    ([0.0, 2.0, 4.0], [2.0], np.array([0], np.int8), -1, [0, 1, 2]),
    ([0.0, 1.0, 2.0], [1.0], np.array([100], np.int8), -1, [100, 101, 102]),
    ([-1.0, 0.0, 1.0, 300.0], [1.0], np.array([0], np.uint8), -1, [0, 0, 1, 255]),
    ([0.0, 1.0, -1.0], [1.0], np.array([128], np.uint8), -1, [128, 129, 127]),
    ([[0.0, 1.0, 2.0], [10.0, 11.0, 12.0]], [1.0, 2.0, 3.0], np.zeros(3, np.int8), 1, [[0, 0, 1], [10, 6, 4]]),
    ([[0.0, 1.0, 2.0], [10.0, 20.0, 30.0]], [1.0, 10.0], np.zeros(2, np.int8), -1, [[0, 1, 2], [1, 2, 3]]),
    ([[[0.0, 1.0], [2.0, 4.0]], [[10.0, 20.0], [30.0, 40.0]]], [1.0, 2.0, 5.0, 10.0], np.zeros(4, np.int8), -1,
     [[[0, 1], [1, 2]], [[2, 4], [3, 4]]]),
]
_REF_DEQUANTIZE_KATS = [
    (np.array([0, 1, -1], np.int8), [1.0], np.array([0], np.int8), -1, [0.0, 1.0, -1.0]),
    (np.array([100, 101, 102], np.int8), [2.0], np.array([100], np.int8), -1, [0.0, 2.0, 4.0]),
    (np.array([128, 129, 127], np.uint8), [0.5], np.array([128], np.uint8), -1, [0.0, 0.5, -0.5]),
    (np.array([[0, 0, 1], [10, 5, 4]], np.int8), [1.0, 2.0, 3.0], np.zeros(3, np.int8), 1,
     [[0.0, 0.0, 3.0], [10.0, 10.0, 12.0]]),
    (np.array([[1, 2, 3], [4, 5, 6]], np.int8), [0.5, 2.0], np.zeros(2, np.int8), -1,
     [[0.5, 1.0, 1.5], [8.0, 10.0, 12.0]]),
]


@pytest.mark.parametrize("case", range(len(_REF_QUANTIZE_KATS)))
def test_quantize_reference_kats(case):
    x, scale, zp, axis, want = _REF_QUANTIZE_KATS[case]
    got = oracle.quantize_linear(np.array(x, np.float32), scale, zp, axis=axis, out_dtype=zp.dtype)
    assert got.tolist() == want
    got16 = oracle.quantize_linear(np.array(x, np.float16), scale, zp, axis=axis, out_dtype=zp.dtype)
    assert got16.tolist() == want


@pytest.mark.parametrize("case", range(len(_REF_DEQUANTIZE_KATS)))
def test_dequantize_reference_kats(case):
    x, scale, zp, axis, want = _REF_DEQUANTIZE_KATS[case]
    assert oracle.dequantize_linear(x, scale, zp, axis=axis).tolist() == want
    assert oracle.dequantize_linear(x, scale, zp, axis=axis, out_dtype=np.float16).tolist() == want


@pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not runnable on this host")
def test_fp_activation_route_port_matches_reference():
    """f32/f16 activations with per-tensor / per-token parameters x s8 weights: quantise, int8
    matmul, dequantize -- the composed restatement equals the reference Linear bit for bit."""
    rng = np.random.default_rng(12)
    for (m, n, k) in [(37, 53, 600), (6, 200, 64), (130, 70, 257)]:
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
        for fdt in (np.float32, np.float16):
            a = (rng.standard_normal((m, k)) * 2).astype(fdt)
            bias = (rng.normal(size=n) * 3).astype(fdt)
            for sa, za in ((0.03, 0), (0.03, 3), (rng.uniform(0.01, 0.05, m).astype(np.float32), 0),
                           (rng.uniform(0.01, 0.05, m).astype(np.float32), rng.integers(-9, 10, m).astype(np.int32))):
                for relu in (False, True):
                    p = oracle.linear_fp_act(a, w, scale_a=sa, zp_a=za, bias=bias, relu=relu, scale_w=sw)
                    r = oracle.linear_fp_act(a, w, scale_a=sa, zp_a=za, bias=bias, relu=relu, scale_w=sw, impl="ref")
                    assert np.array_equal(p.view(np.uint8), r.view(np.uint8)), (m, n, k, fdt, relu)
