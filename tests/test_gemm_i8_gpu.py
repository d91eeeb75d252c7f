"""Parity of the int8 CUDA engines with the CPU oracle, through the C ABI.

Mirrors the reference's differential CUDA tests (tests/test_cuda_matmul.cpp:681-889,
tests/test_cuda_linear.cpp:190-351): same bytes to both sides, integer outputs compared
byte for byte; ragged M/N/K tails, odd N, per-token / per-channel parameters, all five
destinations, both operand poses, batch broadcast -- plus pitched views with canary bytes,
which the reference leaves untested.
"""
import numpy as np
import pytest
import torch

import oracle
from nnops_b200 import capi, ops, synth

pytestmark = pytest.mark.gpu


def _run_case(dev, m, n, k, *, out_kind="s32", a_unsigned=False, relu=False, bias=True, per_token=False,
              per_channel=False, zero_points=False, out_scale=1.0, out_zp=0, engine="auto", seed=0,
              expect_engine=None, act="none", min_clip=-np.inf, max_clip=np.inf, min_workspace=False,
              expect_shared_k=None):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8) if a_unsigned else rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    kw = {}
    kw["scale_a"] = rng.uniform(0.01, 0.03, m).astype(np.float32) if per_token else 0.02
    kw["scale_w"] = rng.uniform(0.001, 0.02, n).astype(np.float32) if per_channel else 0.01
    if zero_points:
        kw["zp_a"] = rng.integers(-9, 10, m).astype(np.int32) if per_token else (128 if a_unsigned else 3)
        kw["zp_w"] = rng.integers(-9, 10, n).astype(np.int32) if per_channel else -2
    int_out = out_kind in ("s32", "s8", "u8")
    b = None
    if bias:
        b = rng.integers(-1000, 1001, n).astype(np.int32) if int_out else \
            (rng.normal(size=n) * 3).astype(np.float32 if out_kind == "f32" else np.float16)
    common = dict(out_kind=out_kind, bias=b, out_scale=out_scale, out_zp=out_zp, **kw)
    want = oracle.gemm_i8(a, w, relu=relu, min_clip=min_clip, max_clip=max_clip, **common)
    ta, tw = torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev)
    if expect_engine is not None:
        o = torch.empty((m, n), dtype=ops._OUT_TORCH[out_kind], device=dev)
        assert ops.gemm_i8_engine(ta, tw, o, engine=engine, **common) == expect_engine
    if expect_shared_k is not None:
        # The scratch for sharing K among the SMs is what the full workspace has over the minimum.
        import ctypes
        from nnops_b200 import capi
        o = torch.empty((m, n), dtype=ops._OUT_TORCH[out_kind], device=dev)
        probe = ops.gemm_i8_args(ta, tw, o, engine=engine, min_workspace=True, **common)
        full = capi.lib().nnb200_gemm_i8_workspace_bytes(ctypes.byref(probe))
        least = capi.lib().nnb200_gemm_i8_min_workspace_bytes(ctypes.byref(probe))
        assert (full > least) == expect_shared_k
    got = ops.gemm_i8(ta, tw, relu=relu, activation=("relu" if relu and not int_out else act), engine=engine,
                      min_clip=min_clip, max_clip=max_clip, min_workspace=min_workspace, **common)
    torch.cuda.synchronize()
    got = got.cpu().numpy()
    assert got.shape == want.shape
    if not np.array_equal(got.view(np.uint8), want.view(np.uint8)):
        bad = np.argwhere(got != want)
        raise AssertionError(f"{len(bad)} mismatches of {got.size}; first {bad[:5].tolist()} "
                             f"got {got[tuple(bad[0])]} want {want[tuple(bad[0])]}")


@pytest.mark.parametrize("engine", ["umma", "generic"])
def test_tiny_s32(cuda_device, nnb200_lib, engine):
    _run_case(cuda_device, 128, 64, 128, engine=engine, bias=False)


@pytest.mark.parametrize("engine", ["umma", "generic"])
@pytest.mark.parametrize("shape", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (100, 200, 300),
                                   (129, 257, 130), (1, 16, 16), (17, 33, 48), (300, 1000, 96), (64, 4096, 64)])
def test_s32_shapes(cuda_device, nnb200_lib, engine, shape):
    m, n, k = shape
    _run_case(cuda_device, m, n, k, engine=engine, seed=m + n + k)


@pytest.mark.parametrize("out_kind", ["s32", "s8", "u8", "f32", "f16"])
@pytest.mark.parametrize("relu", [False, True])
def test_destinations_umma(cuda_device, nnb200_lib, out_kind, relu):
    _run_case(cuda_device, 200, 330, 512, out_kind=out_kind, relu=relu, per_token=True, per_channel=True,
              out_scale=1.7, out_zp=0 if out_kind == "s32" else 5, engine="umma", expect_engine="umma", seed=7)


@pytest.mark.parametrize("out_kind", ["s32", "s8", "u8", "f32", "f16"])
@pytest.mark.parametrize("a_unsigned", [False, True])
def test_zero_points(cuda_device, nnb200_lib, out_kind, a_unsigned):
    for engine in ("umma", "generic"):
        _run_case(cuda_device, 77, 130, 272, out_kind=out_kind, a_unsigned=a_unsigned, relu=True, per_token=True,
                  per_channel=True, zero_points=True, out_scale=2.3, out_zp=0 if out_kind == "s32" else -3,
                  engine=engine, seed=11)


def test_scalar_zero_points_u8(cuda_device, nnb200_lib):
    _run_case(cuda_device, 64, 96, 160, out_kind="s8", a_unsigned=True, zero_points=True, out_scale=3.0, engine="umma")


def test_fp_clip(cuda_device, nnb200_lib):
    _run_case(cuda_device, 40, 100, 256, out_kind="f32", per_channel=True, min_clip=-1.5, max_clip=2.5, engine="umma")


@pytest.mark.parametrize("m", [1, 2, 3, 8, 9, 16])
def test_decode_engines(cuda_device, nnb200_lib, m):
    """M <= 16 on a layer of modest width: the streaming warp-MMA engine (K a multiple of 64); for
    any other K the tensor-core engine with the weights as the 128-row operand; the dp4a engine
    on request."""
    few = "decode"
    _run_case(cuda_device, m, 520, 1024, out_kind="s8", relu=True, per_channel=True, out_scale=1.1,
              expect_engine=few, seed=m)
    _run_case(cuda_device, m, 520, 1024, out_kind="s8", relu=True, per_channel=True, out_scale=1.1,
              engine="decode", expect_engine="decode", seed=m)
    _run_case(cuda_device, m, 520, 1024, out_kind="s8", relu=True, per_channel=True, out_scale=1.1,
              engine="narrow", expect_engine="narrow", seed=m)
    # K not a multiple of 64
    _run_case(cuda_device, m, 130, 4096 + 16, out_kind="s32", a_unsigned=True, zero_points=True, per_token=True,
              per_channel=True, expect_engine="skinny", seed=m + 50)
    _run_case(cuda_device, m, 130, 4096 + 16, out_kind="s32", a_unsigned=True, zero_points=True, per_token=True,
              per_channel=True, engine="narrow", expect_engine="narrow", seed=m + 50)
    # ragged channel count (n % 16 != 0), u8 activations with zero points, K with a partial unroll group
    _run_case(cuda_device, m, 1003, 64 * 37, out_kind="s32", a_unsigned=True, zero_points=True, per_token=True,
              per_channel=True, engine="decode", expect_engine="decode", seed=m + 70)
    _run_case(cuda_device, m, 48, 64, out_kind="f16", per_channel=True, engine="decode", expect_engine="decode",
              seed=m + 90)


@pytest.mark.parametrize("m", [17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("out_kind", ["s32", "s8", "u8", "f32", "f16"])
def test_skinny_engine(cuda_device, nnb200_lib, m, out_kind):
    """17..128 activation rows: the weights are the MMA's 128-row operand, the accumulator comes
    out transposed.  Ragged N and K, u8 activations, zero points, every destination."""
    _run_case(cuda_device, m, 1003, 528, out_kind=out_kind, a_unsigned=(m % 2 == 0), relu=True, per_token=True,
              per_channel=True, zero_points=True, out_scale=1.9, out_zp=0 if out_kind == "s32" else 4,
              engine="skinny", expect_engine="skinny", seed=m)
    _run_case(cuda_device, m, 4096, 4096, out_kind=out_kind, relu=True, per_channel=True, out_scale=1.3,
              engine="skinny", expect_engine="skinny", seed=m + 1)


@pytest.mark.parametrize("shape", [(1280, 16384), (11008, 4096), (28672, 1024), (2999, 8192 + 48), (19000, 2048)])
@pytest.mark.parametrize("m", [9, 16, 33, 64, 100, 128])
def test_skinny_engine_shared_k(cuda_device, nnb200_lib, knobs, m, shape):
    """Layers whose 128-channel tiles do not fill the SMs evenly: every SM takes an equal share
    of all K blocks, tiles are finished by whichever part arrives last.  Few tiles with a long K
    (a tile in a dozen parts), ragged N and K, zero points (both halves of the workspace in use),
    and the same call with the minimum workspace (whole tiles per SM)."""
    knobs("i8_share_k", 2)   # offer the split for short shares too
    n, k = shape
    kinds = ["s32", "s8", "u8", "f32", "f16"]
    out_kind = kinds[(m + n) % 5]
    zp = (m + n // 7) % 2 == 0
    for least in (False, True):
        _run_case(cuda_device, m, n, k, out_kind=out_kind, a_unsigned=(m % 2 == 0), relu=True, per_token=True,
                  per_channel=True, zero_points=zp, out_scale=90.0, out_zp=0 if out_kind == "s32" else 4,
                  engine="skinny", expect_engine="skinny", seed=m + n, min_workspace=least, expect_shared_k=True)


def test_skinny_engine_shared_k_by_default_on_long_streams(cuda_device, nnb200_lib):
    _run_case(cuda_device, 12, 28672, 8192, out_kind="s8", per_channel=True, out_scale=90.0, expect_engine="skinny",
              expect_shared_k=True, seed=5)
    _run_case(cuda_device, 12, 11008, 4096, out_kind="s8", per_channel=True, out_scale=90.0, engine="skinny",
              expect_engine="skinny", expect_shared_k=False, seed=6)


def test_skinny_engine_shared_k_not_offered_when_tiles_fill_the_sms(cuda_device, nnb200_lib, knobs):
    knobs("i8_share_k", 2)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    _run_case(cuda_device, 24, 128 * sms, 2048, out_kind="s8", per_channel=True, out_scale=40.0, engine="skinny",
              expect_engine="skinny", expect_shared_k=False)
    _run_case(cuda_device, 24, 640, 512, out_kind="s8", per_channel=True, out_scale=40.0, engine="skinny",
              expect_engine="skinny", expect_shared_k=False)


@pytest.mark.parametrize("case", [(8, 28672, 1024, "decode"), (12, 4096, 1024, "decode"), (16, 12288, 512, "decode"),
                                  (12, 14336, 512, "skinny"), (16, 28672, 512, "skinny"), (24, 4096, 1024, "umma"),
                                  (100, 9472, 512, "umma"), (24, 11008, 512, "skinny"), (64, 28672, 512, "skinny"),
                                  (100, 11008, 512, "skinny"), (100, 28672, 512, "umma"), (129, 11008, 512, "umma"),
                                  (12, 4096, 28672, "skinny"), (8, 4096, 28672, "decode")])
def test_few_row_engine_choice(cuda_device, nnb200_lib, case):
    """The measured crossovers between the streaming engine, weights-as-rows and the square engine."""
    m, n, k, want = case
    _run_case(cuda_device, m, n, k, out_kind="s8", per_channel=True, out_scale=30.0, expect_engine=want, seed=m + n)


def test_narrow_layer_with_long_k_depends_on_the_workspace(cuda_device, nnb200_lib):
    """4096 channels, K = 14336, 24 rows: with the full workspace the weights-as-rows engine
    shares K among all SMs; with the minimum one the call stays on the square engine.  Same bytes."""
    m, n, k = 24, 4096, 14336
    rng = np.random.default_rng(77)
    a = torch.from_numpy(rng.integers(-127, 128, (m, k), dtype=np.int8)).to(cuda_device)
    w = torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).to(cuda_device)
    sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
    kw = dict(out_kind="s8", scale_a=0.02, scale_w=sw, out_scale=150.0, relu=True)
    o = torch.empty((m, n), dtype=torch.int8, device=cuda_device)
    assert ops.gemm_i8_engine(a, w, o, **kw) == "skinny"
    assert ops.gemm_i8_engine(a, w, o, min_workspace=True, **kw) == "umma"
    full = ops.gemm_i8(a, w, **kw).cpu().numpy()
    least = ops.gemm_i8(a, w, min_workspace=True, **kw).cpu().numpy()
    want = oracle.gemm_i8(a.cpu().numpy(), w.cpu().numpy(), **kw)
    assert np.array_equal(full, want) and np.array_equal(least, want)


def test_skinny_engine_small_m_on_request(cuda_device, nnb200_lib):
    for m in (1, 5, 16):
        _run_case(cuda_device, m, 520, 1024, out_kind="s8", relu=True, per_channel=True, out_scale=1.1,
                  engine="skinny", expect_engine="skinny", seed=m)


@pytest.mark.parametrize("out_kind", ["s32", "s8", "u8", "f32", "f16"])
def test_decode_destinations(cuda_device, nnb200_lib, out_kind):
    _run_case(cuda_device, 5, 700, 4096, out_kind=out_kind, relu=True, per_token=True, per_channel=True,
              out_scale=1.9, out_zp=0 if out_kind == "s32" else 4, expect_engine="decode", seed=21)


@pytest.mark.parametrize("bn", [320, 384, 448, 512])
def test_wide_single_wave_tiles(cuda_device, nnb200_lib, bn, knobs):
    """Tiles wider than 256 columns (two MMAs per k-step, one accumulator): forced through the
    measurement override, once with one tile per CTA and once with several per CTA."""
    knobs("i8_bn", bn)
    _run_case(cuda_device, 300, 1500, 512, out_kind="s8", relu=True, per_token=True, per_channel=True,
              zero_points=True, out_scale=1.9, out_zp=2, engine="umma", seed=bn)
    _run_case(cuda_device, 1100, 4000 + bn, 256, out_kind="s32", per_channel=True, engine="umma", seed=bn + 1)
    _run_case(cuda_device, 2048, 8192, 128, out_kind="f16", per_channel=True, engine="umma", seed=bn + 2)


@pytest.mark.parametrize("form", [2, 1, 3])
@pytest.mark.parametrize("case", [(1100, 9000, 512, "s8"), (2048, 9472, 256, "s32"), (777, 19000, 384, "f16"),
                                  (4096, 4736, 640, "u8"), (600, 20000, 96, "f32"), (1024, 9728, 128, "s8")])
def test_cta_pair_form(cuda_device, nnb200_lib, case, form, knobs):
    """256-row tiles over clusters of two CTAs (tcgen05.mma cta_group::2): forced ("2" = the
    default pair form or an error; 1 and 3 are its earlier variants), ragged M / N / K including
    odd and single counts of 128-byte k-blocks (two share a barrier slot), every destination."""
    m, n, k, kind = case
    knobs("i8_pair", form)
    _run_case(cuda_device, m, n, k, out_kind=kind, relu=True, per_token=True, per_channel=True, zero_points=True,
              out_scale=0.9, out_zp=0 if kind == "s32" else 3, engine="umma", seed=m + n)


@pytest.mark.parametrize("pair", [0, 2])
@pytest.mark.parametrize("case", [(1100, 9000, 512 + 128 * 3, "s8", 1), (2048, 9472, 640, "s32", 5), (1024, 9728, 128, "u8", 7),
                                  (640, 20000, 96, "f16", 3)])
def test_k_blocks_walked_from_a_rotated_start(cuda_device, nnb200_lib, case, pair, knobs):
    """Tiles may start their walk over the K blocks at different blocks (integer sums do not depend
    on the order): same bytes as the oracle for single-CTA and pair tiles, odd block counts, a
    single block, a ragged last block."""
    m, n, k, kind, step = case
    knobs("i8_pair", pair)
    knobs("i8_k_rotate", step)
    _run_case(cuda_device, m, n, k, out_kind=kind, relu=True, per_token=True, per_channel=True, zero_points=True,
              out_scale=0.9, out_zp=0 if kind == "s32" else 3, engine="umma", seed=m + k)


def _np_activation(name, x, alpha, beta):
    """The activations of the fp epilogue (act_apply in csrc/epilogue.cuh; reference:
    include/nnops/core/epilogue.hpp), in float64."""
    x = x.astype(np.float64)
    if name == "relu":
        return np.maximum(x, 0)
    if name == "relu6":
        return np.minimum(np.maximum(x, 0), 6)
    if name == "leaky_relu":
        return np.where(x > 0, x, alpha * x)
    if name == "sigmoid":
        return 1 / (1 + np.exp(-x))
    if name == "tanh":
        return np.tanh(x)
    if name == "gelu":
        return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if name == "silu":
        return x / (1 + np.exp(-x))
    if name == "hard_swish":
        return x * np.minimum(np.maximum(x + 3, 0), 6) * (beta / 6)
    if name == "elu":
        return np.where(x > 0, x, alpha * (np.exp(np.minimum(x, 0)) - 1))
    raise KeyError(name)


@pytest.mark.parametrize("engine", ["umma", "generic"])
@pytest.mark.parametrize("zero_points", [False, True])
@pytest.mark.parametrize("out_kind", ["f32", "f16"])
@pytest.mark.parametrize("act", ["relu", "gelu", "sigmoid", "tanh", "leaky_relu", "silu", "hard_swish", "elu", "relu6"])
def test_fp_destinations_apply_every_activation(cuda_device, nnb200_lib, act, out_kind, zero_points, engine):
    """fp destinations: dequantise, bias, clip, then the activation.  The tensor-core epilogue has
    a loop per (compensation live, activation class); each must give what the activation applied
    to the SAME call's un-activated f32 output gives (that output is bit-exact against the oracle
    elsewhere), to f32 / f16 rounding and the accuracy of the device's exp / tanh."""
    m, n, k = 200, 328, 256
    rng = np.random.default_rng(len(act) * 7 + (1 if zero_points else 0))
    a = torch.from_numpy(rng.integers(-127, 128, (m, k), dtype=np.int8)).to(cuda_device)
    w = torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).to(cuda_device)
    kw = dict(scale_a=0.004, scale_w=rng.uniform(0.0005, 0.002, n).astype(np.float32), engine=engine,
              bias=rng.uniform(-1, 1, n).astype(np.float32), min_clip=-5.0, max_clip=7.0)
    if zero_points:
        kw.update(zp_a=5, zp_w=rng.integers(-4, 5, n).astype(np.int32))
    base = ops.gemm_i8(a, w, out_kind="f32", **kw).cpu().numpy()
    assert np.abs(base).max() > 1.0 and (base < 0).any() and (base > 0).any()
    if out_kind == "f16":
        kw["bias"] = kw["bias"].astype(np.float16)
        base = ops.gemm_i8(a, w, out_kind="f32", **{**kw, "bias": kw["bias"].astype(np.float32)}).cpu().numpy()
    got = ops.gemm_i8(a, w, out_kind=out_kind, activation=act, act_alpha=0.1, act_beta=1.5, **kw)
    torch.cuda.synchronize()
    want = _np_activation(act, base, 0.1, 1.5)
    err = np.abs(got.cpu().numpy().astype(np.float64) - want)
    tol = (2e-6 + 2e-6 * np.abs(want)) if out_kind == "f32" else (1e-3 + 1e-3 * np.abs(want))
    assert (err <= tol).all(), (act, float(err.max()), float(np.abs(want).max()))


def test_transposed_poses_off_the_tma_rule_use_generic(cuda_device, nnb200_lib):
    """[K, M] activations and [K, N] weights whose row pitch is not a multiple of 16 bytes cannot
    be addressed by TMA: the generic engine serves them."""
    rng = np.random.default_rng(5)
    m, n, k = 70, 90, 200
    a_km = rng.integers(-127, 128, (k, m), dtype=np.int8)   # MatMul transpose_a storage
    w_kn = rng.integers(-127, 128, (k, n), dtype=np.int8)   # MatMul without transpose_b
    want = oracle.gemm_i8(a_km.T, w_kn.T, out_kind="s8", out_scale=40.0)
    ta = torch.from_numpy(a_km).to(cuda_device).t()
    tw = torch.from_numpy(w_kn).to(cuda_device).t()
    o = torch.empty((m, n), dtype=torch.int8, device=cuda_device)
    assert ops.gemm_i8_engine(ta, tw, o, out_kind="s8", out_scale=40.0) == "generic"
    got = ops.gemm_i8(ta, tw, out_kind="s8", out_scale=40.0)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("pose", ["nn", "tn", "tt", "nt"])          # (transpose_a, transpose_b) of MatMul: n = no, t = yes
@pytest.mark.parametrize("shape", [(256, 512, 384), (144, 272, 208), (1008, 4112, 96), (2048, 9008, 640), (144, 144, 144),
                                   (528, 4112, 2080)])   # the last one: CTA pairs (K >= 2048, 51 tiles of 256 x 256)
@pytest.mark.parametrize("out_kind", ["s32", "s8", "f16"])
def test_matmul_poses_on_the_tensor_core_engine(cuda_device, nnb200_lib, pose, shape, out_kind):
    """MatMul's four operand poses on the tcgen05 engine (reference: one tile kernel templated on
    TransA / TransB, src/backend/cuda/matmul/matmul_i8_ptx.cu:22-24).  'nn' is MatMul's default:
    A [M, K], B [K, N].  M / N / K off the tile sizes (multiples of 16, as TMA's pitch rule asks), u8 and
    s8 activations, zero points, every kind of destination."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + len(pose))
    a_unsigned = (m + n) % 2 == 0
    a_t, b_t = pose[0] == "t", pose[1] == "t"
    # Storage: A as [M, K] or (transpose_a) [K, M]; B as [K, N] or (transpose_b) [N, K].
    a_store = rng.integers(0, 256, (k, m) if a_t else (m, k), dtype=np.uint8) if a_unsigned else \
        rng.integers(-127, 128, (k, m) if a_t else (m, k), dtype=np.int8)
    b_store = rng.integers(-127, 128, (n, k) if b_t else (k, n), dtype=np.int8)
    a_log = a_store.T if a_t else a_store              # logical [M, K]
    w_log = b_store if b_t else b_store.T              # logical [N, K]
    kw = dict(out_kind=out_kind, scale_a=rng.uniform(0.01, 0.03, m).astype(np.float32),
              scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32), zp_a=128 if a_unsigned else 3,
              zp_w=rng.integers(-9, 10, n).astype(np.int32), out_scale=2.3, out_zp=0 if out_kind == "s32" else 4)
    want = oracle.gemm_i8(a_log, w_log, **kw)
    ta = torch.from_numpy(a_store).to(cuda_device)
    tb = torch.from_numpy(b_store).to(cuda_device)
    ta = ta.t() if a_t else ta
    tw = tb if b_t else tb.t()
    o = torch.empty((m, n), dtype=ops._OUT_TORCH[out_kind], device=cuda_device)
    assert ops.gemm_i8_engine(ta, tw, o, engine="umma", **kw) == "umma"
    got = ops.gemm_i8(ta, tw, engine="umma", **kw).cpu().numpy()
    if not np.array_equal(got.view(np.uint8), want.view(np.uint8)):
        bad = np.argwhere(got != want)
        raise AssertionError(f"{len(bad)} mismatches of {got.size}; first {bad[:5].tolist()}")


@pytest.mark.parametrize("pose", ["nn", "tn", "tt"])
def test_matmul_poses_on_cta_pairs(cuda_device, nnb200_lib, pose, knobs):
    """MN-major operands on the CTA-pair kernel (forced on a small ragged shape, an odd count of
    k-blocks): same bytes as on single CTAs and as the oracle."""
    m, n, k = 304, 528, 2192
    rng = np.random.default_rng(17 + len(pose))
    a_t, b_t = pose[0] == "t", pose[1] == "t"
    a_store = rng.integers(-127, 128, (k, m) if a_t else (m, k), dtype=np.int8)
    b_store = rng.integers(-127, 128, (n, k) if b_t else (k, n), dtype=np.int8)
    a_log = a_store.T if a_t else a_store
    w_log = b_store if b_t else b_store.T
    kw = dict(out_kind="s8", scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32), scale_a=0.02, out_scale=1.7,
              bias=rng.integers(-500, 501, n).astype(np.int32), relu=True)
    want = oracle.gemm_i8(a_log, w_log, **kw)
    ta = torch.from_numpy(a_store).to(cuda_device)
    tb = torch.from_numpy(b_store).to(cuda_device)
    ta = ta.t() if a_t else ta
    tw = tb if b_t else tb.t()
    knobs("i8_pair", 2)
    got = ops.gemm_i8(ta, tw, engine="umma", **kw)
    torch.cuda.synchronize()
    assert capi.take_device_error() == 0
    assert np.array_equal(got.cpu().numpy(), want)
    knobs("i8_pair", 0)
    assert torch.equal(ops.gemm_i8(ta, tw, engine="umma", **kw), got)


def test_matmul_default_pose_takes_the_tensor_core_engine_by_itself(cuda_device, nnb200_lib):
    """MatMul::create({}, Backend::CUDA) on s8 [M, K] x [K, N] must not fall to the SIMT engine."""
    m = n = k = 1024
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=cuda_device)
    b_kn = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=cuda_device)
    o = torch.empty((m, n), dtype=torch.int32, device=cuda_device)
    assert ops.gemm_i8_engine(a, b_kn.t(), o, out_kind="s32") == "umma"
    got = ops.gemm_i8(a, b_kn.t(), out=o)
    want = oracle.gemm_i8(a.cpu().numpy(), b_kn.cpu().numpy().T)
    assert np.array_equal(got.cpu().numpy(), want)


def test_batched_and_broadcast(cuda_device, nnb200_lib):
    rng = np.random.default_rng(6)
    b, m, n, k = 3, 130, 140, 256
    a = rng.integers(-127, 128, (b, m, k), dtype=np.int8)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
    got = ops.gemm_i8(torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device), out_kind="s8",
                      scale_w=sw, out_scale=0.5).cpu().numpy()
    for i in range(b):
        assert np.array_equal(got[i], oracle.gemm_i8(a[i], w, out_kind="s8", scale_w=sw, out_scale=0.5))


@pytest.mark.parametrize("out_kind", ["s8", "s32"])
def test_pitched_views_keep_padding(cuda_device, nnb200_lib, out_kind):
    """Row pitches wider than the rows on every operand; padding bytes of the output stay untouched."""
    rng = np.random.default_rng(8)
    m, n, k = 150, 200, 260
    a_pad = torch.from_numpy(rng.integers(-127, 128, (m, k + 28), dtype=np.int8)).to(cuda_device)
    w_pad = torch.from_numpy(rng.integers(-127, 128, (n, k + 12), dtype=np.int8)).to(cuda_device)
    a, w = a_pad[:, :k], w_pad[:, :k]
    tdt = ops._OUT_TORCH[out_kind]
    out_pad = torch.full((m, n + 24), 0x5A if out_kind == "s8" else 0x5A5A5A5A, dtype=tdt, device=cuda_device)
    ops.gemm_i8(a, w, out_kind=out_kind, out=out_pad[:, :n], out_scale=30.0, relu=True)
    want = oracle.gemm_i8(a.cpu().numpy(), w.cpu().numpy(), out_kind=out_kind, out_scale=30.0, relu=True)
    got = out_pad.cpu().numpy()
    assert np.array_equal(got[:, :n], want)
    assert np.all(got[:, n:] == (0x5A if out_kind == "s8" else 0x5A5A5A5A))


def test_unaligned_falls_back(cuda_device, nnb200_lib):
    """K = 100 rows are not 16-byte pitched: the tensor-core engine must decline, result still exact."""
    rng = np.random.default_rng(9)
    a = torch.from_numpy(rng.integers(-127, 128, (130, 100), dtype=np.int8)).to(cuda_device)
    w = torch.from_numpy(rng.integers(-127, 128, (140, 100), dtype=np.int8)).to(cuda_device)
    o = torch.empty((130, 140), dtype=torch.int32, device=cuda_device)
    assert ops.gemm_i8_engine(a, w, o, out_kind="s32") == "generic"
    got = ops.gemm_i8(a, w, out=o)
    assert np.array_equal(got.cpu().numpy(), oracle.gemm_i8(a.cpu().numpy(), w.cpu().numpy()))


def test_config1_bit_exact(cuda_device, nnb200_lib):
    c = synth.config1()
    got = ops.gemm_i8(torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w).to(cuda_device), **c.kwargs())
    assert np.array_equal(got.cpu().numpy(), oracle.gemm_i8(c.a, c.w, **c.kwargs()))


@pytest.mark.parametrize("out_scale", [0.05, 1.6])
def test_config2_bit_exact(cuda_device, nnb200_lib, out_scale):
    c = synth.config2(out_scale=out_scale)
    got = ops.gemm_i8(torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w).to(cuda_device), **c.kwargs())
    want = oracle.gemm_i8(c.a, c.w, **c.kwargs())
    got = got.cpu().numpy()
    assert np.array_equal(got, want)
    if out_scale > 1:
        inside = np.count_nonzero((want > 0) & (want < 127))
        assert inside > want.size // 4, "in-range variant must exercise the rounding path"


def test_config5_whole_output_and_linearity(cuda_device, nnb200_lib):
    """Full-size sharded shape on one GPU: every one of the 4096 x 28672 output bytes against the
    compiled reference CPU route (the reference's own CUDA tests memcmp whole outputs the same
    way, tests/test_cuda_linear.cpp:190-351), in-range variant included so that the rounding
    path is exercised on every tile; then an exact size-independent property of the s32 route
    (additivity in A).  Without the compiled reference (no VNNI on the host) the C restatement
    checks a sample of rows instead."""
    for out_scale in (0.05, 1.6):
        c = synth.config5(out_scale=out_scale)
        ta, tw = torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w).to(cuda_device)
        got = ops.gemm_i8(ta, tw, **c.kwargs())
        kw = c.kwargs()
        if oracle.have_ref():
            want = oracle.gemm_i8(c.a, c.w, impl="ref", **kw)
            got_h = got.cpu().numpy()
            if not np.array_equal(got_h, want):
                bad = np.argwhere(got_h != want)
                raise AssertionError(f"{len(bad)} of {want.size} bytes differ; first {bad[:5].tolist()}")
            if out_scale > 1:
                assert np.count_nonzero((want > 0) & (want < 127)) > want.size // 4
        else:
            rows = np.random.default_rng(0).choice(c.a.shape[0], 48, replace=False)
            want = oracle.gemm_i8(np.ascontiguousarray(c.a[rows]), c.w, **kw)
            assert np.array_equal(got[torch.from_numpy(rows).to(cuda_device)].cpu().numpy(), want)
    # Linearity: (A1 + A2) W^T == A1 W^T + A2 W^T exactly in int32 (values halved to stay in s8).
    a1 = (ta // 2)
    a2 = ta - a1
    s = ops.gemm_i8(a1, tw) + ops.gemm_i8(a2, tw)
    full = ops.gemm_i8(ta, tw)
    assert torch.equal(s, full)


@pytest.mark.parametrize("shape", [(512, 1024, 1024), (300, 2048 + 16, 512), (4096, 3584, 256)])
@pytest.mark.parametrize("out_kind", ["s8", "u8"])
@pytest.mark.parametrize("peers", [1, 2, 7])
def test_multi_destination_epilogue_local(cuda_device, nnb200_lib, shape, out_kind, peers):
    """The sharded write-back on ONE GPU: the kernel stores its [M, n] window into `out` and into
    `peers` more buffers that play the other ranks' copies (plain local memory here).  Every copy
    must equal the oracle inside the window and stay untouched outside it.  One peer takes the
    variant with a single staging tile per warp and the deeper ring, more take the other."""
    import ctypes as C
    from nnops_b200 import capi
    m, n, k = shape
    rng = np.random.default_rng(m + n)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    kw = dict(out_kind=out_kind, bias=rng.integers(-1000, 1001, n).astype(np.int32), relu=True, scale_a=0.02,
              scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32), out_scale=1.6, out_zp=2)
    want = oracle.gemm_i8(a, w, **kw)
    n_full, col0 = 2 * n + 64, n + 32            # the window sits in the middle of a wider matrix
    tdt = ops._OUT_TORCH[out_kind]
    copies = [torch.full((m, n_full), 0x5A, dtype=tdt, device=cuda_device) for _ in range(1 + peers)]
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    keep = []
    args = ops.gemm_i8_args(ta, tw, copies[0][:, col0:col0 + n], keep=keep, **kw)
    args.num_peer_outs = peers
    for i in range(peers):
        args.peer_out[i] = copies[i + 1][:, col0:col0 + n].data_ptr()
    capi.check(nnb200_lib.nnb200_gemm_i8(C.byref(args), torch.cuda.current_stream(cuda_device).cuda_stream), "gemm")
    torch.cuda.synchronize()
    for c in copies:
        got = c.cpu().numpy()
        assert np.array_equal(got[:, col0:col0 + n], want)
        assert np.all(got[:, :col0] == 0x5A) and np.all(got[:, col0 + n:] == 0x5A)


def test_multi_destination_rejections(cuda_device, nnb200_lib):
    import ctypes as C
    from nnops_b200 import capi
    a = torch.zeros((256, 256), dtype=torch.int8, device=cuda_device)
    w = torch.zeros((256, 256), dtype=torch.int8, device=cuda_device)
    o32 = torch.full((256, 256), 7, dtype=torch.int32, device=cuda_device)
    other = torch.zeros((256, 256), dtype=torch.int32, device=cuda_device)
    args = ops.gemm_i8_args(a, w, o32, out_kind="s32")
    args.num_peer_outs = 1
    args.peer_out[0] = other.data_ptr()
    assert nnb200_lib.nnb200_gemm_i8(C.byref(args), None) == capi.UNSUPPORTED     # 8-bit destinations only
    torch.cuda.synchronize()
    assert bool((o32 == 7).all())
