"""Parity of the Q4_1 CUDA kernels with the CPU oracle, through the C ABI.

Tolerances follow the benchmark contract: f32 output rtol 2e-3, f16 output rtol 1e-2, each
with an absolute floor of rtol * rms(reference) (a purely relative test is unsatisfiable near
zero).  The oracle accumulates in f64, so it is an order-free expected value like the one the
reference's own test recomputes (tests/test_matmul_q4_1.cpp:190-224).
"""
import numpy as np
import pytest
import torch

import oracle
from nnops_b200 import ops, synth

pytestmark = pytest.mark.gpu

RTOL_F32 = 2e-3
RTOL_F16 = 1e-2


def _close(got, ref, rtol):
    got = got.astype(np.float32)
    ref = ref.astype(np.float32)
    tol = rtol * np.abs(ref) + rtol * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside tolerance; max err {np.abs(got - ref).max()}"


def test_decode_matches_oracle_bitwise(cuda_device, nnb200_lib):
    rng = np.random.default_rng(0)
    for k in (32, 64, 100, 4096):
        wb = synth.q4_1_weights(rng, 9, k)
        got = ops.q4_1_decode(torch.from_numpy(wb).to(cuda_device), k).cpu().numpy()
        want = np.stack([oracle.q4_1_decode(wb[i], k) for i in range(wb.shape[0])])
        assert np.array_equal(got, want)


@pytest.mark.parametrize("engine", ["gemv_simt", "gemv_mma", "gemv_dsq"])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 11])
@pytest.mark.parametrize("a_dtype,out_dtype", [("f16", "f32"), ("f16", "f16"), ("f32", "f32")])
def test_gemv_small(cuda_device, nnb200_lib, m, a_dtype, out_dtype, engine):
    rng = np.random.default_rng(m)
    n, k = (203, 1000) if engine == "gemv_simt" else (203, 1024)   # ragged N; ragged K on the CUDA-core engine
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16 if a_dtype == "f16" else np.float32)
    bias = rng.standard_normal(n).astype(np.float32 if out_dtype == "f32" else np.float16)
    want = oracle.q4_1_matmul(a, wb, k, out_dtype=out_dtype, bias=bias)
    got = ops.linear_q4_1(torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device), k,
                          out_dtype=torch.float32 if out_dtype == "f32" else torch.float16, bias=bias,
                          engine=engine)
    _close(got.cpu().numpy(), want, RTOL_F32 if out_dtype == "f32" else RTOL_F16)


ENGINE_IDS = {"gemv_mma": 4, "gemv_dsq": 6}


@pytest.mark.parametrize("engine", ["gemv_mma", "gemv_dsq"])
@pytest.mark.parametrize("shape", [(1, 16, 128), (4, 40, 384), (8, 130, 4096 + 128), (7, 17, 8192 + 256), (3, 64, 4096),
                                   (2, 33, 12288), (1, 5000, 2048 + 128), (1, 37, 32768), (2, 2400, 640)])
def test_gemv_mma_edges(cuda_device, nnb200_lib, shape, engine):
    """Fewer block groups than K-quarter warps, K spanning several staged chunks, channel counts
    off the 16-row tile, and a weight view whose row pitch is wider than its rows."""
    m, n, k = shape
    rng = np.random.default_rng(n + k)
    nblk = k // 32
    ld = nblk + 4                                   # padded pitch, still a multiple of 4 blocks
    wb_dense = synth.q4_1_weights(rng, n, k)
    wb = np.zeros((n, ld * 20), dtype=np.uint8)
    wb[:, : nblk * 20] = wb_dense
    a = rng.standard_normal((m, k)).astype(np.float16)
    ta = torch.from_numpy(a).to(cuda_device)
    tw = torch.from_numpy(wb).to(cuda_device)[:, : nblk * 20]
    # The deferred-scaling engine stages one pass's activations whole in shared memory (64 KB).
    mp = 1 if m == 1 else (2 if m == 2 else (4 if m <= 4 else 8))      # MMA columns per block
    fits = mp * (-(-nblk // 8) * 8) * 64 <= 64 * 1024
    want_id = ENGINE_IDS[engine] if (engine == "gemv_mma" or fits) else 4
    assert ops.q4_1_engine(ta, tw, k, engine=engine) == want_id
    assert ops.q4_1_engine(ta, tw, k, engine="gemv") == (6 if (fits and m == 1) else 4)   # automatic choice
    got = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float32, engine=engine)
    _close(got.cpu().numpy(), oracle.q4_1_matmul(a, wb_dense, k, out_dtype="f32"), RTOL_F32)


@pytest.mark.parametrize("engine", ["gemv_mma", "gemv_dsq"])
@pytest.mark.parametrize("m", [1, 4, 7])
@pytest.mark.parametrize("aligned", [True, False])
def test_gemv_mma_f32_activations(cuda_device, nnb200_lib, m, aligned, engine):
    """f32 activations on the warp-MMA engine: each row feeds two MMA columns (hi and lo f16
    parts), four rows per pass; accuracy stays at f32 level."""
    rng = np.random.default_rng(m + 40)
    n, k = 300, 4096
    wb = synth.q4_1_weights(rng, n, k)
    a = (rng.standard_normal((m, k)) * 5).astype(np.float32)
    if aligned:
        ta = torch.from_numpy(a).to(cuda_device)
    else:
        ta = torch.from_numpy(np.pad(a, ((0, 0), (1, 2)))).to(cuda_device)[:, 1:k + 1]   # 4-byte aligned rows only
    tw = torch.from_numpy(wb).to(cuda_device)
    assert ops.q4_1_engine(ta, tw, k, engine=engine) == ENGINE_IDS[engine]
    got = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float32, engine=engine).cpu().numpy()
    # The per-weight-dequantising engine rounds each weight to f16 (like the reference's f16
    # route); the deferred-scaling engine multiplies exact nibbles and scales in f32.
    want = oracle.q4_1_matmul(a, wb, k, out_dtype="f32", w_round_f16=(engine == "gemv_mma")).astype(np.float64)
    err = np.abs(got.astype(np.float64) - want).max() / np.sqrt(np.mean(want ** 2))
    assert err < 2e-5, err


def test_gemv_falls_back_when_rows_are_not_bulk_copyable(cuda_device, nnb200_lib):
    """K = 1000 (31.25 blocks): rows are not a whole number of 16-byte pieces, so the CUDA-core
    GEMV must be chosen -- and still match."""
    rng = np.random.default_rng(12)
    m, n, k = 3, 50, 1000
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    assert ops.q4_1_engine(ta, tw, k, engine="gemv") == 3
    got = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float32)
    _close(got.cpu().numpy(), oracle.q4_1_matmul(a, wb, k, out_dtype="f32"), RTOL_F32)


@pytest.mark.parametrize("engine", ["gemv_simt", "gemv_mma", "gemv_dsq"])
@pytest.mark.parametrize("m", [1, 8])
def test_config3_gemv(cuda_device, nnb200_lib, m, engine):
    c = synth.config3(m)
    want = oracle.q4_1_matmul(c.a, c.w_blocks, c.k, out_dtype="f32")
    got = ops.linear_q4_1(torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w_blocks).to(cuda_device), c.k,
                          out_dtype=torch.float32, engine=engine).cpu().numpy()
    _close(got, want, RTOL_F32)
    if engine == "gemv_dsq":
        # Exact nibbles, exact products, f32 sums: the only error left is f32 accumulation.
        err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max() / np.sqrt(np.mean(want.astype(np.float64) ** 2))
        assert err < 2e-5, err


def test_gemv_dsq_subnormal_and_large_activations(cuda_device, nnb200_lib):
    """The nibbles enter the MMA as f16 subnormals (q * 2^-24): activations from the smallest
    normal f16 magnitudes to the largest must still give exact products."""
    rng = np.random.default_rng(77)
    n, k = 96, 1024
    wb = synth.q4_1_weights(rng, n, k)
    for scale in (1e-4, 1.0, 3e3):
        a = (rng.standard_normal((2, k)) * scale).astype(np.float16)
        want = oracle.q4_1_matmul(a, wb, k, out_dtype="f32").astype(np.float64)
        got = ops.linear_q4_1(torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device), k,
                              out_dtype=torch.float32, engine="gemv_dsq").cpu().numpy().astype(np.float64)
        err = np.abs(got - want).max() / np.sqrt(np.mean(want ** 2))
        assert err < 2e-5, (scale, err)


@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 256, 256), (130, 300, 512), (64, 1000, 160),
                                   (300, 260, 1000), (2048, 1024, 512),
                                   (1024, 4864, 256), (1000, 4810, 320), (520, 9500, 96)])  # 256-row tiles
@pytest.mark.parametrize("out_dtype", ["f16", "f32"])
def test_gemm_umma_shapes(cuda_device, nnb200_lib, shape, out_dtype):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    want = oracle.q4_1_matmul(a, wb, k, out_dtype=out_dtype, w_round_f16=True)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    tdt = torch.float16 if out_dtype == "f16" else torch.float32
    o = torch.empty((m, n), dtype=tdt, device=cuda_device)
    got = ops.linear_q4_1(ta, tw, k, out=o, engine="gemm")
    _close(got.cpu().numpy(), want, RTOL_F16 if out_dtype == "f16" else RTOL_F32)


@pytest.mark.parametrize("shape", [(128, 128, 64), (130, 300, 512), (64, 1000, 160), (300, 260, 1000),
                                   (2048, 1024, 512), (1000, 4810, 320), (520, 9500, 96), (640, 7168, 128)])
@pytest.mark.parametrize("out_dtype", ["f16", "f32"])
def test_gemm_two_pass_shapes(cuda_device, nnb200_lib, shape, out_dtype):
    """Expand-then-dense-GEMM form: ragged M / N / K, every tile width the picker can choose."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + 1)
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    want = oracle.q4_1_matmul(a, wb, k, out_dtype=out_dtype, w_round_f16=True)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    tdt = torch.float16 if out_dtype == "f16" else torch.float32
    assert ops.q4_1_engine(ta, tw, k, out_dtype=tdt, engine="gemm_two_pass") == 5
    assert ops.q4_1_engine(ta, tw, k, out_dtype=tdt) == (5 if m >= 256 else 1)
    o = torch.empty((m, n), dtype=tdt, device=cuda_device)
    got = ops.linear_q4_1(ta, tw, k, out=o, engine="gemm_two_pass")
    _close(got.cpu().numpy(), want, RTOL_F16 if out_dtype == "f16" else RTOL_F32)


@pytest.mark.parametrize("shape", [(700, 5000, 1000), (2048, 4096, 64), (1024, 7000, 192), (520, 9500, 96)])
def test_gemm_two_pass_pair_forms_agree(cuda_device, nnb200_lib, shape, knobs):
    """The dense pass of the two-pass form has a single-CTA kernel and three CTA-pair variants
    (knob f16_pair: 0 = single, 1 / 3 = earlier pair forms, default = two k-blocks per barrier
    slot with one commit): the accumulation order is the same in all of them, so the outputs are
    bit-identical -- odd and single counts of k-blocks included."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + 3)
    ta = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).to(cuda_device)
    tw = torch.from_numpy(synth.q4_1_weights(rng, n, k)).to(cuda_device)
    ref = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float16, engine="gemm_two_pass").clone()
    for form in (0, 1, 3, 2):
        knobs("f16_pair", form)
        got = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float16, engine="gemm_two_pass")
        assert torch.equal(got, ref), form


@pytest.mark.parametrize("shape", [(96, 160, 512), (130, 300, 1000), (600, 1100, 320), (2048, 1024, 96)])
@pytest.mark.parametrize("out_dtype", ["f32", "f16"])
def test_gemm_two_pass_f32_activations(cuda_device, nnb200_lib, shape, out_dtype):
    """f32 activations (the reference's f32 -> f32 pose) at GEMM sizes: split into [hi | lo] f16 in
    the scratch, dense GEMM over 2K with the weights repeating.  Held to the f32 tolerance."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + 2)
    wb = synth.q4_1_weights(rng, n, k)
    a = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    want = oracle.q4_1_matmul(a, wb, k, out_dtype=out_dtype, w_round_f16=True)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    tdt = torch.float16 if out_dtype == "f16" else torch.float32
    assert ops.q4_1_engine(ta, tw, k, out_dtype=tdt) == 5
    got = ops.linear_q4_1(ta, tw, k, out_dtype=tdt)
    _close(got.cpu().numpy(), want, RTOL_F16 if out_dtype == "f16" else RTOL_F32)
    if out_dtype == "f32":   # the split carries 22 mantissa bits: far inside the tolerance
        ref64 = oracle.q4_1_matmul(a, wb, k, out_dtype="f32", w_round_f16=True).astype(np.float64)
        err = np.abs(got.cpu().numpy().astype(np.float64) - ref64).max() / np.sqrt(np.mean(ref64 ** 2))
        assert err < 2e-5, err


def test_gemm_two_pass_needs_its_scratch(cuda_device, nnb200_lib):
    """Without the scratch the same call runs the fused kernel: same result within tolerance."""
    import ctypes as C
    from nnops_b200 import capi
    rng = np.random.default_rng(8)
    m, n, k = 600, 512, 256
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    o = torch.empty((m, n), dtype=torch.float16, device=cuda_device)
    args = ops.q4_1_args(ta, tw, o, k)                       # no workspace set
    assert capi.lib().nnb200_q4_1_workspace_bytes(C.byref(args)) == n * k * 2
    assert capi.lib().nnb200_q4_1_engine(C.byref(args)) == 1
    capi.check(capi.lib().nnb200_linear_q4_1(C.byref(args), torch.cuda.current_stream().cuda_stream), "q4_1")
    want = oracle.q4_1_matmul(a, wb, k, out_dtype="f16", w_round_f16=True)
    _close(o.cpu().numpy(), want, RTOL_F16)


def test_gemm_epilogue_bias_relu(cuda_device, nnb200_lib):
    rng = np.random.default_rng(4)
    m, n, k = 256, 384, 256
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    bias = rng.standard_normal(n).astype(np.float16)
    want = np.maximum(oracle.q4_1_matmul(a, wb, k, out_dtype="f32", w_round_f16=True) + bias.astype(np.float32), 0)
    for engine in ("gemm", "gemm_two_pass"):
        got = ops.linear_q4_1(torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device), k,
                              out_dtype=torch.float16, bias=bias, activation="relu", engine=engine)
        _close(got.cpu().numpy(), want, RTOL_F16)


@pytest.mark.parametrize("engine", ["gemm", "gemm_two_pass"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu", "hard_swish"])
def test_gemm_epilogue_alpha_bias_clip_activation(cuda_device, nnb200_lib, engine, out_dtype, act):
    """alpha, bias, clip and every activation class of the tensor-core GEMMs' drain (one loop per
    class): what the same arithmetic in float64 gives on the SAME engine's plain f32 product."""
    rng = np.random.default_rng(11)
    m, n, k = 256, 392, 256
    wb = torch.from_numpy(synth.q4_1_weights(rng, n, k)).to(cuda_device)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).to(cuda_device)
    bias = rng.uniform(-2, 2, n).astype(np.float32)
    plain = ops.linear_q4_1(a, wb, k, out_dtype=torch.float32, engine=engine).cpu().numpy().astype(np.float64)
    b_t = torch.from_numpy(bias.astype(np.float16 if out_dtype == torch.float16 else np.float32)).to(cuda_device)
    got = ops.linear_q4_1(a, wb, k, out_dtype=out_dtype, bias=b_t, alpha=0.75, min_clip=-6.0, max_clip=9.0,
                          activation=act, act_alpha=0.1, act_beta=1.5, engine=engine)
    torch.cuda.synchronize()
    x = np.clip(plain * 0.75 + b_t.cpu().numpy().astype(np.float64), -6.0, 9.0)
    if act == "relu":
        want = np.maximum(x, 0)
    elif act == "gelu":
        want = 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    elif act == "silu":
        want = x / (1 + np.exp(-x))
    elif act == "hard_swish":
        want = x * np.clip(x + 3, 0, 6) * (1.5 / 6)
    else:
        want = x
    err = np.abs(got.cpu().numpy().astype(np.float64) - want)
    tol = (1e-5 + 1e-5 * np.abs(want)) if out_dtype == torch.float32 else (2e-3 + 2e-3 * np.abs(want))
    assert (err <= tol).all(), (act, float(err.max()))


def _close_abs_rms(got, ref, rtol, atol_rms):
    """|got - ref| <= atol_rms * rms(ref) + rtol * |ref| elementwise."""
    got = got.astype(np.float32)
    ref = ref.astype(np.float32)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    bad = np.abs(got - ref) > atol_rms * rms + rtol * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside tolerance; max err {np.abs(got - ref).max()}, rms {rms}"
    return rms


def test_config4_whole_output_vs_reference(cuda_device, nnb200_lib):
    """Full prefill shape, every row.  Expected value: the reference's f32-activation Linear
    (f32 activations holding the f16 values, so both sides read identical operands), rounded
    once to f16 -- rtol 1e-2 with an absolute floor of 1e-2 * rms.  The reference's own
    f16 -> f16 route is compared too, but only loosely: it rounds its partial sums to f16
    every 128 k (src/backend/cpu/matmul/matmul_helper.h:19-22), its own tests allow 5e-2
    (tests/common/test_helpers.hpp:36-43), and its distance to the f32 route is reported."""
    c = synth.config4()
    ta, tw = torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w_blocks).to(cuda_device)
    for engine in ("auto", "gemm"):             # two-pass form (default with scratch) and the fused kernel
        got = ops.linear_q4_1(ta, tw, c.k, out_dtype=torch.float16, engine=engine).cpu().numpy()
        if oracle.have_ref():
            want32 = oracle.q4_1_matmul(c.a.astype(np.float32), c.w_blocks, c.k, out_dtype="f32", impl="ref")
            want = want32.astype(np.float16)
            rms = _close_abs_rms(got, want, RTOL_F16, RTOL_F16)
            ref16 = oracle.q4_1_matmul(c.a, c.w_blocks, c.k, out_dtype="f16", impl="ref").astype(np.float32)
            ours = np.abs(got.astype(np.float32) - want32).max() / rms
            theirs = np.abs(ref16 - want32).max() / rms
            print(f"config 4 [{engine}]: max |err| / rms vs the reference f32 route: this library {ours:.2e}, "
                  f"the reference's f16 route {theirs:.2e}")
            assert np.abs(got.astype(np.float32) - ref16).max() <= 5e-2 * rms
        else:
            rows = np.random.default_rng(1).choice(c.a.shape[0], 24, replace=False)
            want = oracle.q4_1_matmul(np.ascontiguousarray(c.a[rows]), c.w_blocks, c.k, out_dtype="f16")
            _close(got[rows], want, RTOL_F16)


@pytest.mark.parametrize("m", [1, 8])
def test_config3_vs_reference_route(cuda_device, nnb200_lib, m):
    """Config 3 (f16 activations, f32 output) is not a reference pose: its expected value is the
    reference's f32 -> f32 Linear fed f32 activations that hold the f16 values.  Also the
    reference pose f16 -> f16 against the reference's own fused small-M route."""
    if not oracle.have_ref():
        pytest.skip("compiled reference route not runnable on this host")
    c = synth.config3(m)
    ta, tw = torch.from_numpy(c.a).to(cuda_device), torch.from_numpy(c.w_blocks).to(cuda_device)
    want = oracle.q4_1_matmul(c.a.astype(np.float32), c.w_blocks, c.k, out_dtype="f32", impl="ref")
    got = ops.linear_q4_1(ta, tw, c.k, out_dtype=torch.float32).cpu().numpy()
    _close(got, want, RTOL_F32)
    want16 = oracle.q4_1_matmul(c.a, c.w_blocks, c.k, out_dtype="f16", impl="ref")
    got16 = ops.linear_q4_1(ta, tw, c.k, out_dtype=torch.float16).cpu().numpy()
    _close(got16, want16, RTOL_F16)
