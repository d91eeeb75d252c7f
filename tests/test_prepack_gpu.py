"""Prepacked int8 weights (nnb200_i8_pack): the blob's sections, and calls against it -- byte for
byte what the unpacked call and the oracle give, with fewer kernels when zero points are in play
and the tensor-core engine for weights whose own storage would not qualify."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from nnops_b200 import capi, ops

pytestmark = pytest.mark.gpu


def _weights(rng, n, k):
    return rng.integers(-127, 128, (n, k), dtype=np.int8)


@pytest.mark.parametrize("n,k", [(130, 200), (64, 64), (1003, 96), (17, 1000)])
@pytest.mark.parametrize("kn_storage", [False, True])
def test_blob_sections(cuda_device, nnb200_lib, n, k, kn_storage):
    rng = np.random.default_rng(n + k)
    w = _weights(rng, n, k)
    scale = rng.uniform(0.001, 0.02, n).astype(np.float32)
    zp = rng.integers(-9, 10, n).astype(np.int32)
    if kn_storage:
        tw = torch.from_numpy(np.ascontiguousarray(w.T)).to(cuda_device).t()      # [K, N] storage, logical [N, K]
    else:
        tw = torch.from_numpy(np.pad(w, ((0, 0), (0, 5)))).to(cuda_device)[:, :k]  # odd pitch
    p = ops.prepack_i8(tw, scale_w=scale, zp_w=torch.from_numpy(zp).to(cuda_device))   # host scales, device zps
    torch.cuda.synchronize()
    pitch = (k + 15) // 16 * 16
    assert p.blob.numel() == n * (pitch + 12)
    rows = p.blob[: n * pitch].view(torch.int8).view(n, pitch).cpu().numpy()
    assert np.array_equal(rows[:, :k], w)
    assert not rows[:, k:].any(), "pad columns must be zero"
    assert np.array_equal(p.scale_w.cpu().numpy(), scale)
    assert np.array_equal(p.zp_w.cpu().numpy(), zp)
    assert np.array_equal(p.r_w.cpu().numpy(), w.astype(np.int32).sum(axis=1))


def test_scalar_parameters_fill_the_sections(cuda_device, nnb200_lib):
    rng = np.random.default_rng(3)
    w = _weights(rng, 70, 130)
    p = ops.prepack_i8(torch.from_numpy(w).to(cuda_device), scale_w=0.015, zp_w=-2)
    assert np.all(p.scale_w.cpu().numpy() == np.float32(0.015))
    assert np.all(p.zp_w.cpu().numpy() == -2)


@pytest.mark.parametrize("out_kind", ["s32", "s8", "f16"])
def test_packed_call_matches_oracle_and_skips_the_weight_sweep(cuda_device, nnb200_lib, out_kind):
    rng = np.random.default_rng(11)
    m, n, k = 77, 130, 272
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    w = _weights(rng, n, k)
    kw = dict(scale_a=rng.uniform(0.01, 0.03, m).astype(np.float32), zp_a=rng.integers(100, 140, m).astype(np.int32),
              out_scale=2.3, out_zp=0 if out_kind == "s32" else -3)
    sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
    zw = rng.integers(-9, 10, n).astype(np.int32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32) if out_kind != "f16" else rng.normal(size=n).astype(np.float16)
    want = oracle.gemm_i8(a, w, out_kind=out_kind, bias=bias, relu=True, scale_w=sw, zp_w=zw, **kw)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    packed = ops.prepack_i8(tw, scale_w=sw, zp_w=zw)
    act = "relu" if out_kind == "f16" else "none"
    lib = capi.lib()
    n0 = lib.nnb200_launch_count()
    plain = ops.gemm_i8(ta, tw, out_kind=out_kind, bias=bias, relu=True, activation=act, scale_w=sw, zp_w=zw, **kw)
    n1 = lib.nnb200_launch_count()
    got = ops.gemm_i8_packed(ta, packed, out_kind=out_kind, bias=bias, relu=True, activation=act, **kw)
    n2 = lib.nnb200_launch_count()
    assert np.array_equal(got.cpu().numpy().view(np.uint8), want.view(np.uint8))
    assert np.array_equal(plain.cpu().numpy().view(np.uint8), want.view(np.uint8))
    assert (n1 - n0, n2 - n1) == (3, 2), "packed: R_a sweep + GEMM; unpacked: R_a, R_w sweeps + GEMM"


def test_packing_makes_any_weight_storage_tensor_core_eligible(cuda_device, nnb200_lib):
    """A weight stored [K, N] (MatMul without transpose_b) with K not a multiple of 16 runs on
    the generic engine as it is, and on the tensor-core engine once packed -- same bytes out."""
    rng = np.random.default_rng(5)
    m, n, k = 200, 330, 1000
    a_np = rng.integers(-127, 128, (m, k + 8), dtype=np.int8)            # 16-byte row pitch for A
    w_kn = rng.integers(-127, 128, (k, n), dtype=np.int8)
    a = torch.from_numpy(a_np).to(cuda_device)[:, :k]
    tw = torch.from_numpy(w_kn).to(cuda_device).t()
    sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
    want = oracle.gemm_i8(a_np[:, :k], w_kn.T, out_kind="s8", scale_w=sw, out_scale=1.7, relu=True)
    o = torch.empty((m, n), dtype=torch.int8, device=cuda_device)
    assert ops.gemm_i8_engine(a, tw, o, out_kind="s8", scale_w=sw, out_scale=1.7, relu=True) == "generic"
    packed = ops.prepack_i8(tw, scale_w=sw)
    assert ops.gemm_i8_engine(a, packed.w, o, out_kind="s8", scale_w=packed.scale_w, out_scale=1.7, relu=True) == "umma"
    got = ops.gemm_i8_packed(a, packed, out_kind="s8", out_scale=1.7, relu=True)
    assert np.array_equal(got.cpu().numpy(), want)


def test_packed_decode(cuda_device, nnb200_lib):
    rng = np.random.default_rng(6)
    m, n, k = 4, 520, 1024
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = _weights(rng, n, k)
    sw = rng.uniform(0.001, 0.02, n).astype(np.float32)
    want = oracle.gemm_i8(a, w, out_kind="s8", scale_w=sw, out_scale=1.1, relu=True)
    packed = ops.prepack_i8(torch.from_numpy(w).to(cuda_device), scale_w=sw)
    got = ops.gemm_i8_packed(torch.from_numpy(a).to(cuda_device), packed, out_kind="s8", out_scale=1.1, relu=True)
    assert np.array_equal(got.cpu().numpy(), want)


def test_rejections(cuda_device, nnb200_lib):
    lib = capi.lib()
    w = torch.zeros((8, 32), dtype=torch.int8, device=cuda_device)
    blob = torch.zeros(lib.nnb200_i8_pack_bytes(8, 32), dtype=torch.uint8, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    too_small = lib.nnb200_i8_pack(w.data_ptr(), 8, 32, 32, 1, None, 1.0, None, 0, blob.data_ptr(), blob.numel() - 1, stream)
    assert too_small == capi.INVALID_ARGUMENT
    no_unit_stride = lib.nnb200_i8_pack(w.data_ptr(), 8, 16, 64, 2, None, 1.0, None, 0, blob.data_ptr(), blob.numel(), stream)
    assert no_unit_stride == capi.INVALID_ARGUMENT
    assert lib.nnb200_i8_pack_bytes(0, 32) == 0
    torch.cuda.synchronize()
    assert not blob.any(), "a refused pack wrote nothing"


# ---- Q4_1: separated nibble and (d, m) planes ---------------------------------------------------

def _q4_problem(n, k, m, seed, a_dtype=np.float16):
    from nnops_b200 import synth
    rng = np.random.default_rng(seed)
    wb = synth.q4_1_weights(rng, n, k)
    a = rng.standard_normal((m, k)).astype(a_dtype)
    return wb, a


def test_q4_1_pack_is_a_pure_relayout(cuda_device, nnb200_lib):
    """Every block's 4-byte (d, m) header and 16 nibble bytes reappear unchanged in the two planes
    (from a padded source pitch too); pack_bytes follows the stated geometry."""
    from nnops_b200 import capi
    for n, k, pad in ((9, 32, 0), (33, 1000, 3), (130, 4096, 0), (17, 4096 + 128, 4)):
        nblk = (k + 31) // 32
        wb, _ = _q4_problem(n, k, 1, n + k)
        src = np.zeros((n, (nblk + pad) * 20), dtype=np.uint8)
        src[:, : nblk * 20] = wb
        tw = torch.from_numpy(src).to(cuda_device)[:, : nblk * 20]
        pk = ops.prepack_q4_1(tw, k)
        assert pk.blob.numel() == capi.lib().nnb200_q4_1_pack_bytes(n, k) == n * (nblk * 16 + (-(-nblk // 4) * 4) * 4)
        blocks = wb.reshape(n, nblk, 20)
        assert np.array_equal(pk.qs.cpu().numpy().reshape(n, nblk, 16), blocks[:, :, 4:])
        assert np.array_equal(pk.dm.cpu().numpy().reshape(n, nblk, 4), blocks[:, :, :4])


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 11])
@pytest.mark.parametrize("a_dtype,out_dtype", [("f16", "f32"), ("f16", "f16"), ("f32", "f32")])
def test_q4_1_packed_gemv(cuda_device, nnb200_lib, m, a_dtype, out_dtype):
    """The GEMV on packed planes: same values as on the raw stream (the arithmetic is the same,
    only the loads differ), within the f32 tolerance of the CPU oracle."""
    n, k = 203, 1024
    wb, a = _q4_problem(n, k, m, m, np.float16 if a_dtype == "f16" else np.float32)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    pk = ops.prepack_q4_1(tw, k)
    tdt = torch.float32 if out_dtype == "f32" else torch.float16
    assert ops.q4_1_engine(ta, pk, k, out_dtype=tdt) == 6
    got = ops.linear_q4_1(ta, pk, k, out_dtype=tdt)
    raw = ops.linear_q4_1(ta, tw, k, out_dtype=tdt, engine="gemv_dsq")
    assert torch.equal(got, raw), "packed and raw weights must give identical results"
    want = oracle.q4_1_matmul(a, wb, k, out_dtype=out_dtype)
    rtol = 2e-3 if out_dtype == "f32" else 1e-2
    tol = rtol * np.abs(want.astype(np.float32)) + rtol * float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    assert np.all(np.abs(got.cpu().numpy().astype(np.float32) - want.astype(np.float32)) <= tol)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (8, 4096, 4096), (1, 5000, 2048 + 128), (2, 37, 12288), (1, 16, 128)])
def test_q4_1_packed_gemv_shapes(cuda_device, nnb200_lib, shape):
    m, n, k = shape
    wb, a = _q4_problem(n, k, m, n + k)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    pk = ops.prepack_q4_1(tw, k)
    got = ops.linear_q4_1(ta, pk, k, out_dtype=torch.float32)
    raw = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float32, engine="gemv_dsq")
    assert torch.equal(got, raw)
    want = oracle.q4_1_matmul(a, wb, k, out_dtype="f32").astype(np.float64)
    err = np.abs(got.cpu().numpy().astype(np.float64) - want).max() / np.sqrt(np.mean(want ** 2))
    assert err < 2e-5, err


def test_q4_1_packed_two_pass_gemm(cuda_device, nnb200_lib):
    """A tall call on packed weights expands the planes once and runs the dense GEMM: bit-identical
    to the same call on the raw stream."""
    m, n, k = 600, 1100, 320
    wb, a = _q4_problem(n, k, m, 5)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    pk = ops.prepack_q4_1(tw, k)
    assert ops.q4_1_engine(ta, pk, k, out_dtype=torch.float16) == 5
    got = ops.linear_q4_1(ta, pk, k, out_dtype=torch.float16)
    raw = ops.linear_q4_1(ta, tw, k, out_dtype=torch.float16, engine="gemm_two_pass")
    assert torch.equal(got, raw)


def test_q4_1_packed_refusals(cuda_device, nnb200_lib):
    """Shapes no engine serves on packed weights are refused, not silently mis-read: the fused GEMM
    and the per-weight GEMV engines only understand the raw stream."""
    import ctypes as C
    from nnops_b200 import capi
    wb, a = _q4_problem(64, 256, 40, 1)
    ta, tw = torch.from_numpy(a).to(cuda_device), torch.from_numpy(wb).to(cuda_device)
    pk = ops.prepack_q4_1(tw, 256)
    out = torch.full((40, 64), 7.0, dtype=torch.float16, device=cuda_device)
    for engine in ("gemm", "gemv_mma", "gemv_simt"):
        args = ops.q4_1_args(ta, pk, out, 256, engine=engine)
        assert capi.lib().nnb200_linear_q4_1(C.byref(args), None) == capi.UNSUPPORTED
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
