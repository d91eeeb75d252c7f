"""QuantizeLinear / DequantizeLinear CUDA kernels against the CPU oracle, through the C ABI:
byte for byte, all three granularities, f32/f16 x s8/u8, ties, non-finite inputs, rows whose
length breaks the vector path, misaligned bases, and a tensor larger than L2."""
import zlib

import numpy as np
import pytest
import torch

import oracle
from nnops_b200 import ops

pytestmark = pytest.mark.gpu

CASES = [
    # shape, axis, granularity
    ((70001,), -1, "tensor"),            # scalar kernel (length not a multiple of 4)
    ((64, 4096), -1, "tensor"),
    ((37, 75), -1, "token"),             # scalar kernel
    ((200, 1028), -1, "token"),          # f32: vector kernel with a 4-element CPU-tail region per row
    ((50, 1032), -1, "token"),           # f32 and f16 vector kernels, 8-element CPU-tail region per row
    ((5, 12, 24), 1, "channel"),
    ((6, 50), 1, "channel"),             # channel = last axis: inner 1
    ((4, 100, 64), 0, "channel"),
    ((3, 16, 8, 20), 2, "channel"),
]


def _params(rng, shape, axis, gran, qdt):
    count = {"tensor": 1, "token": int(np.prod(shape[:-1])), "channel": shape[axis]}[gran]
    scale = rng.uniform(0.05, 3.0, count).astype(np.float32)
    zp = (rng.integers(-128, 128, count) if qdt == np.int8 else rng.integers(0, 256, count)).astype(qdt)
    return scale, zp


@pytest.mark.parametrize("qdt", [np.int8, np.uint8])
@pytest.mark.parametrize("fdt", [np.float32, np.float16])
@pytest.mark.parametrize("shape,axis,gran", CASES)
def test_quantize_matches_oracle(cuda_device, nnb200_lib, shape, axis, gran, fdt, qdt):
    rng = np.random.default_rng(zlib.crc32(repr((shape, axis, fdt.__name__, qdt.__name__)).encode()))
    scale, zp = _params(rng, shape, axis, gran, qdt)
    x = (rng.standard_normal(shape) * 60).astype(fdt)
    flat = x.reshape(-1)
    flat[::5] = ((rng.integers(-90, 90, flat[::5].size) + 0.5) * scale[0]).astype(fdt)   # exact ties
    flat[:3] = [np.inf, -np.inf, np.nan]
    if fdt == np.float32:
        flat[3:5] = [3e9, -3e9]
    want = oracle.quantize_linear(x, scale, zp, axis=axis, out_dtype=qdt)
    got = ops.quantize_linear(torch.from_numpy(x).to(cuda_device), torch.from_numpy(scale), torch.from_numpy(zp),
                              axis=axis, out_dtype=torch.int8 if qdt == np.int8 else torch.uint8)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("qdt", [np.int8, np.uint8])
@pytest.mark.parametrize("fdt", [np.float32, np.float16])
@pytest.mark.parametrize("shape,axis,gran", CASES)
def test_dequantize_matches_oracle(cuda_device, nnb200_lib, shape, axis, gran, fdt, qdt):
    rng = np.random.default_rng(zlib.crc32(repr((shape, axis, fdt.__name__, qdt.__name__, 1)).encode()))
    scale, zp = _params(rng, shape, axis, gran, qdt)
    xq = (rng.integers(-128, 128, shape) if qdt == np.int8 else rng.integers(0, 256, shape)).astype(qdt)
    want = oracle.dequantize_linear(xq, scale, zp, axis=axis, out_dtype=fdt)
    got = ops.dequantize_linear(torch.from_numpy(xq).to(cuda_device), torch.from_numpy(scale), torch.from_numpy(zp),
                                axis=axis, out_dtype=torch.float32 if fdt == np.float32 else torch.float16)
    assert np.array_equal(got.cpu().numpy().view(np.uint8), want.view(np.uint8))


def test_misaligned_bases_take_the_scalar_kernels(cuda_device, nnb200_lib):
    rng = np.random.default_rng(3)
    n = 4096
    x = (rng.standard_normal(n + 1) * 30).astype(np.float32)
    tx = torch.from_numpy(x).to(cuda_device)[1:]                 # 4-byte aligned only
    ty = torch.zeros(n + 3, dtype=torch.int8, device=cuda_device)[3:]   # odd byte offset
    ops.quantize_linear(tx, [0.7], torch.tensor([3], dtype=torch.int8), out=ty)
    want = oracle.quantize_linear(x[1:], [0.7], np.array([3], np.int8))
    assert np.array_equal(ty.cpu().numpy(), want)
    back = ops.dequantize_linear(ty, [0.7], torch.tensor([3], dtype=torch.int8))
    assert np.array_equal(back.cpu().numpy(), oracle.dequantize_linear(want, [0.7], np.array([3], np.int8)))


def test_empty_and_rejections(cuda_device, nnb200_lib):
    e = ops.quantize_linear(torch.empty((0, 8), device=cuda_device), [1.0], torch.tensor([0], dtype=torch.int8))
    assert e.shape == (0, 8)
    with pytest.raises(ValueError):
        ops.quantize_linear(torch.zeros((4, 8), device=cuda_device), [1.0, 2.0, 3.0],
                            torch.zeros(3, dtype=torch.int8))        # 3 scales for 4 rows


def test_round_trip_full_size(cuda_device, nnb200_lib):
    """The activation tensor of the headline layer (4096 x 8192, 134 MB as f32 -- larger than
    L2): quantize per token, dequantize, quantize again; the second quantization must
    reproduce the first (idempotence of Q after DQ), and a sampled band equals the oracle."""
    g = torch.Generator(device="cpu").manual_seed(7)
    x = torch.randn((4096, 8192), generator=g, dtype=torch.float32)
    scale = (x.abs().amax(dim=1) / 127.0).to(torch.float32)
    zp = torch.zeros(4096, dtype=torch.int8)
    xd = x.to(cuda_device)
    q1 = ops.quantize_linear(xd, scale, zp)
    dq = ops.dequantize_linear(q1, scale, zp)
    q2 = ops.quantize_linear(dq, scale, zp)
    assert torch.equal(q1, q2)
    band = slice(1000, 1064)
    want = oracle.quantize_linear(x[band].numpy(), scale[band].numpy(), zp[band].numpy())
    assert np.array_equal(q1[band].cpu().numpy(), want)
    want_dq = oracle.dequantize_linear(want, scale[band].numpy(), zp[band].numpy())
    assert np.array_equal(dq[band].cpu().numpy(), want_dq)
