"""Deterministic synthetic inputs for the benchmark configurations.

No dataset is involved: the Llama shape names are only shapes.  Every tensor is drawn from a
numpy Philox stream seeded ``1000*(config-1) + tensor_index`` (0 = activations, 1 = weights,
2 = bias, 3 = weight scales), so the GPU run, the CPU baseline and the golden fixtures all read
the same bytes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

Q4_1_BLOCK_BYTES = 20
Q4_1_BLOCK_ELEMS = 32


def _rng(config: int, tensor: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(1000 * (config - 1) + tensor))


def s8_uniform(rng: np.random.Generator, shape) -> np.ndarray:
    """Uniform integers in [-127, 127]."""
    return rng.integers(-127, 128, size=shape, dtype=np.int8)


@dataclass
class Int8Case:
    name: str
    a: np.ndarray          # s8 [M,K]
    w: np.ndarray          # s8 [N,K]
    bias: np.ndarray       # s32 [N]
    out_kind: str
    relu: bool
    scale_a: float
    scale_w: np.ndarray | float
    out_scale: float

    @property
    def ops(self) -> int:
        return 2 * self.a.shape[0] * self.w.shape[0] * self.a.shape[1]

    def kwargs(self) -> dict:
        return dict(out_kind=self.out_kind, bias=self.bias, relu=self.relu, scale_a=self.scale_a,
                    scale_w=self.scale_w, out_scale=self.out_scale)


def config1(m: int = 128, n: int = 1024, k: int = 1024) -> Int8Case:
    """s8 x s8 -> s32, int32 bias, no epilogue."""
    return Int8Case("cfg1_s32", s8_uniform(_rng(1, 0), (m, k)), s8_uniform(_rng(1, 1), (n, k)),
                    _rng(1, 2).integers(-2**15, 2**15 + 1, size=n).astype(np.int32), "s32", False, 1.0, 1.0, 1.0)


def _requant_case(config: int, name: str, m: int, n: int, k: int, out_scale: float) -> Int8Case:
    return Int8Case(name, s8_uniform(_rng(config, 0), (m, k)), s8_uniform(_rng(config, 1), (n, k)),
                    _rng(config, 2).integers(-1000, 1001, size=n).astype(np.int32), "s8", True, 0.02,
                    _rng(config, 3).uniform(0.001, 0.02, size=n).astype(np.float32), out_scale)


def config2(m: int = 512, n: int = 11008, k: int = 4096, out_scale: float = 0.05) -> Int8Case:
    """Llama-7B MLP shape: s8 requant epilogue with per-channel weight scales, bias, Relu.
    With the stated scales ~94 % of outputs saturate; ``out_scale=1.6`` keeps them in range so
    the rounding path is exercised."""
    return _requant_case(2, "cfg2_s8_relu", m, n, k, out_scale)


def config5(m: int = 4096, n: int = 28672, k: int = 8192, out_scale: float = 0.05) -> Int8Case:
    """Llama-3-70B MLP shape, the sharded configuration (same epilogue as config 2)."""
    return _requant_case(5, "cfg5_s8_relu", m, n, k, out_scale)


def q4_1_weights(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """uint8 [n, ceil(k/32)*20]: per block d = f16(U[0.005,0.02]), m = f16(-8*d*U[0.8,1.2]) computed
    from the rounded d, 16 nibble bytes uniform in 0..255."""
    nblk = (k + Q4_1_BLOCK_ELEMS - 1) // Q4_1_BLOCK_ELEMS
    d = rng.uniform(0.005, 0.02, size=(n, nblk)).astype(np.float16)
    u = rng.uniform(0.8, 1.2, size=(n, nblk)).astype(np.float32)
    mn = (-8.0 * d.astype(np.float32) * u).astype(np.float16)
    qs = rng.integers(0, 256, size=(n, nblk, 16), dtype=np.uint8)
    blocks = np.empty((n, nblk, Q4_1_BLOCK_BYTES), dtype=np.uint8)
    blocks[:, :, 0:2] = d.view(np.uint8).reshape(n, nblk, 2)
    blocks[:, :, 2:4] = mn.view(np.uint8).reshape(n, nblk, 2)
    blocks[:, :, 4:] = qs
    return blocks.reshape(n, nblk * Q4_1_BLOCK_BYTES)


@dataclass
class Q41Case:
    name: str
    a: np.ndarray          # f16 [M,K]
    w_blocks: np.ndarray   # uint8 [N, K/32*20]
    k: int
    out_dtype: str

    @property
    def flops(self) -> int:
        return 2 * self.a.shape[0] * self.w_blocks.shape[0] * self.k

    @property
    def bytes(self) -> int:
        """Algorithmic bytes of one call: weight stream + activations + output."""
        out_b = 2 if self.out_dtype == "f16" else 4
        return self.w_blocks.size + self.a.size * 2 + self.a.shape[0] * self.w_blocks.shape[0] * out_b


def config3(m: int = 1, n: int = 4096, k: int = 4096) -> Q41Case:
    """Decode-step GEMV: f16 activations ~N(0,1), f32 output."""
    a = _rng(3, 0).standard_normal(size=(8, k)).astype(np.float32).astype(np.float16)[:m]
    return Q41Case(f"cfg3_gemv_m{m}", np.ascontiguousarray(a), q4_1_weights(_rng(3, 1), n, k), k, "f32")


def config4(m: int = 2048, n: int = 14336, k: int = 4096) -> Q41Case:
    """Prefill GEMM, Llama-3-8B up-projection shape: f16 in, f16 out."""
    a = _rng(4, 0).standard_normal(size=(m, k)).astype(np.float32).astype(np.float16)
    return Q41Case("cfg4_gemm", a, q4_1_weights(_rng(4, 1), n, k), k, "f16")
