"""Thin torch-tensor front end over the C ABI, used by the tests, the bench and the sharded
layer.  torch provides device memory and streams only; every computation is a libnnb200 call.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import capi

_OUT_TORCH = {"s32": torch.int32, "s8": torch.int8, "u8": torch.uint8, "f32": torch.float32, "f16": torch.float16}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _dev_array(v, dtype: torch.dtype, device: torch.device, count: int | None):
    """Scalar -> (None, scalar); tensor/sequence -> (device tensor, neutral scalar)."""
    if v is None:
        return None, None
    if isinstance(v, (int, float)):
        return None, v
    t = torch.as_tensor(v, dtype=dtype).to(device).contiguous()
    if count is not None and t.numel() != count:
        raise ValueError(f"expected {count} quantization entries, got {t.numel()}")
    return t, None


def gemm_i8_args(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, out_kind: str, bias=None, relu=False,
                 activation="none", act_alpha=0.0, act_beta=1.0, min_clip=-math.inf, max_clip=math.inf,
                 scale_a=1.0, scale_w=1.0, zp_a=0, zp_w=0, out_scale=1.0, out_zp=0, workspace=None,
                 engine="auto", r_w: torch.Tensor | None = None, min_workspace: bool = False,
                 keep: list | None = None) -> capi.GemmI8Args:
    """Fill the C argument block.  ``a`` is [M,K] or [B,M,K] (s8/u8), ``w`` the LOGICAL [N,K]
    (or [B,N,K]) s8 matrix -- pass ``w_kn.transpose(-1,-2)`` for a weight stored [K,N].
    Tensors created for quantization arrays are appended to ``keep`` so they outlive the call."""
    keep = keep if keep is not None else []
    dev = a.device
    batched = a.dim() == 3 or w.dim() == 3
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    o3 = out if out.dim() == 3 else out.unsqueeze(0)
    batch = max(a3.shape[0], w3.shape[0]) if batched else 1
    m, k = a3.shape[1], a3.shape[2]
    n = w3.shape[1]
    if w3.shape[2] != k:
        raise ValueError("K mismatch")
    sa, sa0 = _dev_array(scale_a, torch.float32, dev, m)
    sw, sw0 = _dev_array(scale_w, torch.float32, dev, n)
    za, za0 = _dev_array(zp_a, torch.int32, dev, m)
    zw, zw0 = _dev_array(zp_w, torch.int32, dev, n)
    keep.extend(t for t in (sa, sw, za, zw) if t is not None)
    if bias is not None:
        bdt = torch.int32 if out_kind in ("s32", "s8", "u8") else _OUT_TORCH[out_kind]
        bias = torch.as_tensor(bias).to(device=dev, dtype=bdt).contiguous()
        keep.append(bias)

    def stride_or_one(t, dim, size):
        return t.stride(dim) if size > 1 else (1 if dim == 2 else t.stride(dim))

    args = capi.GemmI8Args(
        a=a3.data_ptr(), w=w3.data_ptr(), out=o3.data_ptr(), m=m, n=n, k=k,
        a_stride_m=a3.stride(1), a_stride_k=stride_or_one(a3, 2, k),
        w_stride_n=w3.stride(1), w_stride_k=stride_or_one(w3, 2, k),
        ldc=o3.stride(1), batch=batch,
        a_batch_stride=a3.stride(0) if a3.shape[0] > 1 else 0,
        w_batch_stride=w3.stride(0) if w3.shape[0] > 1 else 0,
        out_batch_stride=o3.stride(0) if o3.shape[0] > 1 else 0,
        a_unsigned=int(a.dtype == torch.uint8), out_kind=capi.OUT_KINDS[out_kind],
        bias=bias.data_ptr() if bias is not None else None,
        relu=int(bool(relu)), activation=capi.ACTIVATIONS[activation],
        act_alpha=act_alpha, act_beta=act_beta, min_clip=min_clip, max_clip=max_clip,
        scale_a=sa.data_ptr() if sa is not None else None,
        scale_w=sw.data_ptr() if sw is not None else None,
        zp_a=za.data_ptr() if za is not None else None,
        zp_w=zw.data_ptr() if zw is not None else None,
        scale_a_scalar=1.0 if sa0 is None else float(sa0), scale_w_scalar=1.0 if sw0 is None else float(sw0),
        zp_a_scalar=0 if za0 is None else int(za0), zp_w_scalar=0 if zw0 is None else int(zw0),
        zp_a_nonzero=int(za is not None and bool((za != 0).any().item())),
        zp_w_nonzero=int(zw is not None and bool((zw != 0).any().item())),
        out_scale=float(out_scale), out_zp=int(out_zp),
        workspace=None, workspace_bytes=0, force_engine=capi.ENGINES[engine],
        r_w=r_w.data_ptr() if r_w is not None else None)
    # min_workspace: only what the call cannot do without (no scratch for sharing K among SMs).
    size_fn = capi.lib().nnb200_gemm_i8_min_workspace_bytes if min_workspace else capi.lib().nnb200_gemm_i8_workspace_bytes
    need = size_fn(C.byref(args))
    if need:
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
            keep.append(workspace)
        args.workspace = workspace.data_ptr()
        args.workspace_bytes = workspace.numel()
    return args


def gemm_i8(a: torch.Tensor, w: torch.Tensor, *, out_kind: str = "s32", out: torch.Tensor | None = None, **kw):
    """out = epilogue(a @ w^T) on the current CUDA stream.  Returns the output tensor."""
    if not a.is_cuda:
        raise RuntimeError("nnops_b200.gemm_i8 needs CUDA tensors; there is no CPU path")
    batched = a.dim() == 3 or w.dim() == 3
    m = a.shape[-2]
    n = w.shape[-2]
    if out is None:
        shape = (max(a.shape[0] if a.dim() == 3 else 1, w.shape[0] if w.dim() == 3 else 1), m, n) if batched else (m, n)
        out = torch.empty(shape, dtype=_OUT_TORCH[out_kind], device=a.device)
    keep: list = []
    args = gemm_i8_args(a, w, out, out_kind=out_kind, keep=keep, **kw)
    with torch.cuda.device(a.device):
        capi.check(capi.lib().nnb200_gemm_i8(C.byref(args), _stream_ptr(a.device)), "nnb200_gemm_i8")
    return out


class PackedI8:
    """A prepacked int8 weight: one device blob holding W as [N][pitch] k-contiguous plus the
    per-channel scale, zero point and row-sum sections (see nnb200_i8_pack in nnb200.h)."""

    def __init__(self, blob: torch.Tensor, n: int, k: int, zp_nonzero: bool):
        self.blob, self.n, self.k, self.zp_nonzero = blob, n, k, zp_nonzero
        view = capi.I8Packed()
        capi.check(capi.lib().nnb200_i8_packed_view(blob.data_ptr(), n, k, C.byref(view)), "nnb200_i8_packed_view")
        pitch = view.pitch
        self.w = blob[: n * pitch].view(torch.int8).view(n, pitch)[:, :k]          # [N, K] view with the packed pitch
        self.scale_w = blob[n * pitch: n * pitch + 4 * n].view(torch.float32)
        self.zp_w = blob[n * pitch + 4 * n: n * pitch + 8 * n].view(torch.int32)
        self.r_w = blob[n * pitch + 8 * n: n * pitch + 12 * n].view(torch.int32)


def prepack_i8(w: torch.Tensor, *, scale_w=1.0, zp_w=0) -> PackedI8:
    """Pack the LOGICAL [N, K] s8 weight ``w`` (any strides: pass ``w_kn.t()`` for [K, N] storage)
    with its per-channel or per-tensor parameters (host or device arrays, or scalars)."""
    if w.dim() != 2 or w.dtype != torch.int8 or not w.is_cuda:
        raise ValueError("w must be a 2-D int8 CUDA tensor")
    n, k = w.shape
    if w.stride(0) != 1 and w.stride(1) != 1:
        raise ValueError("one of the weight's strides must be 1")
    blob = torch.empty(capi.lib().nnb200_i8_pack_bytes(n, k), dtype=torch.uint8, device=w.device)
    keep = []

    def arr(v, dt):
        if isinstance(v, (int, float)):
            return None, v
        t = torch.as_tensor(v, dtype=dt).contiguous()       # stays where it is: host or device
        if t.numel() != n:
            raise ValueError(f"expected {n} per-channel entries")
        keep.append(t)
        return t, (1.0 if dt is torch.float32 else 0)

    s, s0 = arr(scale_w, torch.float32)
    z, z0 = arr(zp_w, torch.int32)
    with torch.cuda.device(w.device):
        capi.check(capi.lib().nnb200_i8_pack(
            w.data_ptr(), n, k, w.stride(0) if n > 1 or w.stride(0) == 1 else k, w.stride(1) if k > 1 else 1,
            s.data_ptr() if s is not None else None, float(s0), z.data_ptr() if z is not None else None, int(z0),
            blob.data_ptr(), blob.numel(), _stream_ptr(w.device)), "nnb200_i8_pack")
        if any(not t.is_cuda for t in keep):
            torch.cuda.current_stream(w.device).synchronize()   # host arrays must outlive the copies
    zp_nonzero = bool((z != 0).any().item()) if z is not None else int(z0) != 0
    return PackedI8(blob, n, k, zp_nonzero)


def gemm_i8_packed(a: torch.Tensor, packed: PackedI8, **kw):
    """gemm_i8 against a prepacked weight: per-channel arrays and row sums come from the blob."""
    return gemm_i8(a, packed.w, scale_w=packed.scale_w, zp_w=packed.zp_w if packed.zp_nonzero else 0,
                   r_w=packed.r_w, **kw)


def gemm_i8_engine(a, w, out, **kw) -> str:
    args = gemm_i8_args(a, w, out, **kw)
    return capi.ENGINE_NAMES.get(capi.lib().nnb200_gemm_i8_engine(C.byref(args)), "invalid")


class PackedQ41:
    """A prepacked Q4_1 weight: one device blob holding the nibble plane (16 bytes per block, every
    block 16-byte aligned) and the plane of (f16 d, f16 m) pairs (see nnb200_q4_1_pack)."""

    def __init__(self, blob: torch.Tensor, n: int, k: int):
        self.blob, self.n, self.k = blob, n, k
        view = capi.Q41Packed()
        capi.check(capi.lib().nnb200_q4_1_packed_view(blob.data_ptr(), n, k, C.byref(view)), "nnb200_q4_1_packed_view")
        self.qs_ptr, self.qs_pitch, self.dm_ptr, self.dm_pitch = view.qs, view.qs_pitch, view.dm, view.dm_pitch
        nblk = (k + 31) // 32
        self.qs = blob[: n * self.qs_pitch * 16].view(n, self.qs_pitch * 16)[:, : nblk * 16]
        self.dm = blob[n * self.qs_pitch * 16:].view(n, self.dm_pitch * 4)[:, : nblk * 4]


def prepack_q4_1(w_blocks: torch.Tensor, k: int) -> PackedQ41:
    """Repack raw Q4_1 rows (uint8 [N, ceil(K/32)*20], any 20-byte-multiple pitch) into planes."""
    if w_blocks.dtype != torch.uint8 or w_blocks.dim() != 2 or w_blocks.stride(1) != 1 or w_blocks.stride(0) % 20:
        raise ValueError("w_blocks must be a uint8 [N, row_bytes] tensor whose row pitch is a multiple of 20")
    n = w_blocks.shape[0]
    blob = torch.empty(capi.lib().nnb200_q4_1_pack_bytes(n, k), dtype=torch.uint8, device=w_blocks.device)
    with torch.cuda.device(w_blocks.device):
        capi.check(capi.lib().nnb200_q4_1_pack(w_blocks.data_ptr(), w_blocks.stride(0) // 20, n, k, blob.data_ptr(),
                                               blob.numel(), _stream_ptr(w_blocks.device)), "nnb200_q4_1_pack")
    return PackedQ41(blob, n, k)


def q4_1_args(a: torch.Tensor, w_blocks, out: torch.Tensor, k: int, *, bias=None, activation="none",
              act_alpha=0.0, act_beta=1.0, min_clip=-math.inf, max_clip=math.inf, alpha=1.0, engine="auto",
              overlap_previous: bool = False, keep: list | None = None) -> capi.Q41Args:
    """``w_blocks``: raw rows (uint8 [N, ceil(K/32)*20]) or a PackedQ41."""
    keep = keep if keep is not None else []
    if isinstance(w_blocks, PackedQ41):
        pk = w_blocks
        if a.stride(1) != 1 or out.stride(1) != 1:
            raise ValueError("activations and output must be row-major")
        if bias is not None:
            bias = torch.as_tensor(bias).to(device=a.device, dtype=out.dtype).contiguous()
            keep.append(bias)
        return capi.Q41Args(
            a=a.data_ptr(), w_blocks=pk.qs_ptr, out=out.data_ptr(), m=a.shape[0], n=pk.n, k=k, lda=a.stride(0),
            ldw_blocks=pk.qs_pitch, ldc=out.stride(0), a_f16=int(a.dtype == torch.float16),
            out_f16=int(out.dtype == torch.float16), bias=bias.data_ptr() if bias is not None else None,
            activation=capi.ACTIVATIONS[activation], act_alpha=act_alpha, act_beta=act_beta, min_clip=min_clip,
            max_clip=max_clip, alpha=alpha, workspace=None, workspace_bytes=0, force_engine=capi.Q4_ENGINES[engine],
            flags=capi.Q4_FLAG_OVERLAP_PREVIOUS if overlap_previous else 0, w_dm=pk.dm_ptr, ld_dm=pk.dm_pitch)
    if w_blocks.dtype != torch.uint8 or w_blocks.dim() != 2 or w_blocks.stride(1) != 1 or w_blocks.stride(0) % 20:
        raise ValueError("w_blocks must be a uint8 [N, row_bytes] tensor whose row pitch is a multiple of 20")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("activations and output must be row-major")
    if bias is not None:
        bias = torch.as_tensor(bias).to(device=a.device, dtype=out.dtype).contiguous()
        keep.append(bias)
    return capi.Q41Args(
        a=a.data_ptr(), w_blocks=w_blocks.data_ptr(), out=out.data_ptr(),
        m=a.shape[0], n=w_blocks.shape[0], k=k, lda=a.stride(0), ldw_blocks=w_blocks.stride(0) // 20,
        ldc=out.stride(0), a_f16=int(a.dtype == torch.float16), out_f16=int(out.dtype == torch.float16),
        bias=bias.data_ptr() if bias is not None else None, activation=capi.ACTIVATIONS[activation],
        act_alpha=act_alpha, act_beta=act_beta, min_clip=min_clip, max_clip=max_clip, alpha=alpha,
        workspace=None, workspace_bytes=0, force_engine=capi.Q4_ENGINES[engine],
        flags=capi.Q4_FLAG_OVERLAP_PREVIOUS if overlap_previous else 0)


def linear_q4_1(a: torch.Tensor, w_blocks: torch.Tensor, k: int, *, out_dtype: torch.dtype | None = None,
                out: torch.Tensor | None = None, **kw) -> torch.Tensor:
    """out[M,N] = a[M,K] @ dequant(w_blocks)[N,K]^T.  ``w_blocks``: uint8 [N, ceil(K/32)*20]."""
    if not a.is_cuda:
        raise RuntimeError("nnops_b200.linear_q4_1 needs CUDA tensors; there is no CPU path")
    if a.dtype not in (torch.float16, torch.float32):
        raise ValueError("activations must be f16 or f32")
    n_out = w_blocks.n if isinstance(w_blocks, PackedQ41) else w_blocks.shape[0]
    if out is None:
        out = torch.empty((a.shape[0], n_out), dtype=out_dtype or a.dtype, device=a.device)
    keep: list = []
    args = q4_1_args(a, w_blocks, out, k, keep=keep, **kw)
    need = capi.lib().nnb200_q4_1_workspace_bytes(C.byref(args))
    if need > 0:
        # Scratch for the expanded weights of the two-pass form; torch's allocator is
        # stream-ordered, so letting it go after the call is safe.
        scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
        keep.append(scratch)
        args.workspace = scratch.data_ptr()
        args.workspace_bytes = need
    with torch.cuda.device(a.device):
        capi.check(capi.lib().nnb200_linear_q4_1(C.byref(args), _stream_ptr(a.device)), "nnb200_linear_q4_1")
    return out


def q4_1_engine(a: torch.Tensor, w_blocks: torch.Tensor, k: int, *, out_dtype: torch.dtype = torch.float32,
                engine: str = "auto") -> int:
    """Engine code nnb200_linear_q4_1 would pick (1 fused GEMM, 3 GEMV on CUDA cores, 4 GEMV with warp
    MMA, 5 two-pass GEMM) when given the scratch it asks for."""
    n_out = w_blocks.n if isinstance(w_blocks, PackedQ41) else w_blocks.shape[0]
    out = torch.empty((a.shape[0], n_out), dtype=out_dtype, device=a.device)
    args = q4_1_args(a, w_blocks, out, k, engine=engine)
    need = capi.lib().nnb200_q4_1_workspace_bytes(C.byref(args))
    if need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
        args.workspace = scratch.data_ptr()
        args.workspace_bytes = need
    return capi.lib().nnb200_q4_1_engine(C.byref(args))


def q4_1_decode(w_blocks: torch.Tensor, k: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    out = torch.empty((w_blocks.shape[0], k), dtype=out_dtype, device=w_blocks.device)
    with torch.cuda.device(w_blocks.device):
        capi.check(capi.lib().nnb200_q4_1_decode(w_blocks.data_ptr(), w_blocks.stride(0) // 20, w_blocks.shape[0], k,
                                                 out.data_ptr(), int(out_dtype == torch.float16), out.stride(0),
                                                 _stream_ptr(w_blocks.device)), "nnb200_q4_1_decode")
    return out


def _quant_view(shape, axis: int, param_count: int) -> tuple[int, int, int]:
    """[outer][rows][inner] of a dense tensor: one parameter = per tensor; axis < 0 = one per
    innermost row; else one per index along ``axis`` (the operator's granularity rule,
    reference include/nnops/ops/quant_linear.hpp:38-45)."""
    shape = tuple(int(s) for s in shape)
    numel = math.prod(shape)
    if param_count <= 1:
        return 1, 1, numel
    if axis < 0:
        return 1, numel // shape[-1] if shape[-1] else 0, shape[-1]
    return math.prod(shape[:axis]), shape[axis], math.prod(shape[axis + 1:])


def _quant_params(scale, zero_point, device):
    scale = torch.as_tensor(scale, dtype=torch.float32).reshape(-1).to(device).contiguous()
    zero_point = torch.as_tensor(zero_point).reshape(-1).to(device).contiguous()
    if zero_point.dtype not in (torch.int8, torch.uint8) or zero_point.numel() != scale.numel():
        raise ValueError("zero_point must be int8/uint8 with one entry per scale")
    return scale, zero_point


def quantize_linear(x: torch.Tensor, scale, zero_point, *, axis: int = -1, out_dtype: torch.dtype = torch.int8,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """QuantizeLinear on the GPU: f32/f16 -> s8/u8."""
    if x.dtype not in (torch.float32, torch.float16) or not x.is_contiguous():
        raise ValueError("x must be a contiguous f32/f16 tensor")
    scale, zero_point = _quant_params(scale, zero_point, x.device)
    y = out if out is not None else torch.empty(x.shape, dtype=out_dtype, device=x.device)
    outer, rows, inner = _quant_view(x.shape, axis, scale.numel())
    if rows != scale.numel():
        raise ValueError("scale count does not match the tensor and axis")
    args = capi.QuantLinearArgs(x=x.data_ptr(), y=y.data_ptr(), outer=outer, rows=rows, inner=inner,
                                scale=scale.data_ptr(), zero_point=zero_point.data_ptr(),
                                zp_unsigned=int(zero_point.dtype == torch.uint8),
                                float_f16=int(x.dtype == torch.float16), int_unsigned=int(y.dtype == torch.uint8))
    with torch.cuda.device(x.device):
        capi.check(capi.lib().nnb200_quantize_linear(C.byref(args), _stream_ptr(x.device)), "nnb200_quantize_linear")
    return y


def dequantize_linear(x: torch.Tensor, scale, zero_point, *, axis: int = -1, out_dtype: torch.dtype = torch.float32,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """DequantizeLinear on the GPU: s8/u8 -> f32/f16."""
    if x.dtype not in (torch.int8, torch.uint8) or not x.is_contiguous():
        raise ValueError("x must be a contiguous int8/uint8 tensor")
    scale, zero_point = _quant_params(scale, zero_point, x.device)
    y = out if out is not None else torch.empty(x.shape, dtype=out_dtype, device=x.device)
    outer, rows, inner = _quant_view(x.shape, axis, scale.numel())
    if rows != scale.numel():
        raise ValueError("scale count does not match the tensor and axis")
    args = capi.QuantLinearArgs(x=x.data_ptr(), y=y.data_ptr(), outer=outer, rows=rows, inner=inner,
                                scale=scale.data_ptr(), zero_point=zero_point.data_ptr(),
                                zp_unsigned=int(zero_point.dtype == torch.uint8),
                                float_f16=int(y.dtype == torch.float16), int_unsigned=int(x.dtype == torch.uint8))
    with torch.cuda.device(x.device):
        capi.check(capi.lib().nnb200_dequantize_linear(C.byref(args), _stream_ptr(x.device)),
                   "nnb200_dequantize_linear")
    return y


def linear_fp_act(a: torch.Tensor, w: torch.Tensor, *, scale_a, zp_a=0, act_dtype: torch.dtype = torch.int8, **kw):
    """f32/f16 activations carrying quantization parameters x s8 weights [N,K] -> a's dtype:
    the same two C-ABI calls the C++ backend glue makes for this route (quantise A with its
    per-tensor / per-token scale and int32 zero point, then the int8 matmul with the
    dequantizing epilogue).  ``scale_a`` / ``zp_a`` are scalars or per-row arrays."""
    if a.dim() != 2 or a.dtype not in (torch.float32, torch.float16) or not a.is_contiguous():
        raise ValueError("a must be a contiguous 2-D f32/f16 tensor")
    m, k = a.shape
    per_token = not (isinstance(scale_a, (int, float)) and isinstance(zp_a, int))
    count = m if per_token else 1
    scale = torch.as_tensor(scale_a, dtype=torch.float32).reshape(-1).to(a.device).expand(count).contiguous()
    zp = torch.as_tensor(zp_a, dtype=torch.int32).reshape(-1).to(a.device).expand(count).contiguous()
    aq = torch.empty((m, k), dtype=act_dtype, device=a.device)
    outer, rows, inner = (1, m, k) if per_token else (1, 1, m * k)
    args = capi.QuantLinearArgs(x=a.data_ptr(), y=aq.data_ptr(), outer=outer, rows=rows, inner=inner,
                                scale=scale.data_ptr(), zero_point=zp.data_ptr(), zp_unsigned=capi.ZP_S32,
                                float_f16=int(a.dtype == torch.float16), int_unsigned=int(act_dtype == torch.uint8))
    with torch.cuda.device(a.device):
        capi.check(capi.lib().nnb200_quantize_linear(C.byref(args), _stream_ptr(a.device)), "nnb200_quantize_linear")
    out_kind = "f32" if a.dtype == torch.float32 else "f16"
    return gemm_i8(aq, w, out_kind=out_kind, scale_a=scale if per_token else float(scale_a),
                   zp_a=zp if per_token else int(zp_a), **kw)


class PackedConvI8:
    """The k-major filter blob of nnb200_conv2d_i8_pack and the geometry it was cut for."""

    def __init__(self, blob: torch.Tensor, kh: int, kw: int, icg: int, oc: int, groups: int):
        self.blob, self.kh, self.kw, self.icg, self.oc, self.groups = blob, kh, kw, icg, oc, groups


def prepack_conv2d_i8(w: torch.Tensor, groups: int = 1) -> PackedConvI8:
    """w: s8 HWIO [KH, KW, IC/G, OC] (any strides) on the device."""
    if not w.is_cuda or w.dtype != torch.int8 or w.dim() != 4:
        raise RuntimeError("prepack_conv2d_i8 needs a CUDA s8 HWIO filter")
    kh, kw, icg, oc = w.shape
    lib = capi.lib()
    blob = torch.empty(lib.nnb200_conv2d_i8_pack_bytes(kh, kw, icg, oc), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        capi.check(lib.nnb200_conv2d_i8_pack(w.data_ptr(), w.stride(0), w.stride(1), w.stride(2), w.stride(3), kh, kw,
                                             icg, oc, groups, blob.data_ptr(), _stream_ptr(w.device)),
                   "nnb200_conv2d_i8_pack")
    return PackedConvI8(blob, kh, kw, icg, oc, groups)


def conv2d_out_hw(ih, iw, kh, kw, stride=(1, 1), dilation=(1, 1), padding=(0, 0)):
    oh = (ih + 2 * padding[0] - ((kh - 1) * dilation[0] + 1)) // stride[0] + 1
    ow = (iw + 2 * padding[1] - ((kw - 1) * dilation[1] + 1)) // stride[1] + 1
    return oh, ow


def conv2d_i8(x: torch.Tensor, w, *, stride=(1, 1), dilation=(1, 1), padding=(0, 0), groups: int = 1,
              out_kind: str = "s8", out: torch.Tensor | None = None, bias=None, relu=False, activation="none",
              act_alpha=0.0, act_beta=1.0, min_clip=-math.inf, max_clip=math.inf, scale_x=1.0, zp_x=0, scale_w=1.0,
              zp_w=0, out_scale=1.0, out_zp=0, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """int8 Conv2D on the current CUDA stream: x [N, IH, IW, IC] u8/s8 (NHWC, any strides), w an s8 HWIO filter
    [KH, KW, IC/G, OC] or a PackedConvI8; returns [N, OH, OW, OC]."""
    if not x.is_cuda:
        raise RuntimeError("nnops_b200.conv2d_i8 needs CUDA tensors; there is no CPU path")
    dev = x.device
    packed = isinstance(w, PackedConvI8)
    n, ih, iw, ic = x.shape
    if packed:
        kh, kw, icg, oc = w.kh, w.kw, w.icg, w.oc
    else:
        kh, kw, icg, oc = w.shape
    oh, ow = conv2d_out_hw(ih, iw, kh, kw, stride, dilation, padding)
    if out is None:
        out = torch.empty((n, oh, ow, oc), dtype=_OUT_TORCH[out_kind], device=dev)
    keep: list = []
    sw, sw0 = _dev_array(scale_w, torch.float32, dev, oc)
    zw, zw0 = _dev_array(zp_w, torch.int32, dev, oc)
    if bias is not None:
        bdt = torch.int32 if out_kind in ("s8", "u8") else _OUT_TORCH[out_kind]
        bias = torch.as_tensor(bias).to(device=dev, dtype=bdt).contiguous()
    args = capi.Conv2dI8Args(
        input=x.data_ptr(), weight=w.blob.data_ptr() if packed else w.data_ptr(), out=out.data_ptr(),
        batch=n, ih=ih, iw=iw, ic=ic, oh=oh, ow=ow, oc=oc, kh=kh, kw=kw, stride_h=stride[0], stride_w=stride[1],
        dil_h=dilation[0], dil_w=dilation[1], pad_h=padding[0], pad_w=padding[1], groups=groups,
        in_stride_n=x.stride(0), in_stride_h=x.stride(1), in_stride_w=x.stride(2), in_stride_c=x.stride(3),
        w_stride_kh=0 if packed else w.stride(0), w_stride_kw=0 if packed else w.stride(1),
        w_stride_ic=0 if packed else w.stride(2), w_stride_oc=0 if packed else w.stride(3),
        out_stride_n=out.stride(0), out_stride_h=out.stride(1), out_stride_w=out.stride(2),
        weight_packed=int(packed), a_unsigned=int(x.dtype == torch.uint8), out_kind=capi.OUT_KINDS[out_kind],
        bias=bias.data_ptr() if bias is not None else None, relu=int(bool(relu)),
        activation=capi.ACTIVATIONS[activation], act_alpha=act_alpha, act_beta=act_beta, min_clip=min_clip,
        max_clip=max_clip, scale_w=sw.data_ptr() if sw is not None else None,
        zp_w=zw.data_ptr() if zw is not None else None, scale_x=float(scale_x),
        scale_w_scalar=1.0 if sw0 is None else float(sw0), zp_x=int(zp_x), zp_w_scalar=0 if zw0 is None else int(zw0),
        zp_w_nonzero=int(zw is not None and bool((zw != 0).any().item())), out_scale=float(out_scale),
        out_zp=int(out_zp), workspace=None, workspace_bytes=0)
    need = capi.lib().nnb200_conv2d_i8_workspace_bytes(C.byref(args))
    if need:
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        keep.append(workspace)
        args.workspace = workspace.data_ptr()
        args.workspace_bytes = workspace.numel()
    with torch.cuda.device(dev):
        capi.check(capi.lib().nnb200_conv2d_i8(C.byref(args), _stream_ptr(dev)), "nnb200_conv2d_i8")
    return out
