"""ctypes bindings of libnnb200's C ABI (include/nnb200.h).

Loading fails loudly when the library has not been built: there is no CPU or PyTorch
fallback for any call here.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libnnb200.so"

OK, INVALID_ARGUMENT, UNSUPPORTED, NOT_INITIALIZED, OUT_OF_MEMORY, INTERNAL = range(6)
STATUS_NAMES = ["ok", "invalid_argument", "unsupported", "not_initialized", "out_of_memory", "internal"]
OUT_KINDS = {"s32": 0, "s8": 1, "u8": 2, "f32": 3, "f16": 4}
ACTIVATIONS = {"none": 0, "relu": 1, "gelu": 2, "sigmoid": 3, "tanh": 4, "leaky_relu": 5, "silu": 6,
               "hard_swish": 7, "elu": 8, "relu6": 9}
ENGINES = {"auto": 0, "umma": 1, "narrow": 2, "generic": 3, "decode": 4, "skinny": 5}
ENGINE_NAMES = {v: k for k, v in ENGINES.items()}
Q4_ENGINES = {"auto": 0, "gemm": 1, "gemv": 2, "gemv_simt": 3, "gemv_mma": 4, "gemm_two_pass": 5, "gemv_dsq": 6}
STATIC_SCRATCH_BYTES = 1 << 20
# Measurement / test switches (NNB200_KNOB_* in nnb200.h); process-wide, negative = default.
KNOBS = {"group_m": 0, "i8_bn": 1, "i8_pair": 2, "i8_peer_staging": 3, "f16_pair": 4, "i8_share_k": 5, "q4_gemv": 6,
         "conv_form": 7, "i8_k_rotate": 8}


class GemmI8Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a_stride_m", C.c_int64), ("a_stride_k", C.c_int64),
        ("w_stride_n", C.c_int64), ("w_stride_k", C.c_int64),
        ("ldc", C.c_int64), ("batch", C.c_int64),
        ("a_batch_stride", C.c_int64), ("w_batch_stride", C.c_int64), ("out_batch_stride", C.c_int64),
        ("a_unsigned", C.c_int32), ("out_kind", C.c_int32),
        ("bias", C.c_void_p),
        ("relu", C.c_int32), ("activation", C.c_int32),
        ("act_alpha", C.c_float), ("act_beta", C.c_float),
        ("min_clip", C.c_float), ("max_clip", C.c_float),
        ("scale_a", C.c_void_p), ("scale_w", C.c_void_p), ("zp_a", C.c_void_p), ("zp_w", C.c_void_p),
        ("scale_a_scalar", C.c_float), ("scale_w_scalar", C.c_float),
        ("zp_a_scalar", C.c_int32), ("zp_w_scalar", C.c_int32),
        ("zp_a_nonzero", C.c_int32), ("zp_w_nonzero", C.c_int32),
        ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("force_engine", C.c_int32),
        ("num_peer_outs", C.c_int32), ("peer_out", C.c_void_p * 7),
        ("r_w", C.c_void_p),
        ("multicast_out", C.c_void_p),
    ]


class Q41Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("w_blocks", C.c_void_p), ("out", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("lda", C.c_int64), ("ldw_blocks", C.c_int64), ("ldc", C.c_int64),
        ("a_f16", C.c_int32), ("out_f16", C.c_int32),
        ("bias", C.c_void_p),
        ("activation", C.c_int32),
        ("act_alpha", C.c_float), ("act_beta", C.c_float),
        ("min_clip", C.c_float), ("max_clip", C.c_float),
        ("alpha", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("force_engine", C.c_int32), ("flags", C.c_int32),
        ("w_dm", C.c_void_p), ("ld_dm", C.c_int64),
    ]


Q4_FLAG_OVERLAP_PREVIOUS = 1

# Every symbol include/nnb200.h declares: (name, restype, argtypes).
ZP_S8, ZP_U8, ZP_S32 = 0, 1, 2   # nnb200_quant_linear_args.zp_unsigned: storage type of the zero points


class I8Packed(C.Structure):
    """Mirror of nnb200_i8_packed: the sections of a packed int8 weight."""
    _fields_ = [("w", C.c_void_p), ("pitch", C.c_int64), ("scale_w", C.c_void_p), ("zp_w", C.c_void_p),
                ("r_w", C.c_void_p)]


class Q41Packed(C.Structure):
    """Mirror of nnb200_q4_1_packed: the two planes of a packed Q4_1 weight."""
    _fields_ = [("qs", C.c_void_p), ("qs_pitch", C.c_int64), ("dm", C.c_void_p), ("dm_pitch", C.c_int64)]


class QuantLinearArgs(C.Structure):
    """Mirror of nnb200_quant_linear_args."""
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p),
        ("outer", C.c_int64), ("rows", C.c_int64), ("inner", C.c_int64),
        ("scale", C.c_void_p), ("zero_point", C.c_void_p),
        ("zp_unsigned", C.c_int32), ("float_f16", C.c_int32), ("int_unsigned", C.c_int32),
    ]


class Conv2dI8Args(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("weight", C.c_void_p), ("out", C.c_void_p),
        ("batch", C.c_int64), ("ih", C.c_int64), ("iw", C.c_int64), ("ic", C.c_int64),
        ("oh", C.c_int64), ("ow", C.c_int64), ("oc", C.c_int64),
        ("kh", C.c_int64), ("kw", C.c_int64), ("stride_h", C.c_int64), ("stride_w", C.c_int64),
        ("dil_h", C.c_int64), ("dil_w", C.c_int64), ("pad_h", C.c_int64), ("pad_w", C.c_int64), ("groups", C.c_int64),
        ("in_stride_n", C.c_int64), ("in_stride_h", C.c_int64), ("in_stride_w", C.c_int64), ("in_stride_c", C.c_int64),
        ("w_stride_kh", C.c_int64), ("w_stride_kw", C.c_int64), ("w_stride_ic", C.c_int64), ("w_stride_oc", C.c_int64),
        ("out_stride_n", C.c_int64), ("out_stride_h", C.c_int64), ("out_stride_w", C.c_int64),
        ("weight_packed", C.c_int32), ("a_unsigned", C.c_int32), ("out_kind", C.c_int32),
        ("bias", C.c_void_p), ("relu", C.c_int32), ("activation", C.c_int32),
        ("act_alpha", C.c_float), ("act_beta", C.c_float), ("min_clip", C.c_float), ("max_clip", C.c_float),
        ("scale_w", C.c_void_p), ("zp_w", C.c_void_p),
        ("scale_x", C.c_float), ("scale_w_scalar", C.c_float), ("zp_x", C.c_int32), ("zp_w_scalar", C.c_int32),
        ("zp_w_nonzero", C.c_int32), ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


SYMBOLS = [
    ("nnb200_gemm_i8_workspace_bytes", C.c_size_t, [C.POINTER(GemmI8Args)]),
    ("nnb200_gemm_i8_min_workspace_bytes", C.c_size_t, [C.POINTER(GemmI8Args)]),
    ("nnb200_gemm_i8", C.c_int, [C.POINTER(GemmI8Args), C.c_void_p]),
    ("nnb200_gemm_i8_static_scratch", C.c_int, [C.POINTER(GemmI8Args), C.c_void_p]),
    ("nnb200_gemm_i8_engine", C.c_int, [C.POINTER(GemmI8Args)]),
    ("nnb200_q4_1_workspace_bytes", C.c_size_t, [C.POINTER(Q41Args)]),
    ("nnb200_linear_q4_1", C.c_int, [C.POINTER(Q41Args), C.c_void_p]),
    ("nnb200_q4_1_engine", C.c_int, [C.POINTER(Q41Args)]),
    ("nnb200_q4_1_decode", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32,
                                     C.c_int64, C.c_void_p]),
    ("nnb200_i8_pack_bytes", C.c_size_t, [C.c_int64, C.c_int64]),
    ("nnb200_i8_pack", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_float,
                                 C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("nnb200_i8_packed_view", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.POINTER(I8Packed)]),
    ("nnb200_q4_1_pack_bytes", C.c_size_t, [C.c_int64, C.c_int64]),
    ("nnb200_q4_1_pack", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("nnb200_q4_1_packed_view", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.POINTER(Q41Packed)]),
    ("nnb200_conv2d_i8_workspace_bytes", C.c_size_t, [C.POINTER(Conv2dI8Args)]),
    ("nnb200_conv2d_i8", C.c_int, [C.POINTER(Conv2dI8Args), C.c_void_p]),
    ("nnb200_conv2d_i8_pack_bytes", C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    ("nnb200_conv2d_i8_pack", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    ("nnb200_quantize_linear", C.c_int, [C.POINTER(QuantLinearArgs), C.c_void_p]),
    ("nnb200_dequantize_linear", C.c_int, [C.POINTER(QuantLinearArgs), C.c_void_p]),
    ("nnb200_interleave_shards", C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int64,
                                           C.c_void_p]),
    ("nnb200_rank_barrier", C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int64, C.c_void_p]),
    ("nnb200_take_device_error", C.c_int, [C.POINTER(C.c_int32)]),
    ("nnb200_selftest_wait_limit", C.c_int, [C.c_int64, C.c_void_p]),
    ("nnb200_copy_h2d_async", C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("nnb200_scratch_alloc_async", C.c_int, [C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p]),
    ("nnb200_scratch_free_async", C.c_int, [C.c_void_p, C.c_void_p]),
    ("nnb200_peer_buffer_alloc", C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    ("nnb200_peer_buffer_free", C.c_int, [C.c_void_p]),
    ("nnb200_peer_buffer_export", C.c_int, [C.c_void_p, C.c_char_p]),
    ("nnb200_peer_buffer_open", C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    ("nnb200_peer_buffer_close", C.c_int, [C.c_void_p]),
    ("nnb200_enable_peer_access", C.c_int, [C.c_int32]),
    ("nnb200_is_device_pointer", C.c_int, [C.c_void_p]),
    ("nnb200_measure_i8_mma_peak", C.c_int, [C.c_int32, C.c_int32, C.POINTER(C.c_double), C.c_void_p]),
    ("nnb200_set_knob", C.c_int, [C.c_int, C.c_int]),
    ("nnb200_get_knob", C.c_int, [C.c_int]),
    ("nnb200_launch_count", C.c_uint64, []),
    ("nnb200_version", C.c_char_p, []),
]

_lib = None


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built (python -m nnops_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nnops_b200.build` "
                "(the CUDA library is the only implementation; there is no fallback)")
        l = C.CDLL(str(LIB_PATH))
        for name, res, args in SYMBOLS:
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


class Nnb200Error(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{what}: {name}")


def check(status: int, what: str) -> None:
    if status != OK:
        raise Nnb200Error(status, what)


def set_knob(name: str, value: int) -> int:
    """Set a measurement switch; returns the previous value (-1 = default)."""
    return lib().nnb200_set_knob(KNOBS[name], int(value))


def take_device_error() -> int:
    code = C.c_int32(0)
    check(lib().nnb200_take_device_error(C.byref(code)), "nnb200_take_device_error")
    return code.value


DEVICE_ERROR_SELFTEST = 7
DEVICE_ERROR_PEER_WAIT = 8
RANK_FLAG_BYTES = 64


def selftest_wait_limit(limit_cycles: int = 2_000_000, stream=None) -> None:
    """Launch the wait self-test: its barrier wait runs out and records DEVICE_ERROR_SELFTEST."""
    check(lib().nnb200_selftest_wait_limit(int(limit_cycles), stream), "nnb200_selftest_wait_limit")
