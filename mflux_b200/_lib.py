"""ctypes binding of libmfx.so, the C-ABI library declared in include/mfx.h.

There is no fallback: if the shared library has not been built (python -m mflux_b200.build) every
operation raises. Status codes are turned into ValueError (caller mistakes: shapes, dtypes,
alignment) or RuntimeError (device / CUDA failures), mirroring how the reference surfaces MLX
errors as Python exceptions.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmfx.so"

# mfx_dtype
F32, BF16, F16 = 0, 1, 2
# mfx_qmode
QMODE_MLX, QMODE_DOC = 0, 1
# mfx_epilogue
EPI_NONE, EPI_GELU_ERF, EPI_GELU_TANH, EPI_GATE_RESIDUAL, EPI_SILU, EPI_SWIGLU, EPI_PEER_SCATTER = 0, 1, 2, 3, 4, 5, 6
TP_MAX_WORLD = 8

_VALUE_ERRORS = {-1, -2, -3, -4, -7, -9}
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024


class TpScatter(ctypes.Structure):
    """struct mfx_tp_scatter (include/mfx.h)."""

    _fields_ = [
        ("world", c_int),
        ("rank", c_int),
        ("rows_per_rank", c_int64),
        ("row_offset", c_int64),
        ("D", c_int64),
        ("dst", c_void_p * TP_MAX_WORLD),
        ("flags", c_void_p * TP_MAX_WORLD),
        ("done_counter", c_void_p),
    ]


class TpFuseArgs(ctypes.Structure):
    """struct mfx_tp_fuse_args (include/mfx.h)."""

    _fields_ = [
        ("world", c_int),
        ("rank", c_int),
        ("batch", c_int64),
        ("rows_per_rank", c_int64),
        ("seq_pad", c_int64),
        ("seq", c_int64),
        ("split", c_int64),
        ("D", c_int64),
        ("x", c_void_p),
        ("partials", c_void_p),
        ("rs_flags", c_void_p),
        ("rs_target", c_int),
        ("epoch_base", c_void_p),
        ("bias", c_void_p * 2),
        ("bias_dtype", c_int),
        ("gate", c_void_p * 2),
        ("shift", c_void_p * 2),
        ("scale", c_void_p * 2),
        ("mod_dtype", c_int),
        ("mod_batch_stride", c_int64),
        ("eps", ctypes.c_float),
        ("push_dst", c_void_p * TP_MAX_WORLD),
        ("ag_flags", c_void_p * TP_MAX_WORLD),
        ("done_counter", c_void_p),
        ("push_local_only", c_int),
    ]


class FmhaArgs(ctypes.Structure):
    """struct mfx_fmha_args (include/mfx.h)."""

    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("q_row_stride", c_int64),
        ("q_batch_stride", c_int64),
        ("kv_row_stride", c_int64),
        ("kv_batch_stride", c_int64),
        ("seq_q", c_int64),
        ("seq_kv", c_int64),
        ("batch", c_int64),
        ("heads", c_int),
        ("kv_heads", c_int),
        ("scale", ctypes.c_float),
        ("key_bias", c_void_p),
        ("bias_batch_stride", c_int64),
        ("out", c_void_p),
        ("out_row_stride", c_int64),
        ("out_batch_stride", c_int64),
    ]


class QLinearArgs(ctypes.Structure):
    """struct mfx_qlinear_args (include/mfx.h)."""

    _fields_ = [
        ("x", c_void_p),
        ("x_row_stride", c_int64),
        ("x_batch_stride", c_int64),
        ("rows", c_int64),
        ("batch", c_int64),
        ("K", c_int64),
        ("N", c_int64),
        ("wq", c_void_p),
        ("scales", c_void_p),
        ("biases", c_void_p),
        ("sb_dtype", c_int),
        ("bits", c_int),
        ("group_size", c_int),
        ("prepared", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("bias", c_void_p),
        ("bias_dtype", c_int),
        ("epilogue", c_int),
        ("gate", c_void_p),
        ("gate_dtype", c_int),
        ("gate_batch_stride", c_int64),
        ("residual", c_void_p),
        ("res_row_stride", c_int64),
        ("res_batch_stride", c_int64),
        ("y", c_void_p),
        ("y_dtype", c_int),
        ("y_row_stride", c_int64),
        ("y_batch_stride", c_int64),
        ("lora_t", c_void_p),
        ("lora_t_row_stride", c_int64),
        ("lora_t_batch_stride", c_int64),
        ("lora_b", c_void_p),
        ("lora_ld", c_int64),
        ("lora_r", c_int64),
        ("scatter", ctypes.POINTER(TpScatter)),
    ]


class NormArgs(ctypes.Structure):
    """struct mfx_norm_args (include/mfx.h)."""

    _fields_ = [
        ("x", c_void_p),
        ("x_dtype", c_int),
        ("x_row_stride", c_int64),
        ("x_batch_stride", c_int64),
        ("rows", c_int64),
        ("batch", c_int64),
        ("D", c_int64),
        ("shift", c_void_p),
        ("scale", c_void_p),
        ("mod_dtype", c_int),
        ("mod_batch_stride", c_int64),
        ("weight", c_void_p),
        ("weight_dtype", c_int),
        ("eps", ctypes.c_float),
        ("rms", c_int),
        ("y", c_void_p),
        ("y_row_stride", c_int64),
        ("y_batch_stride", c_int64),
    ]


# name -> (restype, argtypes); every symbol include/mfx.h declares
class PostPreNormArgs(ctypes.Structure):
    """struct mfx_post_pre_norm_args (include/mfx.h)."""

    _fields_ = [
        ("y", c_void_p),
        ("y_dtype", c_int),
        ("y_row_stride", c_int64),
        ("y_batch_stride", c_int64),
        ("rows", c_int64),
        ("batch", c_int64),
        ("D", c_int64),
        ("weight", c_void_p),
        ("weight_dtype", c_int),
        ("eps", ctypes.c_float),
        ("gate", c_void_p),
        ("gate_dtype", c_int),
        ("gate_batch_stride", c_int64),
        ("residual", c_void_p),
        ("res_row_stride", c_int64),
        ("res_batch_stride", c_int64),
        ("next_out", c_void_p),
        ("next_row_stride", c_int64),
        ("next_batch_stride", c_int64),
        ("next_weight", c_void_p),
        ("next_weight_dtype", c_int),
        ("next_scale", c_void_p),
        ("next_scale_dtype", c_int),
        ("next_scale_batch_stride", c_int64),
        ("next_eps", ctypes.c_float),
    ]


SIGNATURES = {
    "mfx_version": (c_int, []),
    "mfx_status_str": (c_char_p, [c_int]),
    "mfx_last_cuda_error": (c_char_p, []),
    "mfx_poll_device_status": (c_int, [ctypes.POINTER(c_int), c_void_p]),
    "mfx_quantize_affine": (
        c_int,
        [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "mfx_dequantize_affine": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_int, c_void_p],
    ),
    "mfx_qlinear_prepared_bytes": (ctypes.c_size_t, [c_int64, c_int64, c_int, c_int]),
    "mfx_qlinear_prepare": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, ctypes.c_size_t, c_void_p],
    ),
    "mfx_qlinear": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
         c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p, ctypes.c_size_t, c_void_p],
    ),
    "mfx_qlinear_static_scratch": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
         c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p],
    ),
    "mfx_qlinear_ex": (c_int, [ctypes.POINTER(QLinearArgs), c_void_p]),
    "mfx_norm_modulate": (c_int, [ctypes.POINTER(NormArgs), c_void_p]),
    "mfx_qknorm_rope": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
         c_void_p, ctypes.c_float, c_void_p],
    ),
    "mfx_qknorm_rope_gqa": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_void_p, ctypes.c_float, c_void_p],
    ),
    "mfx_act_mul": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                            c_void_p]),
    "mfx_fmha": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, ctypes.c_float, c_void_p, c_int64,
         c_int64, c_void_p],
    ),
    "mfx_fmha_ex": (c_int, [ctypes.POINTER(FmhaArgs), c_void_p]),
    "mfx_fmha_bias": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, ctypes.c_float, c_void_p, c_int64,
         c_void_p, c_int64, c_int64, c_void_p],
    ),
    "mfx_tp_fuse": (c_int, [ctypes.POINTER(TpFuseArgs), c_void_p]),
    "mfx_tp_signal": (c_int, [ctypes.POINTER(c_void_p), c_int, c_void_p]),
    "mfx_tp_wait": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "mfx_vec_sum_act": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int64, c_void_p]),
    "mfx_gate_residual": (
        c_int,
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64,
         c_int64, c_int64, c_void_p],
    ),
    "mfx_norm_gate_residual": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int,
                                       ctypes.c_float, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int64,
                                       c_void_p]),
    "mfx_post_pre_norm": (c_int, [ctypes.POINTER(PostPreNormArgs), c_void_p]),
    "mfx_cfg_combine": (c_int, [c_void_p, c_void_p, c_int, ctypes.c_float, c_int, c_void_p, c_int64, c_int64, c_void_p]),
    "mfx_euler_step": (c_int, [c_void_p, c_int, c_void_p, c_int, ctypes.c_float, c_void_p, c_int64, c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load libmfx.so once; raise loudly when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m mflux_b200.build` (needs nvcc; no GPU needed to build). There is no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Raise the Python exception that corresponds to a negative mfx_status."""
    if status == 0:
        return
    lib = load()
    msg = lib.mfx_status_str(status).decode()
    detail = lib.mfx_last_cuda_error().decode() if status == -6 else ""
    text = f"{what}: {msg}" + (f" [{detail}]" if detail else "")
    if status in _VALUE_ERRORS:
        raise ValueError(text)
    raise RuntimeError(text)
