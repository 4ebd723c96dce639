"""NumPy restatement of MLX's group-wise affine quantizer and quantized linear layer.

Test infrastructure (see oracle/__init__.py): parity unpinned, MLX itself is not available.

Reference call sites this follows:
  * src/mflux/models/common/weights/loading/weight_applier.py:93-103 -> mlx.nn.quantize(model,
    class_predicate, bits) -> Linear.to_quantized -> mx.quantize(weight, group_size=64, bits)
  * src/mflux/models/common/lora/layer/linear_lora_layer.py:14-16 (packed shape: the input
    dimension equals weight.shape[1] * 32 / bits)
  * every nn.Linear of the transformer blocks, executed as
    mx.quantized_matmul(x, w, scales, biases, transpose=True, group_size=64, bits) + bias

Two quantizer modes are restated:
  "mlx"  the algorithm MLX ships (affine mode): per group of `group_size` values along the input
         dimension take w_min/w_max, scale = max((w_max - w_min) / (2^bits - 1), 1e-7), orient the
         scale so that the extreme with the larger magnitude ("edge") maps to code 0, then snap
         scale to edge / rint(edge / scale) so that 0.0 is exactly representable; bias = edge
         (or 0 with the unsnapped scale when rint(edge/scale) == 0). All in float32; scales and
         biases are stored in the dtype of w.
  "doc"  the formula in MLX's documentation: scale = (max - min) /
         (2^bits - 1), bias = min.
Codes: q = clip(rint((w - bias) / scale), 0, 2^bits - 1) with the float32 (unrounded) scale and
bias, round-half-to-even, packed little-end first: code j of a row occupies bits [j*bits, (j+1)*bits) of the
row's bit stream, which is then read as uint32 words. For 4 and 8 bits a word holds 8 / 4 whole codes; for 3, 5
and 6 bits (the other widths of the reference's CLI, src/mflux/cli/defaults/defaults.py:63) MLX packs 8 codes
into 3 or 5 bytes and 4 codes into 3 bytes, the same bit stream.
"""
from __future__ import annotations

import numpy as np

EPS = np.float32(1e-7)
BITS = (3, 4, 5, 6, 8)


def pack_codes(q: np.ndarray, bits: int) -> np.ndarray:
    """Integer codes [N, K] -> uint32 [N, K*bits/32], little-end-first bit stream per row."""
    n, k = q.shape
    q = q.astype(np.uint32)
    if 32 % bits == 0:
        per = 32 // bits
        shifts = (np.arange(per, dtype=np.uint32) * np.uint32(bits)).astype(np.uint32)
        return np.bitwise_or.reduce(q.reshape(n, k // per, per) << shifts, axis=-1).astype(np.uint32)
    stream = ((q[..., None] >> np.arange(bits, dtype=np.uint32)) & np.uint32(1)).astype(np.uint8)   # [N, K, bits]
    stream = stream.reshape(n, k * bits // 32, 32).astype(np.uint32)
    return np.bitwise_or.reduce(stream << np.arange(32, dtype=np.uint32), axis=-1).astype(np.uint32)


def _as_f32(a) -> np.ndarray:
    """float32 view of a numpy array or torch tensor (bf16 tensors are widened exactly)."""
    if hasattr(a, "detach"):
        import torch

        return a.detach().to(torch.float32).cpu().numpy()
    return np.asarray(a, dtype=np.float32)


def round_to_dtype(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to `dtype` ("f32" | "bf16" | "f16") and return them as float32."""
    a = np.asarray(a, dtype=np.float32)
    if dtype == "f32":
        return a
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32).astype(np.uint64)
        lsb = (u >> 16) & 1
        r = ((u + 0x7FFF + lsb) >> 16) << 16
        out = r.astype(np.uint32).view(np.float32)
        return np.where(np.isfinite(a), out, a)
    raise ValueError(dtype)


def quantize_affine(w, group_size: int = 64, bits: int = 4, mode: str = "mlx", dtype: str = "f32"):
    """Quantize W[N, K] row-wise in groups of `group_size` along K.

    Returns (packed uint32 [N, K*bits/32], scales f32 [N, K/group], biases f32 [N, K/group]);
    scales/biases hold values already rounded to `dtype`, the storage dtype of w.
    """
    w = _as_f32(w)
    if w.ndim != 2:
        raise ValueError("w must be [N, K]")
    n, k = w.shape
    if bits not in BITS:
        raise ValueError(f"bits must be one of {BITS}")
    if k % group_size != 0:
        raise ValueError("K must be a multiple of the group size")
    nb = np.float32((1 << bits) - 1)
    g = w.reshape(n, k // group_size, group_size)
    w_max = g.max(axis=-1)
    w_min = g.min(axis=-1)
    with np.errstate(divide="ignore", invalid="ignore"):
        if mode == "mlx":
            scale = np.maximum((w_max - w_min) / nb, EPS).astype(np.float32)
            side = np.abs(w_min) > np.abs(w_max)
            scale = np.where(side, scale, -scale).astype(np.float32)
            edge = np.where(side, w_min, w_max).astype(np.float32)
            q0 = np.rint(edge / scale).astype(np.float32)
            snapped = (edge / np.where(q0 == 0, np.float32(1), q0)).astype(np.float32)
            scale = np.where(q0 == 0, scale, snapped).astype(np.float32)
            bias = np.where(q0 == 0, np.float32(0), edge).astype(np.float32)
        elif mode == "doc":
            scale = ((w_max - w_min) / nb).astype(np.float32)
            bias = w_min.astype(np.float32)
        else:
            raise ValueError(mode)
        q = np.rint((g - bias[..., None]) / scale[..., None])
    q = np.where(np.isfinite(q), q, 0.0)  # constant group in "doc" mode: scale == 0 -> code 0
    q = np.clip(q, 0, nb).astype(np.uint32).reshape(n, k)
    return pack_codes(q, bits), round_to_dtype(scale, dtype), round_to_dtype(bias, dtype)


def unpack_codes(packed: np.ndarray, bits: int) -> np.ndarray:
    """uint32 [N, K*bits/32] -> integer codes [N, K]."""
    packed = np.asarray(packed, dtype=np.uint32)
    if 32 % bits == 0:
        per = 32 // bits
        shifts = (np.arange(per, dtype=np.uint32) * np.uint32(bits)).astype(np.uint32)
        q = (packed[..., None] >> shifts) & np.uint32((1 << bits) - 1)
        return q.reshape(packed.shape[0], -1)
    n = packed.shape[0]
    stream = ((packed[..., None] >> np.arange(32, dtype=np.uint32)) & np.uint32(1)).reshape(n, -1, bits)
    return (stream.astype(np.uint32) << np.arange(bits, dtype=np.uint32)).sum(axis=-1).astype(np.uint32)


def dequantize_affine(packed, scales, biases, group_size: int = 64, bits: int = 4) -> np.ndarray:
    """W_hat[N, K] = q * scale + bias per group, float32 (mx.dequantize semantics)."""
    q = unpack_codes(np.asarray(packed), bits).astype(np.float32)
    n, k = q.shape
    s = _as_f32(scales)[..., None]
    b = _as_f32(biases)[..., None]
    return (q.reshape(n, k // group_size, group_size) * s + b).reshape(n, k).astype(np.float32)


def qlinear(x, packed, scales, biases, bias=None, group_size: int = 64, bits: int = 4) -> np.ndarray:
    """Y[..., N] = X[..., K] . dequant(W)^T + bias in float32 (nn.QuantizedLinear.__call__)."""
    x = _as_f32(x)
    w_hat = dequantize_affine(packed, scales, biases, group_size, bits)
    y = x.reshape(-1, x.shape[-1]) @ w_hat.T
    if bias is not None:
        y = y + _as_f32(bias)[None, :]
    return y.reshape(*x.shape[:-1], w_hat.shape[0]).astype(np.float32)


def rel_l2(a, b) -> float:
    """||a - b|| / ||b|| in float64 (the tolerance metric of the parity tests)."""
    a = _as_f32(a).astype(np.float64).ravel()
    b = _as_f32(b).astype(np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))
