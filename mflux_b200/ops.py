"""Tensor-level operations: PyTorch CUDA tensors in, kernels of libmfx.so underneath.

Each function validates what only the host can know (device, dtype, contiguity), hands raw device
pointers to the C ABI and raises on a non-zero status. There is no fallback path: tensors must
live on a CUDA device and the library must be built.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_void_p

import torch

from . import _lib
from ._lib import (BF16, EPI_GATE_RESIDUAL, EPI_GELU_ERF, EPI_GELU_TANH, EPI_NONE, EPI_SILU, F16, F32, QMODE_DOC,
                   QMODE_MLX, QLinearArgs)

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_EPI = {None: EPI_NONE, "none": EPI_NONE, "gelu": EPI_GELU_ERF, "gelu_erf": EPI_GELU_ERF,
        "gelu_approx": EPI_GELU_TANH, "gelu_tanh": EPI_GELU_TANH, "gate_residual": EPI_GATE_RESIDUAL,
        "silu": EPI_SILU}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}") from None


def _cuda(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")
    return t


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def poll_device_status() -> int:
    """Read and clear the device status word (0 = clean). Raises if a bounded wait gave up."""
    lib = _lib.load()
    v = c_int(0)
    rc = lib.mfx_poll_device_status(byref(v), _stream())
    if rc != 0:
        raise RuntimeError(f"device status {v.value}: {lib.mfx_status_str(rc).decode()}")
    return v.value


def quantize_affine(w: torch.Tensor, group_size: int = 64, bits: int = 4, mode: str = "mlx"):
    """mx.quantize(w, group_size, bits): W[N, K] -> (uint32 [N, K*bits/32], scales, biases [N, K/64])."""
    lib = _lib.load()
    _cuda(w, "w")
    if w.dim() != 2:
        raise ValueError("w must be [N, K]")
    w = w.contiguous()
    n, k = w.shape
    if bits not in (4, 8) or group_size != 64 or k % 64 != 0:
        # validated again by the library; shapes of the outputs need it here
        _lib.check(-3 if (bits not in (4, 8) or group_size != 64) else -1, "quantize_affine")
    wq = torch.empty((n, k * bits // 32), dtype=torch.uint32, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=w.dtype, device=w.device)
    biases = torch.empty_like(scales)
    qm = {"mlx": QMODE_MLX, "doc": QMODE_DOC}[mode]
    rc = lib.mfx_quantize_affine(_ptr(w), _dt(w), n, k, bits, group_size, qm, _ptr(wq), _ptr(scales), _ptr(biases),
                                 _stream())
    _lib.check(rc, "mfx_quantize_affine")
    return wq, scales, biases


def dequantize_affine(wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
                      bits: int = 4, dtype: torch.dtype | None = None) -> torch.Tensor:
    """mx.dequantize: packed [N, K*bits/32] -> dense [N, K]."""
    lib = _lib.load()
    _cuda(wq, "wq")
    wq, scales, biases = wq.contiguous(), scales.contiguous(), biases.contiguous()
    n = wq.shape[0]
    k = wq.shape[1] * 32 // bits
    out = torch.empty((n, k), dtype=dtype or scales.dtype, device=wq.device)
    rc = lib.mfx_dequantize_affine(_ptr(wq), _ptr(scales), _ptr(biases), _dt(scales), n, k, bits, group_size,
                                   _ptr(out), _dt(out), _stream())
    _lib.check(rc, "mfx_dequantize_affine")
    return out


def prepare_qlinear(wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int = 4,
                    group_size: int = 64) -> torch.Tensor:
    """Kernel-side form of one quantized weight (interleaved codes + transposed bf16 scale/bias pairs).

    Returns an opaque uint8 blob to be passed as `prepared=` to qlinear; build it once per weight.
    """
    lib = _lib.load()
    _cuda(wq, "wq")
    wq, scales, biases = wq.contiguous(), scales.contiguous(), biases.contiguous()
    n = wq.shape[0]
    k = wq.shape[1] * 32 // bits
    nbytes = lib.mfx_qlinear_prepared_bytes(n, k, bits, group_size)
    if nbytes == 0:
        _lib.check(-3 if (bits not in (4, 8) or group_size != 64) else -1, "prepare_qlinear")
    blob = torch.empty(nbytes, dtype=torch.uint8, device=wq.device)
    rc = lib.mfx_qlinear_prepare(_ptr(wq), _ptr(scales), _ptr(biases), _dt(scales), n, k, bits, group_size,
                                 _ptr(blob), nbytes, _stream())
    _lib.check(rc, "mfx_qlinear_prepare")
    return blob


def _rows_view(t: torch.Tensor, name: str):
    """(tensor, rows, batch, row_stride, batch_stride) of a [..., rows, cols] tensor whose last dim is dense."""
    if t.dim() < 2:
        raise ValueError(f"{name} must have at least 2 dims")
    if t.stride(-1) != 1:
        t = t.contiguous()
    if t.dim() == 2:
        return t, t.shape[0], 1, t.stride(0), 0
    if t.dim() > 3:
        t = t.reshape(-1, t.shape[-2], t.shape[-1])
    return t, t.shape[1], t.shape[0], t.stride(1), t.stride(0)


def qlinear(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
            bias: torch.Tensor | None = None, *, bits: int = 4, group_size: int = 64, epilogue: str | None = None,
            gate: torch.Tensor | None = None, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
            prepared: torch.Tensor | None = None) -> torch.Tensor:
    """nn.QuantizedLinear.__call__: y[..., N] = x[..., K] . dequant(wq)^T + bias, with optional fused epilogue.

    x is [rows, K] or [batch, rows, K] (bf16; row/batch strides may be arbitrary multiples of 8
    elements, the last dim must be dense). `out`, when given, may be a strided view of the same
    leading shape. epilogue "gate_residual" computes residual + gate[batch] * y with gate [batch, N].
    `prepared` is the cached result of prepare_qlinear(wq, scales, biases); without it the weight is
    prepared into a scratch tensor on every call.
    """
    lib = _lib.load()
    _cuda(x, "x")
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    lead = x.shape[:-1]
    if x.dim() == 1:
        x = x.unsqueeze(0)
    xv, rows, batch, x_rs, x_bs = _rows_view(x, "x")
    k = xv.shape[-1]
    n = wq.shape[0]
    if wq.shape[1] * 32 // bits != k:
        raise ValueError(f"x has K={k} but the packed weight encodes K={wq.shape[1] * 32 // bits}")
    if prepared is None:
        wq, scales, biases = wq.contiguous(), scales.contiguous(), biases.contiguous()
        workspace = torch.empty(lib.mfx_qlinear_prepared_bytes(n, k, bits, group_size), dtype=torch.uint8,
                                device=x.device)
    if out is None:
        od = out_dtype or (residual.dtype if residual is not None else torch.bfloat16)
        out = torch.empty((*xv.shape[:-1], n), dtype=od, device=x.device)
        ret = out.reshape(*lead, n)
    else:
        ret = out
    ov, o_rows, o_batch, o_rs, o_bs = _rows_view(out, "out")
    if ov.data_ptr() != out.data_ptr() or (o_rows, o_batch) != (rows, batch) or ov.shape[-1] != n:
        raise ValueError("out must be a [.., rows, N] view with a dense last dim matching x")
    a = QLinearArgs()
    a.x, a.x_row_stride, a.x_batch_stride = xv.data_ptr(), x_rs, x_bs
    a.rows, a.batch, a.K, a.N = rows, batch, k, n
    a.bits, a.group_size = bits, group_size
    if prepared is None:
        a.wq, a.scales, a.biases, a.sb_dtype = wq.data_ptr(), scales.data_ptr(), biases.data_ptr(), _dt(scales)
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    else:
        if prepared.dtype != torch.uint8 or prepared.numel() != lib.mfx_qlinear_prepared_bytes(n, k, bits, group_size):
            raise ValueError("prepared must be the blob prepare_qlinear returned for this weight")
        a.prepared = prepared.data_ptr()
    if bias is not None:
        bias = bias.contiguous()
        a.bias, a.bias_dtype = bias.data_ptr(), _dt(bias)
    a.epilogue = _EPI[epilogue]
    if a.epilogue == EPI_GATE_RESIDUAL:
        if gate is None or residual is None:
            raise ValueError("gate_residual needs gate and residual")
        gate = gate.reshape(-1, n) if gate.stride(-1) == 1 else gate.reshape(-1, n).contiguous()
        if gate.shape[0] != batch:
            raise ValueError("gate must be [batch, N]")
        rv, r_rows, r_batch, r_rs, r_bs = _rows_view(residual, "residual")
        if rv.dtype != ov.dtype or (r_rows, r_batch) != (rows, batch):
            raise ValueError("residual must match out in dtype and leading shape")
        a.gate, a.gate_dtype, a.gate_batch_stride = gate.data_ptr(), _dt(gate), gate.stride(0)
        a.residual, a.res_row_stride, a.res_batch_stride = rv.data_ptr(), r_rs, r_bs
    a.y, a.y_dtype, a.y_row_stride, a.y_batch_stride = ov.data_ptr(), _dt(ov), o_rs, o_bs
    rc = lib.mfx_qlinear_ex(byref(a), _stream())
    _lib.check(rc, "mfx_qlinear_ex")
    return ret
