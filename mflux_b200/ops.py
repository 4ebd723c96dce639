"""Tensor-level operations: PyTorch CUDA tensors in, kernels of libmfx.so underneath.

Each function validates what only the host can know (device, dtype, contiguity), hands raw device
pointers to the C ABI and raises on a non-zero status. There is no fallback path: tensors must
live on a CUDA device and the library must be built.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_void_p
from ctypes import pointer as ctypes_pointer

import torch

from . import _lib
from ._lib import (BF16, EPI_GATE_RESIDUAL, EPI_GELU_ERF, EPI_GELU_TANH, EPI_NONE, EPI_SILU, EPI_SWIGLU, F16, F32, QMODE_DOC,
                   QMODE_MLX, QLinearArgs)

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_EPI = {None: EPI_NONE, "none": EPI_NONE, "gelu": EPI_GELU_ERF, "gelu_erf": EPI_GELU_ERF,
        "gelu_approx": EPI_GELU_TANH, "gelu_tanh": EPI_GELU_TANH, "gate_residual": EPI_GATE_RESIDUAL,
        "silu": EPI_SILU, "swiglu": EPI_SWIGLU}


# Code widths of the affine quantizer: the ones the reference's CLI offers (src/mflux/cli/defaults/defaults.py:63).
BITS = (3, 4, 5, 6, 8)

# Kernel launches issued through this module since import (bench.py reports the count of a timed region).
LAUNCHES = [0]
# When set to a dict, the traced operations append (flops, bytes, start_event, end_event) per launch under their
# kind ("qlinear", "fmha", "glue"): bench.py's roofline legs read the events after the timed region. `flops` and
# `bytes` are the algorithmic work of the launch (2 M N K; 4 B H S^2 128; one read and one write of the rows).
TRACE = None
_trace_open = []


def _trace_begin():
    e0 = torch.cuda.Event(enable_timing=True)
    e0.record()
    _trace_open.append(e0)


def _trace_end(kind: str, flops: float, nbytes: float):
    e1 = torch.cuda.Event(enable_timing=True)
    e1.record()
    TRACE.setdefault(kind, []).append((flops, nbytes, _trace_open.pop(), e1))


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
    """mx.quantize(w, group_size, bits): W[N, K] -> (uint32 [N, K*bits/32], scales, biases [N, K/64]).
    bits is 3, 4, 5, 6 or 8; code j of a row sits at bits [j*bits, (j+1)*bits) of the row's bit stream."""
    lib = _lib.load()
    _cuda(w, "w")
    if w.dim() != 2:
        raise ValueError("w must be [N, K]")
    w = w.contiguous()
    n, k = w.shape
    if bits not in BITS or group_size != 64 or k % 64 != 0:
        # validated again by the library; shapes of the outputs need it here
        _lib.check(-3 if (bits not in BITS or group_size != 64) else -1, "quantize_affine")
    wq = torch.empty((n, k * bits // 32), dtype=torch.uint32, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=w.dtype, device=w.device)
    biases = torch.empty_like(scales)
    qm = {"mlx": QMODE_MLX, "doc": QMODE_DOC}[mode]
    rc = lib.mfx_quantize_affine(_ptr(w), _dt(w), n, k, bits, group_size, qm, _ptr(wq), _ptr(scales), _ptr(biases),
                                 _stream())
    _lib.check(rc, "mfx_quantize_affine")
    LAUNCHES[0] += 1
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
    LAUNCHES[0] += 1
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
        _lib.check(-3 if (bits not in BITS or group_size != 64) else -1, "prepare_qlinear")
    blob = torch.empty(nbytes, dtype=torch.uint8, device=wq.device)
    rc = lib.mfx_qlinear_prepare(_ptr(wq), _ptr(scales), _ptr(biases), _dt(scales), n, k, bits, group_size,
                                 _ptr(blob), nbytes, _stream())
    _lib.check(rc, "mfx_qlinear_prepare")
    LAUNCHES[0] += 2
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
            prepared: torch.Tensor | None = None, lora_t: torch.Tensor | None = None,
            lora_b: torch.Tensor | None = None, lora_r: int = 0, scatter=None) -> torch.Tensor:
    """nn.QuantizedLinear.__call__: y[..., N] = x[..., K] . dequant(wq)^T + bias, with optional fused epilogue.

    Low-rank term (LoRA adapters over the frozen layer): with `lora_t` [..., ld] (= x @ A, same leading shape as
    x) and `lora_b` [N, ld] (row n = scale * B[:, n]), both bf16 with ld a multiple of 64 and zero columns from
    `lora_r` on, the kernel adds lora_t . lora_b^T inside the same accumulation, before bias and epilogue.

    x is [rows, K] or [batch, rows, K] (bf16; row/batch strides may be arbitrary multiples of 8
    elements, the last dim must be dense). `out`, when given, may be a strided view of the same
    leading shape. epilogue "gate_residual" computes residual + gate[batch] * y with gate [batch, N].
    epilogue "swiglu" returns silu(y[..., 0::2]) * y[..., 1::2], N/2 wide (rows of the gate and up
    projections interleaved by the caller). `prepared` is the cached result of
    prepare_qlinear(wq, scales, biases); without it the weight is prepared into a scratch tensor on every call.
    `scatter` (a _lib.TpScatter) turns the call into the producer half of a tensor-parallel reduce-scatter: the
    bf16 product, without bias, goes row by row into the partial-sum slots of the ranks that own the rows; nothing
    is returned.
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
    n_out = n // 2 if _EPI[epilogue] == EPI_SWIGLU else n
    if scatter is not None:
        a = QLinearArgs()
        a.x, a.x_row_stride, a.x_batch_stride = xv.data_ptr(), x_rs, x_bs
        a.rows, a.batch, a.K, a.N = rows, batch, k, n
        a.bits, a.group_size = bits, group_size
        if prepared is None:
            raise ValueError("the scatter epilogue needs a prepared weight")
        a.prepared = prepared.data_ptr()
        a.epilogue, a.y_dtype = _lib.EPI_PEER_SCATTER, BF16
        a.scatter = ctypes_pointer(scatter)
        if TRACE is not None:
            _trace_begin()
        _lib.check(lib.mfx_qlinear_ex(byref(a), _stream()), "mfx_qlinear_ex")
        if TRACE is not None:
            m = rows * batch
            _trace_end("qlinear", 2.0 * m * n * k, n * k * bits / 8 + 4.0 * n * (k // group_size) + 2.0 * m * k
                       + 2.0 * m * n)
        LAUNCHES[0] += 1
        return None
    if out is None:
        od = out_dtype or (residual.dtype if residual is not None else torch.bfloat16)
        out = torch.empty((*xv.shape[:-1], n_out), dtype=od, device=x.device)
        ret = out.reshape(*lead, n_out)
    else:
        ret = out
    ov, o_rows, o_batch, o_rs, o_bs = _rows_view(out, "out")
    if ov.data_ptr() != out.data_ptr() or (o_rows, o_batch) != (rows, batch) or ov.shape[-1] != n_out:
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
    if lora_r:
        if lora_t is None or lora_b is None:
            raise ValueError("a low-rank term needs lora_t and lora_b")
        _cuda(lora_t, "lora_t")
        if lora_t.dtype != torch.bfloat16 or lora_b.dtype != torch.bfloat16:
            raise ValueError("lora_t and lora_b must be bf16")
        if lora_t.dim() == 1:
            lora_t = lora_t.unsqueeze(0)
        tv, t_rows, t_batch, t_rs, t_bs = _rows_view(lora_t, "lora_t")
        ld = tv.shape[-1]
        if (t_rows, t_batch) != (rows, batch) or tuple(lora_b.shape) != (n, ld) or not lora_b.is_contiguous():
            raise ValueError("lora_t must be [.., rows, ld] like x and lora_b a dense [N, ld]")
        a.lora_t, a.lora_t_row_stride, a.lora_t_batch_stride = tv.data_ptr(), t_rs, t_bs
        a.lora_b, a.lora_ld, a.lora_r = lora_b.data_ptr(), ld, int(lora_r)
    if TRACE is not None:
        _trace_begin()
    rc = lib.mfx_qlinear_ex(byref(a), _stream())
    _lib.check(rc, "mfx_qlinear_ex")
    if TRACE is not None:
        m = rows * batch
        _trace_end("qlinear", 2.0 * m * n * k, n * k * bits / 8 + 4.0 * n * (k // group_size) + 2.0 * m * k
                   + ov.element_size() * m * n_out)
    LAUNCHES[0] += 1 if prepared is not None else 3
    return ret


def norm_modulate(x: torch.Tensor, shift: torch.Tensor | None = None, scale: torch.Tensor | None = None, *,
                  weight: torch.Tensor | None = None, eps: float = 1e-6, rms: bool = False,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm(affine=False) or RMSNorm(weight) over the last dim, then * (1 + scale) + shift per sample.

    x is [rows, D] or [batch, rows, D] (f32 or bf16, strided views allowed); shift/scale are [batch, D];
    the result is bf16 (optionally written into the strided view `out`).
    """
    lib = _lib.load()
    _cuda(x, "x")
    xv, rows, batch, x_rs, x_bs = _rows_view(x, "x")
    d = xv.shape[-1]
    if out is None:
        out = torch.empty(xv.shape, dtype=torch.bfloat16, device=x.device)
        ret = out.reshape(x.shape)
    else:
        ret = out
    ov, o_rows, o_batch, o_rs, o_bs = _rows_view(out, "out")
    if ov.data_ptr() != out.data_ptr() or (o_rows, o_batch) != (rows, batch) or ov.dtype != torch.bfloat16:
        raise ValueError("out must be a bf16 view shaped like x with a dense last dim")
    a = _lib.NormArgs()
    a.x, a.x_dtype, a.x_row_stride, a.x_batch_stride = xv.data_ptr(), _dt(xv), x_rs, x_bs
    a.rows, a.batch, a.D = rows, batch, d
    mods = [t for t in (shift, scale) if t is not None]
    if mods:
        md = mods[0]
        for t in mods:
            if t.dtype != md.dtype or t.shape[-1] != d or t.stride(-1) != 1 or t.reshape(-1, d).shape[0] != batch:
                raise ValueError("shift/scale must be [batch, D] views of one dtype with a dense last dim")
        strides = {t.stride(0) if t.dim() == 2 else 0 for t in mods}
        if len(strides) != 1:
            raise ValueError("shift and scale must share their batch stride")
        a.mod_dtype, a.mod_batch_stride = _dt(md), strides.pop()
        a.shift = 0 if shift is None else shift.data_ptr()
        a.scale = 0 if scale is None else scale.data_ptr()
    if weight is not None:
        weight = weight.contiguous()
        a.weight, a.weight_dtype = weight.data_ptr(), _dt(weight)
    a.eps, a.rms = eps, int(rms)
    a.y, a.y_row_stride, a.y_batch_stride = ov.data_ptr(), o_rs, o_bs
    if TRACE is not None:
        _trace_begin()
    _lib.check(lib.mfx_norm_modulate(byref(a), _stream()), "mfx_norm_modulate")
    if TRACE is not None:
        _trace_end("glue", 0.0, float(rows * batch * d * (xv.element_size() + 2)))
    LAUNCHES[0] += 1
    return ret


def qknorm_rope(qkv: torch.Tensor, heads: int, q_weight_a: torch.Tensor, k_weight_a: torch.Tensor,
                q_weight_b: torch.Tensor, k_weight_b: torch.Tensor, split: int, cos_sin: torch.Tensor,
                eps: float = 1e-5, kv_heads: int | None = None, rope_mode: str = "pairs") -> torch.Tensor:
    """In place on qkv [batch, seq, (heads + 2*kv_heads)*128] (bf16, q | k | v per token): per-head RMSNorm(128)
    of Q and K, then RoPE. kv_heads defaults to heads.

    Rows s < split use the `_a` weights (text stream), the others the `_b` weights. cos_sin is f32
    [seq, 64, 2] holding (cos, sin) of 64 angles per token: rope_mode "pairs" rotates the (even, odd) pair i by
    angle i; "halves" computes x * cos + (-x[64:], x[:64]) * sin with element j of either half reading angle j // 2
    (ernie_transformer/rope_embedder.py:24-37).
    """
    kv_heads = heads if kv_heads is None else kv_heads
    if rope_mode not in ("pairs", "halves"):
        raise ValueError("rope_mode is 'pairs' or 'halves'")
    lib = _lib.load()
    _cuda(qkv, "qkv")
    if qkv.dtype != torch.bfloat16 or qkv.dim() != 3 or qkv.stride(-1) != 1:
        raise ValueError("qkv must be a bf16 [batch, seq, 3*heads*128] view with a dense last dim")
    batch, seq, width = qkv.shape
    if width != (heads + 2 * kv_heads) * 128:
        raise ValueError("last dim must be (heads + 2 * kv_heads) * 128")
    ws = [w.contiguous() for w in (q_weight_a, k_weight_a, q_weight_b, k_weight_b)]
    if len({w.dtype for w in ws}) != 1 or any(w.numel() != 128 for w in ws):
        raise ValueError("norm weights must be four [128] tensors of one dtype")
    cos_sin = cos_sin.contiguous()
    if cos_sin.dtype != torch.float32 or tuple(cos_sin.shape) != (seq, 64, 2):
        raise ValueError("cos_sin must be f32 [seq, 64, 2]")
    if TRACE is not None:
        _trace_begin()
    rc = lib.mfx_qknorm_rope_gqa(_ptr(qkv), qkv.stride(1), qkv.stride(0), seq, batch, heads, kv_heads,
                                 1 if rope_mode == "halves" else 0, split,
                                 _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]), _ptr(ws[3]), _dt(ws[0]), _ptr(cos_sin), eps,
                                 _stream())
    _lib.check(rc, "mfx_qknorm_rope_gqa")
    if TRACE is not None:   # q and k sections read and written once
        _trace_end("glue", 0.0, float(2 * 2 * batch * seq * heads * 128 * 2))
    LAUNCHES[0] += 1
    return qkv


def fmha(qkv: torch.Tensor, heads: int, scale: float | None = None, out: torch.Tensor | None = None,
         key_bias: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(Q K^T * scale [+ key_bias]) V for head dim 128 on the fused buffer qkv [batch, seq, 3*heads*128]
    (bf16).

    Returns (or fills the strided view `out`) bf16 [batch, seq, heads*128], the layout the reference
    hands to the output projection. `key_bias` is an optional float32 [batch, seq] additive bias per key (the
    reference's key-padding mask: 0 on real keys, -1e9 on padded ones), shared by all heads and queries.
    """
    lib = _lib.load()
    _cuda(qkv, "qkv")
    if qkv.dtype != torch.bfloat16 or qkv.dim() != 3 or qkv.stride(-1) != 1:
        raise ValueError("qkv must be a bf16 [batch, seq, 3*heads*128] view with a dense last dim")
    batch, seq, width = qkv.shape
    hd = heads * 128
    if width != 3 * hd:
        raise ValueError("last dim must be 3 * heads * 128")
    if out is None:
        out = torch.empty((batch, seq, hd), dtype=torch.bfloat16, device=qkv.device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (batch, seq, hd) or out.stride(-1) != 1:
        raise ValueError("out must be a bf16 [batch, seq, heads*128] view with a dense last dim")
    es = qkv.element_size()
    base = qkv.data_ptr()
    sc = float(scale if scale is not None else 128 ** -0.5)
    if TRACE is not None:
        _trace_begin()
    if key_bias is None:
        rc = lib.mfx_fmha(c_void_p(base), c_void_p(base + hd * es), c_void_p(base + 2 * hd * es), qkv.stride(1),
                          qkv.stride(0), seq, batch, heads, sc, _ptr(out), out.stride(1), out.stride(0), _stream())
        _lib.check(rc, "mfx_fmha")
    else:
        _cuda(key_bias, "key_bias")
        if key_bias.dtype != torch.float32 or tuple(key_bias.shape) != (batch, seq) or key_bias.stride(1) != 1:
            raise ValueError("key_bias must be a float32 [batch, seq] tensor with a dense last dim")
        if batch > 1 and key_bias.stride(0) % 4 != 0:
            # every sample's row has to start on a 16-byte boundary: copy into rows padded to a multiple of 4
            padded = torch.zeros(batch, (seq + 3) // 4 * 4, dtype=torch.float32, device=key_bias.device)
            padded[:, :seq] = key_bias
            key_bias = padded[:, :seq]
        rc = lib.mfx_fmha_bias(c_void_p(base), c_void_p(base + hd * es), c_void_p(base + 2 * hd * es), qkv.stride(1),
                               qkv.stride(0), seq, batch, heads, sc, _ptr(key_bias), key_bias.stride(0), _ptr(out),
                               out.stride(1), out.stride(0), _stream())
        _lib.check(rc, "mfx_fmha_bias")
    if TRACE is not None:
        _trace_end("fmha", 4.0 * batch * heads * seq * seq * 128, 0.0)
    LAUNCHES[0] += 1
    return out


def act_mul(y: torch.Tensor, gate: torch.Tensor, act: str = "sigmoid") -> torch.Tensor:
    """y *= act(gate) in place on bf16 [batch, rows, D] views (dense last dim, D a multiple of 8); act is "sigmoid"
    or "gelu" (erf)."""
    if act not in ("sigmoid", "gelu"):
        raise ValueError("act is 'sigmoid' or 'gelu'")
    lib = _lib.load()
    _cuda(y, "y")
    _cuda(gate, "gate")
    if y.dtype != torch.bfloat16 or gate.dtype != torch.bfloat16 or y.dim() != 3 or y.shape != gate.shape or \
            y.stride(-1) != 1 or gate.stride(-1) != 1:
        raise ValueError("y and gate must be bf16 [batch, rows, D] views of one shape with dense last dims")
    batch, rows, d = y.shape
    rc = lib.mfx_act_mul(_ptr(y), y.stride(1), y.stride(0), _ptr(gate), gate.stride(1), gate.stride(0), rows, batch, d,
                         0 if act == "sigmoid" else 1, _stream())
    _lib.check(rc, "mfx_act_mul")
    LAUNCHES[0] += 1
    return y


def fmha_ex(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, kv_heads: int | None = None,
            scale: float | None = None, key_bias: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(Q K^T * scale [+ key_bias]) V for head dim 128 with keys / values of their own length and head count.

    q is a bf16 [batch, seq_q, heads*128] view, k and v bf16 [batch, seq_kv, kv_heads*128] views with equal
    strides (dense last dim; e.g. slices of one fused projection buffer, or buffers that hold cached tokens behind
    the current ones). Query head h attends to key / value head h // (heads // kv_heads): grouped-query attention
    without repeating K / V (krea2_transformer/attention.py:33-38); seq_kv > seq_q is the cached-reference case of
    flux2_kv_cache.py:51-61. `key_bias` is an optional float32 [batch, seq_kv]. Returns bf16
    [batch, seq_q, heads*128]."""
    lib = _lib.load()
    kv_heads = heads if kv_heads is None else kv_heads
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _cuda(t, name)
        if t.dtype != torch.bfloat16 or t.dim() != 3 or t.stride(-1) != 1:
            raise ValueError(f"{name} must be a bf16 [batch, seq, heads*128] view with a dense last dim")
    batch, seq_q, wq = q.shape
    if wq != heads * 128 or k.shape[-1] != kv_heads * 128 or k.shape != v.shape or k.shape[0] != batch:
        raise ValueError("q must be [batch, seq_q, heads*128], k and v [batch, seq_kv, kv_heads*128]")
    if heads % kv_heads != 0:
        raise ValueError("heads must be a multiple of kv_heads")
    if k.stride() != v.stride():
        raise ValueError("k and v must share their strides")
    seq_kv = k.shape[1]
    if out is None:
        out = torch.empty((batch, seq_q, heads * 128), dtype=torch.bfloat16, device=q.device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (batch, seq_q, heads * 128) or out.stride(-1) != 1:
        raise ValueError("out must be a bf16 [batch, seq_q, heads*128] view with a dense last dim")
    a = _lib.FmhaArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.q_row_stride, a.q_batch_stride = q.stride(1), q.stride(0)
    a.kv_row_stride, a.kv_batch_stride = k.stride(1), k.stride(0)
    a.seq_q, a.seq_kv, a.batch, a.heads, a.kv_heads = seq_q, seq_kv, batch, heads, kv_heads
    a.scale = float(scale if scale is not None else 128 ** -0.5)
    if key_bias is not None:
        _cuda(key_bias, "key_bias")
        if key_bias.dtype != torch.float32 or tuple(key_bias.shape) != (batch, seq_kv) or key_bias.stride(1) != 1:
            raise ValueError("key_bias must be a float32 [batch, seq_kv] tensor with a dense last dim")
        if batch > 1 and key_bias.stride(0) % 4 != 0:
            padded = torch.zeros(batch, (seq_kv + 3) // 4 * 4, dtype=torch.float32, device=key_bias.device)
            padded[:, :seq_kv] = key_bias
            key_bias = padded[:, :seq_kv]
        a.key_bias, a.bias_batch_stride = key_bias.data_ptr(), key_bias.stride(0)
    a.out, a.out_row_stride, a.out_batch_stride = out.data_ptr(), out.stride(1), out.stride(0)
    if TRACE is not None:
        _trace_begin()
    _lib.check(lib.mfx_fmha_ex(byref(a), _stream()), "mfx_fmha_ex")
    if TRACE is not None:
        _trace_end("fmha", 4.0 * batch * heads * seq_q * seq_kv * 128, 0.0)
    LAUNCHES[0] += 1
    return out


def vec_sum_act(a: torch.Tensor, b: torch.Tensor | None = None, c: torch.Tensor | None = None, act: str | None = None,
                out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """act(a + b + c) elementwise; act is None, "silu" or "tanh"."""
    lib = _lib.load()
    _cuda(a, "a")
    ts = [t.contiguous() if t is not None else None for t in (a, b, c)]
    for t in ts[1:]:
        if t is not None and (t.shape != ts[0].shape or t.dtype != ts[0].dtype):
            raise ValueError("operands must share shape and dtype")
    out = torch.empty(ts[0].shape, dtype=out_dtype, device=a.device)
    rc = lib.mfx_vec_sum_act(_ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]), _dt(ts[0]), {None: 0, "silu": 1, "tanh": 2}[act], _ptr(out),
                             _dt(out), out.numel(), _stream())
    _lib.check(rc, "mfx_vec_sum_act")
    LAUNCHES[0] += 1
    return out


def euler_step(latents: torch.Tensor, noise: torch.Tensor, dt: float) -> torch.Tensor:
    """LinearScheduler.step: latents + noise * dt in the latents' dtype."""
    lib = _lib.load()
    _cuda(latents, "latents")
    latents, noise = latents.contiguous(), noise.contiguous()
    if latents.shape != noise.shape:
        raise ValueError("latents and noise must share their shape")
    out = torch.empty_like(latents)
    rc = lib.mfx_euler_step(_ptr(latents), _dt(latents), _ptr(noise), _dt(noise), float(dt), _ptr(out),
                            latents.numel(), _stream())
    _lib.check(rc, "mfx_euler_step")
    LAUNCHES[0] += 1
    return out


def qlinear_plain(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                  bias: torch.Tensor | None = None, *, bits: int = 4, static_scratch: bool = False) -> torch.Tensor:
    """y[M, N] = x[M, K] . dequant(wq)^T + bias through the two plain C entry points.

    static_scratch=False calls mfx_qlinear with a workspace tensor allocated here; static_scratch=True calls
    mfx_qlinear_static_scratch, which allocates nothing and keeps the prepared weight in an array inside
    the library (for callers that cannot allocate device memory when they call; one weight of at most
    32 MiB prepared size, calls must not overlap on the GPU).
    """
    lib = _lib.load()
    _cuda(x, "x")
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise ValueError("x must be a bf16 [M, K] matrix with a dense last dim")
    wq, scales, biases = wq.contiguous(), scales.contiguous(), biases.contiguous()
    m, k = x.shape
    n = wq.shape[0]
    if wq.shape[1] * 32 // bits != k:
        raise ValueError("x and wq disagree on K")
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    bias_c = None if bias is None else bias.contiguous()
    common = (_ptr(x), m, k, x.stride(0), _ptr(wq), _ptr(scales), _ptr(biases), _dt(scales), n, bits, 64,
              _ptr(bias_c), 0 if bias_c is None else _dt(bias_c), _ptr(y), _dt(y), y.stride(0))
    if static_scratch:
        rc = lib.mfx_qlinear_static_scratch(*common, _stream())
        _lib.check(rc, "mfx_qlinear_static_scratch")
    else:
        nbytes = lib.mfx_qlinear_prepared_bytes(n, k, bits, 64)
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x.device)
        rc = lib.mfx_qlinear(*common, _ptr(ws), ws.numel(), _stream())
        _lib.check(rc, "mfx_qlinear")
    LAUNCHES[0] += 3
    return y


def gate_residual(y: torch.Tensor, gate: torch.Tensor, residual: torch.Tensor, bias: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """residual + gate[sample] * (y + bias) in float32 (in place on `residual` when out is None).

    y [batch, rows, D] bf16/f32 dense; residual (and out) float32 [batch, rows, D] views with a dense last dim,
    e.g. a row range of the residual stream; gate [batch, D] (any batch stride), bias [D].
    """
    lib = _lib.load()
    _cuda(y, "y")
    if y.dim() != 3 or not y.is_contiguous():
        raise ValueError("y must be dense [batch, rows, D]")
    out = residual if out is None else out
    b, r, d = y.shape
    for t, name in ((residual, "residual"), (out, "out")):
        if t.dtype != torch.float32 or tuple(t.shape) != (b, r, d) or t.stride(2) != 1:
            raise ValueError(f"{name} must be a float32 [batch, rows, D] view with a dense last dim")
    if (out.stride(0), out.stride(1)) != (residual.stride(0), residual.stride(1)):
        raise ValueError("residual and out must share their strides")
    gate = gate.reshape(b, d) if gate.stride(-1) == 1 else gate.reshape(b, d).contiguous()
    bias_c = None if bias is None else bias.contiguous()
    if TRACE is not None:
        _trace_begin()
    rc = lib.mfx_gate_residual(_ptr(y), _dt(y), _ptr(bias_c), 0 if bias_c is None else _dt(bias_c), _ptr(gate),
                               _dt(gate), gate.stride(0), _ptr(residual), _ptr(out), residual.stride(1),
                               residual.stride(0) if b > 1 else r * residual.stride(1), b, r, d, _stream())
    _lib.check(rc, "mfx_gate_residual")
    if TRACE is not None:
        _trace_end("glue", 0.0, float(b * r * d * (y.element_size() + 8)))
    LAUNCHES[0] += 1
    return out


def cfg_combine(noise: torch.Tensor, noise_negative: torch.Tensor, guidance: float, mode: str = "qwen") -> torch.Tensor:
    """Guided noise in float32. mode "plain": n + g*(n - n_neg); "qwen": n_neg + g*(n - n_neg) rescaled per row
    to ||n|| over the last axis."""
    lib = _lib.load()
    _cuda(noise, "noise")
    noise, noise_negative = noise.contiguous(), noise_negative.contiguous()
    if noise.shape != noise_negative.shape or noise.dtype != noise_negative.dtype:
        raise ValueError("both predictions must share shape and dtype")
    c = noise.shape[-1]
    out = torch.empty(noise.shape, dtype=torch.float32, device=noise.device)
    rc = lib.mfx_cfg_combine(_ptr(noise), _ptr(noise_negative), _dt(noise), float(guidance),
                             {"plain": 0, "qwen": 1}[mode], _ptr(out), noise.numel() // c, c, _stream())
    _lib.check(rc, "mfx_cfg_combine")
    LAUNCHES[0] += 1
    return out


def norm_gate_residual(y: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, gate: torch.Tensor | None = None,
                       eps: float = 1e-5, *, next_weight: torch.Tensor | None = None,
                       next_scale: torch.Tensor | None = None, next_out: torch.Tensor | None = None,
                       next_eps: float | None = None) -> torch.Tensor:
    """residual += gate[sample] * RMSNorm(y) * weight, in place on the float32 view `residual`.

    y is [rows, D] or [batch, rows, D] (bf16 or f32, strided views allowed), gate [batch, D] or None. With
    `next_out` (a bf16 view shaped like y) the same pass also writes the next sub-layer's pre-norm of the updated
    stream: next_out = RMSNorm(residual) * next_weight * (1 + next_scale[sample]).
    """
    lib = _lib.load()
    _cuda(y, "y")
    yv, rows, batch, y_rs, y_bs = _rows_view(y, "y")
    rv, r_rows, r_batch, r_rs, r_bs = _rows_view(residual, "residual")
    d = yv.shape[-1]
    if rv.data_ptr() != residual.data_ptr() or rv.dtype != torch.float32 or (r_rows, r_batch) != (rows, batch) \
            or rv.shape[-1] != d:
        raise ValueError("residual must be a float32 view shaped like y with a dense last dim")
    a = _lib.PostPreNormArgs()
    a.y, a.y_dtype, a.y_row_stride, a.y_batch_stride = yv.data_ptr(), _dt(yv), y_rs, y_bs
    a.rows, a.batch, a.D = rows, batch, d
    weight = weight.contiguous()
    a.weight, a.weight_dtype, a.eps = weight.data_ptr(), _dt(weight), float(eps)
    if gate is not None:
        gate = gate.reshape(-1, d) if gate.stride(-1) == 1 else gate.reshape(-1, d).contiguous()
        if gate.shape[0] != batch:
            raise ValueError("gate must be [batch, D]")
        a.gate, a.gate_dtype, a.gate_batch_stride = gate.data_ptr(), _dt(gate), gate.stride(0)
    a.residual, a.res_row_stride, a.res_batch_stride = rv.data_ptr(), r_rs, r_bs
    if next_out is not None:
        if next_weight is None:
            raise ValueError("next_out needs next_weight")
        ov, o_rows, o_batch, o_rs, o_bs = _rows_view(next_out, "next_out")
        if ov.data_ptr() != next_out.data_ptr() or ov.dtype != torch.bfloat16 or (o_rows, o_batch) != (rows, batch) \
                or ov.shape[-1] != d:
            raise ValueError("next_out must be a bf16 view shaped like y with a dense last dim")
        next_weight = next_weight.contiguous()
        a.next_out, a.next_row_stride, a.next_batch_stride = ov.data_ptr(), o_rs, o_bs
        a.next_weight, a.next_weight_dtype = next_weight.data_ptr(), _dt(next_weight)
        a.next_eps = float(eps if next_eps is None else next_eps)
        if next_scale is not None:
            next_scale = next_scale.reshape(-1, d) if next_scale.stride(-1) == 1 else next_scale.reshape(-1, d).contiguous()
            if next_scale.shape[0] != batch:
                raise ValueError("next_scale must be [batch, D]")
            a.next_scale, a.next_scale_dtype = next_scale.data_ptr(), _dt(next_scale)
            a.next_scale_batch_stride = next_scale.stride(0)
    if TRACE is not None:
        _trace_begin()
    _lib.check(lib.mfx_post_pre_norm(byref(a), _stream()), "mfx_post_pre_norm")
    if TRACE is not None:
        _trace_end("glue", 0.0, float(rows * batch * d * (yv.element_size() + 8 + (2 if next_out is not None else 0))))
    LAUNCHES[0] += 1
    return residual


def tp_fuse(args) -> None:
    """mfx_tp_fuse on a filled _lib.TpFuseArgs: reduce-scatter consumer + gated residual + modulated LayerNorm +
    all-gather producer on the rows this rank owns (see include/mfx.h)."""
    lib = _lib.load()
    if TRACE is not None:
        _trace_begin()
    _lib.check(lib.mfx_tp_fuse(byref(args), _stream()), "mfx_tp_fuse")
    if TRACE is not None:
        rows = args.batch * args.rows_per_rank
        nbytes = rows * args.D * (8 + (2 * args.world if args.partials else 0) + (2 * args.world if args.scale[0] else 0))
        _trace_end("glue", 0.0, float(nbytes))
    LAUNCHES[0] += 1


def tp_signal(flag_ptrs, world: int) -> None:
    """Adds 1 to the int32 counters at the `world` device addresses in `flag_ptrs` (one per rank, peer-mapped) on
    the current stream: the arrival signal after stream-ordered copies to the peers."""
    lib = _lib.load()
    arr = (c_void_p * world)(*[int(v) for v in flag_ptrs[:world]])
    _lib.check(lib.mfx_tp_signal(arr, world, _stream()), "mfx_tp_signal")
    LAUNCHES[0] += 1


def tp_wait(flags: torch.Tensor, world: int, target: int, epoch_base: torch.Tensor | None = None) -> None:
    """Enqueues a bounded wait until the local counters flags[0:world] (int32, bumped by the peers) reach
    target (+ the device int epoch_base[0] when given)."""
    lib = _lib.load()
    _cuda(flags, "flags")
    _lib.check(lib.mfx_tp_wait(_ptr(flags), world, int(target), _ptr(epoch_base), _stream()), "mfx_tp_wait")
    LAUNCHES[0] += 1
