"""Host-side mirror of the mlx.nn surface the reference's hot path is written against.

`Linear`, `QuantizedLinear` and `quantize(model, group_size, bits, class_predicate)` keep the names,
attribute names, shapes and dtypes of mlx.nn (`weight` uint32 [N, K*bits/32], `scales`/`biases`
[N, K/64], optional `bias` [N], `bits`, `group_size`), so that code written for the reference
(weight_applier.py:93-103, the LoRA wrappers of lora/layer/linear_lora_layer.py:9-24, quantized
checkpoints saved by model_saver.py:50-99) maps 1:1. Parameters are torch tensors on a CUDA device;
the arithmetic is libmfx.so (see ops.py). There is no CPU path.
"""
from __future__ import annotations

from typing import Callable

import torch

from . import ops


# Bumped by everything that replaces weights or modules (Module.update, quantize, the LoRA appliers). Caches that
# are derived from several layers' weights (row-fused q/k/v blobs, recorded CUDA graphs) remember the value they
# were built under and are dropped when it has moved on; per-layer prepared blobs are keyed on their own tensors.
_WEIGHTS_EPOCH = [0]


def weights_epoch() -> int:
    return _WEIGHTS_EPOCH[0]


def bump_weights_epoch() -> None:
    _WEIGHTS_EPOCH[0] += 1


def fused_cache(owner) -> dict:
    """`owner._fused`, emptied first if any weight in the process changed since it was last used."""
    if getattr(owner, "_fused_epoch", None) != _WEIGHTS_EPOCH[0]:
        owner._fused = {}
        owner._fused_epoch = _WEIGHTS_EPOCH[0]
    return owner._fused


class Module(torch.nn.Module):
    """torch.nn.Module with the two mlx.nn.Module helpers the reference calls on the hot path."""

    def update(self, weights: dict, strict: bool = True) -> "Module":
        """mlx.nn.Module.update: load a (nested) dict of tensors by attribute path."""
        flat = dict(_flatten(weights))
        own = dict(self.named_parameters()) | dict(self.named_buffers())
        for key, value in flat.items():
            if key not in own:
                if strict:
                    raise ValueError(f"unexpected parameter {key}")
                continue
            target = own[key]
            if tuple(target.shape) != tuple(value.shape) or target.dtype != value.dtype:
                # a quantized skeleton receives packed tensors of its own shape; anything else is an error
                raise ValueError(f"{key}: expected {tuple(target.shape)} {target.dtype}, "
                                 f"got {tuple(value.shape)} {value.dtype}")
            with torch.no_grad():
                target.copy_(value)
            mod = self.get_submodule(key.rsplit(".", 1)[0]) if "." in key else self
            if isinstance(mod, QuantizedLinear):
                mod._prepared = None
        bump_weights_epoch()
        if strict:
            missing = set(own) - set(flat)
            if missing:
                raise ValueError(f"missing parameters: {sorted(missing)[:5]}")
        return self

    def leaf_modules(self):
        return {name: m for name, m in self.named_modules() if not list(m.children())}


def _flatten(tree, prefix=""):
    if isinstance(tree, dict):
        for k, v in tree.items():
            yield from _flatten(v, f"{prefix}{k}.")
    elif isinstance(tree, (list, tuple)):
        for i, v in enumerate(tree):
            yield from _flatten(v, f"{prefix}{i}.")
    else:
        yield prefix[:-1], tree


class Linear(Module):
    """mlx.nn.Linear: y = x W^T + b with weight [out, in]. Dense layers stay on torch.matmul (they are
    not part of the quantized hot path); `to_quantized` is what mlx.nn.quantize looks for."""

    def __init__(self, input_dims: int, output_dims: int, bias: bool = True, device=None,
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        scale = input_dims ** -0.5
        w = torch.empty(output_dims, input_dims, device=device, dtype=torch.float32).uniform_(-scale, scale)
        self.weight = torch.nn.Parameter(w.to(dtype), requires_grad=False)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(output_dims, device=device, dtype=dtype), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x.to(self.weight.dtype), self.weight, self.bias)

    def to_quantized(self, group_size: int = 64, bits: int = 4, mode: str = "mlx") -> "QuantizedLinear":
        return QuantizedLinear.from_linear(self, group_size, bits, mode)


class QuantizedLinear(Module):
    """mlx.nn.QuantizedLinear: group-wise affine quantized weight, y = x . dequant(W)^T + bias."""

    def __init__(self, input_dims: int, output_dims: int, bias: bool = True, group_size: int = 64, bits: int = 4,
                 device=None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if bits not in ops.BITS:
            raise ValueError(f"bits={bits} is not supported (supported: {ops.BITS})")
        if group_size != 64:
            raise ValueError("group_size must be 64")
        if input_dims % group_size != 0:
            raise ValueError(f"The last dimension of the matrix needs to be divisible by the quantization "
                             f"group size {group_size}; got {input_dims}")
        self.group_size, self.bits = group_size, bits
        self.weight = torch.nn.Parameter(
            torch.zeros(output_dims, input_dims * bits // 32, dtype=torch.uint32, device=device), requires_grad=False)
        self.scales = torch.nn.Parameter(
            torch.zeros(output_dims, input_dims // group_size, dtype=dtype, device=device), requires_grad=False)
        self.biases = torch.nn.Parameter(torch.zeros_like(self.scales), requires_grad=False)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(output_dims, device=device, dtype=dtype), requires_grad=False)
        else:
            self.register_parameter("bias", None)
        self._prepared = None

    @classmethod
    def from_linear(cls, linear: Linear, group_size: int = 64, bits: int = 4, mode: str = "mlx"):
        out_dims, in_dims = linear.weight.shape
        ql = cls(in_dims, out_dims, linear.bias is not None, group_size, bits, device=linear.weight.device,
                 dtype=linear.weight.dtype)
        wq, scales, biases = ops.quantize_affine(linear.weight.data, group_size, bits, mode)
        ql.weight.data, ql.scales.data, ql.biases.data = wq, scales, biases
        if linear.bias is not None:
            ql.bias.data = linear.bias.data
        return ql

    @property
    def input_dims(self) -> int:
        return self.weight.shape[1] * 32 // self.bits

    @property
    def output_dims(self) -> int:
        return self.weight.shape[0]

    def prepared(self) -> torch.Tensor:
        """Kernel-side form of the weight, built on first use and rebuilt if the tensors were replaced."""
        key = (self.weight.data_ptr(), self.weight._version, self.scales.data_ptr(), self.scales._version,
               self.biases.data_ptr(), self.biases._version)
        if self._prepared is None or self._prepared[0] != key:
            blob = ops.prepare_qlinear(self.weight.data, self.scales.data, self.biases.data, self.bits,
                                       self.group_size)
            self._prepared = (key, blob)
        return self._prepared[1]

    def forward(self, x: torch.Tensor, *, epilogue: str | None = None, gate: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        return ops.qlinear(x, self.weight.data, self.scales.data, self.biases.data,
                           None if self.bias is None else self.bias.data, bits=self.bits,
                           group_size=self.group_size, epilogue=epilogue, gate=gate, residual=residual, out=out,
                           out_dtype=out_dtype, prepared=self.prepared())

    def dequantize(self, dtype: torch.dtype | None = None) -> torch.Tensor:
        return ops.dequantize_affine(self.weight.data, self.scales.data, self.biases.data, self.group_size, self.bits,
                                     dtype)


def quantize(model: torch.nn.Module, group_size: int = 64, bits: int = 4,
             class_predicate: Callable[[str, torch.nn.Module], bool] | None = None, mode: str = "mlx"):
    """mlx.nn.quantize: replace, in place, every module that has `to_quantized` and passes the predicate.

    The default predicate is the reference's (weight_applier.py:29-31): `hasattr(module, "to_quantized")`.
    Modules whose input dimension is not a multiple of the group size raise, as MLX does.
    """
    if class_predicate is None:
        class_predicate = lambda path, m: hasattr(m, "to_quantized")  # noqa: E731
    todo = []
    for path, module in model.named_modules():
        if path and hasattr(module, "to_quantized") and class_predicate(path, module):
            todo.append(path)
    for path in todo:
        parent_path, _, name = path.rpartition(".")
        parent = model.get_submodule(parent_path) if parent_path else model
        child = getattr(parent, name) if not name.isdigit() else parent[int(name)]
        q = child.to_quantized(group_size=group_size, bits=bits, mode=mode)
        if name.isdigit():
            parent[int(name)] = q
        else:
            setattr(parent, name, q)
    bump_weights_epoch()
    return model
