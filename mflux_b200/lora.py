"""LoRA wrappers over Linear / QuantizedLinear with the reference's names and arithmetic.

`LoRALinear` (src/mflux/models/common/lora/layer/linear_lora_layer.py:7-53): attributes `linear`, `scale`,
`lora_A` [input_dims, r], `lora_B` [r, output_dims]; y = linear(x) + scale * (x @ lora_A) @ lora_B.
`FusedLoRALinear` (fused_linear_lora_layer.py:7-20): `base_linear` plus a list `loras`, y = base(x) + sum of the
adapters' scaled low-rank products.

Execution: the frozen base runs on the quantized-matmul kernel; the two thin matmuls of an adapter are plain library
GEMMs, the second one accumulating in place into the base output (one extra pass over y per adapter). Epilogues
that the unwrapped layer fuses into its matmul (activation, gate * y + residual) are applied afterwards by the
caller for wrapped layers, because the adapter's term has to be added before them.
"""
from __future__ import annotations

import math

import torch

from . import nn


def _low_rank_add(y: torch.Tensor, x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale: float) -> torch.Tensor:
    """y += scale * (x @ a) @ b, in place; x [..., K], y [..., N] (same leading shape)."""
    t = torch.matmul(x.to(a.dtype), a)                      # [..., r]
    if y.dtype != b.dtype:
        return y.add_(torch.matmul(t, b), alpha=scale)
    if y.dim() == 2:
        return y.addmm_(t, b, alpha=scale)
    y3, t3 = y.reshape(-1, y.shape[-2], y.shape[-1]), t.reshape(-1, t.shape[-2], t.shape[-1])
    if y3.data_ptr() != y.data_ptr():                        # reshape had to copy: fall back to an explicit add
        return y.add_(torch.matmul(t, b), alpha=scale)
    y3.baddbmm_(t3, b.unsqueeze(0).expand(t3.shape[0], -1, -1), alpha=scale)
    return y


class LoRALinear(nn.Module):
    def __init__(self, input_dims: int, output_dims: int, r: int = 8, scale: float = 1.0, bias: bool = False,
                 device=None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.linear = nn.Linear(input_dims, output_dims, bias=bias, device=device, dtype=dtype)
        self.scale = scale
        bound = 1 / math.sqrt(input_dims)
        self.lora_A = torch.nn.Parameter(
            torch.empty(input_dims, r, device=device, dtype=torch.float32).uniform_(-bound, bound).to(dtype),
            requires_grad=False)
        self.lora_B = torch.nn.Parameter(
            torch.empty(r, output_dims, device=device, dtype=torch.float32).uniform_(-bound, bound).to(dtype),
            requires_grad=False)

    @staticmethod
    def from_linear(linear, r: int = 16, scale: float = 1.0) -> "LoRALinear":
        output_dims, input_dims = linear.weight.shape
        if isinstance(linear, nn.QuantizedLinear):
            input_dims *= 32 // linear.bits
        dev = linear.weight.device
        dtype = linear.scales.dtype if isinstance(linear, nn.QuantizedLinear) else linear.weight.dtype
        lora_lin = LoRALinear(input_dims, output_dims, r=r, scale=scale, device=dev, dtype=dtype)
        lora_lin.linear = linear
        return lora_lin

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        base_out = self.linear(x)
        return _low_rank_add(base_out, x, self.lora_A.data, self.lora_B.data, self.scale)


class FusedLoRALinear(nn.Module):
    def __init__(self, base_linear, loras: list[LoRALinear]):
        super().__init__()
        self.base_linear = base_linear
        self.loras = torch.nn.ModuleList(loras)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = self.base_linear(x)
        for lora in self.loras:
            _low_rank_add(out, x, lora.lora_A.data, lora.lora_B.data, lora.scale)
        return out


def apply_lora(model: torch.nn.Module, adapters: dict[str, list[tuple[torch.Tensor, torch.Tensor, float]]]):
    """Wrap the linears at the given module paths: one adapter -> LoRALinear, several -> FusedLoRALinear
    (what the reference's loader does per target, lora_loader.py:206-307). Each adapter is (lora_A [in, r],
    lora_B [r, out], scale). Cached fused-projection state of the model is dropped."""
    for path, items in adapters.items():
        parent_path, _, name = path.rpartition(".")
        parent = model.get_submodule(parent_path) if parent_path else model
        child = parent[int(name)] if name.isdigit() else getattr(parent, name)
        if isinstance(child, FusedLoRALinear):      # wrapped before: keep the earlier adapters, add the new ones
            base, wrapped = child.base_linear, list(child.loras)
        elif isinstance(child, LoRALinear):
            base, wrapped = child.linear, [child]
        else:
            base, wrapped = child, []
        for a, b, scale in items:
            w = LoRALinear.from_linear(base, r=a.shape[1], scale=scale)
            dev, dt = w.lora_A.device, w.lora_A.dtype
            if a.shape[0] != w.lora_A.shape[0] or b.shape[1] != w.lora_B.shape[1] or a.shape[1] != b.shape[0]:
                raise ValueError(f"{path}: adapter shapes {tuple(a.shape)}, {tuple(b.shape)} do not fit a "
                                 f"{w.lora_A.shape[0]}->{w.lora_B.shape[1]} linear")
            w.lora_A.data, w.lora_B.data = a.to(dev, dt), b.to(dev, dt)
            wrapped.append(w)
        new = wrapped[0] if len(wrapped) == 1 else FusedLoRALinear(base, wrapped)
        if name.isdigit():
            parent[int(name)] = new
        else:
            setattr(parent, name, new)
    if hasattr(model, "_fused"):
        model._fused = {}
    return model
