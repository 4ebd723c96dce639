"""LoRA wrappers over Linear / QuantizedLinear with the reference's names and arithmetic.

`LoRALinear` (src/mflux/models/common/lora/layer/linear_lora_layer.py:7-53): attributes `linear`, `scale`,
`lora_A` [input_dims, r], `lora_B` [r, output_dims]; y = linear(x) + scale * (x @ lora_A) @ lora_B.
`FusedLoRALinear` (fused_linear_lora_layer.py:7-20): `base_linear` plus a list `loras`, y = base(x) + sum of the
adapters' scaled low-rank products.

Execution over a quantized base: t = x @ [A_1 | A_2 | ...] is one thin library GEMM; the second product runs inside
the quantized-matmul kernel as extra K columns of the same tensor-core accumulation (operands t and the dense
[N, r] matrix of scale_i * B_i^T), so the output is written once and the layer keeps the fused epilogues of the
unwrapped one (activation, gate * y + residual) -- the adapters' term is in the accumulator before they run.
Over a dense base, or with more than 1024 adapter columns, both thin matmuls are library GEMMs, the second one
accumulating in place into the base output (one extra pass over y per adapter), and the caller applies epilogues
afterwards.
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


MAX_FUSED_COLUMNS = 1024   # the kernel's limit on the row length of the low-rank operands


class _FusedTerms:
    """Caches the two dense operands of the kernel's low-rank term for groups of adapters, each group acting on
    its own block of output rows: a_cat = [A_1 | A_2 | ...] ([K, ld], all adapters of all groups side by side) and
    b_rows ([N, ld]) whose row n holds scale_i * B_i[:, n - row0] in adapter i's columns when i belongs to the group
    covering row n, zeros elsewhere. ld is the column count padded to a multiple of 64. A single wrapped layer is
    one group over all rows; row-concatenated layers (fused q/k/v) are one group per layer. Rebuilt when an
    adapter's tensors or scale change."""

    def __init__(self):
        self.key, self.a_cat, self.b_rows, self.rank = None, None, None, 0

    def get(self, adapters, groups=None, n_rows=None):
        """`groups`: list of (first row, adapters of that block) or (first row, row step, adapters) -- a step of 2
        addresses every other row (two layers whose rows are interleaved); default one block of all `adapters`
        from row 0. `n_rows`: rows of b_rows when rows without adapters follow the last group."""
        if groups is None:
            groups = [(0, 1, list(adapters))]
        groups = [g if len(g) == 3 else (g[0], 1, g[1]) for g in groups]
        flat = [l for _, _, ls in groups for l in ls]
        key = tuple((l.lora_A.data_ptr(), l.lora_A._version, l.lora_B.data_ptr(), l.lora_B._version, float(l.scale))
                    for l in flat) + tuple((r0, step) for r0, step, _ in groups)
        if key != self.key:
            rank = sum(l.lora_A.shape[1] for l in flat)
            ld = -(-rank // 64) * 64
            k = flat[0].lora_A.shape[0]
            n = n_rows or max(r0 + step * (ls[0].lora_B.shape[1] - 1) + 1 for r0, step, ls in groups if ls)
            dev = flat[0].lora_A.device
            a_cat = torch.zeros(k, ld, dtype=torch.bfloat16, device=dev)
            b_rows = torch.zeros(n, ld, dtype=torch.bfloat16, device=dev)
            col = 0
            for r0, step, ls in groups:
                for l in ls:
                    r, rows = l.lora_A.shape[1], l.lora_B.shape[1]
                    a_cat[:, col:col + r] = l.lora_A.data
                    b_rows[r0:r0 + step * rows:step, col:col + r] = (float(l.scale) * l.lora_B.data.float()).t()
                    col += r
            self.key, self.a_cat, self.b_rows, self.rank = key, a_cat, b_rows, rank
        return self.a_cat, self.b_rows, self.rank


def split_wrapped(layer):
    """(quantized base, list of adapters) of a QuantizedLinear or of a LoRA wrapper over one; None otherwise."""
    if isinstance(layer, nn.QuantizedLinear):
        return layer, []
    if isinstance(layer, LoRALinear) and isinstance(layer.linear, nn.QuantizedLinear):
        return layer.linear, [layer]
    if isinstance(layer, FusedLoRALinear) and isinstance(layer.base_linear, nn.QuantizedLinear):
        return layer.base_linear, list(layer.loras)
    return None


def _fusable(base, adapters, x) -> bool:
    return (isinstance(base, nn.QuantizedLinear) and x.is_cuda and len(adapters) > 0
            and sum(l.lora_A.shape[1] for l in adapters) <= MAX_FUSED_COLUMNS)


def _fused_forward(base: "nn.QuantizedLinear", terms: _FusedTerms, adapters, x: torch.Tensor, **kw) -> torch.Tensor:
    from . import ops

    a_cat, b_rows, rank = terms.get(adapters)
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    t = torch.matmul(xb, a_cat)                              # [..., ld], rounded to bf16 like the reference's product
    return ops.qlinear(xb, base.weight.data, base.scales.data, base.biases.data,
                       None if base.bias is None else base.bias.data, bits=base.bits, group_size=base.group_size,
                       prepared=base.prepared(), lora_t=t, lora_b=b_rows, lora_r=rank, **kw)


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

    @property
    def fuses_epilogue(self) -> bool:
        """True when forward() accepts the quantized layer's epilogue arguments (quantized base)."""
        return isinstance(self.linear, nn.QuantizedLinear) and self.lora_A.shape[1] <= MAX_FUSED_COLUMNS

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        if _fusable(self.linear, [self], x):
            if not hasattr(self, "_terms"):
                self._terms = _FusedTerms()
            return _fused_forward(self.linear, self._terms, [self], x, **kw)
        if kw:
            raise ValueError("epilogue arguments need a quantized base layer")
        base_out = self.linear(x)
        return _low_rank_add(base_out, x, self.lora_A.data, self.lora_B.data, self.scale)


class FusedLoRALinear(nn.Module):
    def __init__(self, base_linear, loras: list[LoRALinear]):
        super().__init__()
        self.base_linear = base_linear
        self.loras = torch.nn.ModuleList(loras)

    @property
    def fuses_epilogue(self) -> bool:
        return (isinstance(self.base_linear, nn.QuantizedLinear) and len(self.loras) > 0
                and sum(l.lora_A.shape[1] for l in self.loras) <= MAX_FUSED_COLUMNS)

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        loras = list(self.loras)
        if _fusable(self.base_linear, loras, x):
            if not hasattr(self, "_terms"):
                self._terms = _FusedTerms()
            return _fused_forward(self.base_linear, self._terms, loras, x, **kw)
        if kw:
            raise ValueError("epilogue arguments need a quantized base layer")
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
    nn.bump_weights_epoch()   # row-fused blobs and recorded graphs built from the bare layers are stale now
    return model
