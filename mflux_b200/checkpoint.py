"""mflux's on-disk format for (quantized) component weights, read and written with torch tensors.

Layout (src/mflux/models/common/weights/saving/model_saver.py:50-99): `<base>/<subdir>/{i}.safetensors` shards of
at most 2 GiB, each carrying the metadata `quantization_level` and `mflux_version`, plus
`model.safetensors.index.json` with the same metadata and a `weight_map` from key to shard file. Keys are the
dotted parameter paths of the module tree (`transformer_blocks.0.attn.to_q.weight`, `.scales`, `.biases`, `.bias`);
a quantized linear stores `weight` as uint32 [N, K*bits/32] and `scales` / `biases` as [N, K/64], which are the
tensors `nn.QuantizedLinear` holds, so a checkpoint written by the reference loads without re-quantizing.
Reading follows weight_loader.py:145-179: every `*.safetensors` file of the directory is merged, the level comes
from the first shard's metadata, and a directory without that metadata is not in this format.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

VERSION = "mflux-b200"


def flatten_parameters(model: torch.nn.Module) -> dict[str, torch.Tensor]:
    """mlx.utils.tree_flatten(model.parameters()): dotted paths, parameters only, in definition order."""
    return {k: v.detach() for k, v in model.named_parameters()}


def split_weights(weights: dict[str, torch.Tensor], max_file_size_bytes: int = 2 << 30) -> list[dict]:
    """ModelSaver._split_weights: greedy shards in key order, a shard closes before it would exceed the limit."""
    shards, shard, size = [], {}, 0
    for k, v in weights.items():
        nbytes = v.numel() * v.element_size()
        if size + nbytes > max_file_size_bytes and shard:   # (a tensor above the limit gets a shard of its own)
            shards.append(shard)
            shard, size = {}, 0
        shard[k] = v
        size += nbytes
    if shard:
        shards.append(shard)
    return shards


def save_weights(base_path: str | Path, bits: int | None, model: torch.nn.Module, subdir: str = "transformer",
                 max_file_size_bytes: int = 2 << 30, version: str = VERSION) -> list[str]:
    path = Path(base_path) / subdir
    path.mkdir(parents=True, exist_ok=True)
    meta = {"quantization_level": str(bits), "mflux_version": version}
    weight_map, names = {}, []
    for i, shard in enumerate(split_weights(flatten_parameters(model), max_file_size_bytes)):
        name = f"{i}.safetensors"
        save_file({k: v.cpu().contiguous() for k, v in shard.items()}, str(path / name), metadata=meta)
        names.append(name)
        for k in shard:
            weight_map[k] = name
    with open(path / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": meta, "weight_map": weight_map}, f, indent=2)
    return names


def load_weights(path: str | Path, device="cpu"):
    """(flat dict of tensors, quantization level or None, writer version) or (None, None, None) when the directory
    does not hold this format."""
    path = Path(path)
    if not path.exists():
        return None, None, None
    shard_files = sorted(f for f in path.glob("*.safetensors") if not f.name.startswith("._"))
    if not shard_files:
        return None, None, None
    with safe_open(str(shard_files[0]), framework="pt") as f:
        meta = f.metadata() or {}
    level_str, version = meta.get("quantization_level"), meta.get("mflux_version")
    if level_str is None and version is None:
        return None, None, None
    level = None if level_str in (None, "None", "null", "") else int(level_str)
    weights: dict[str, torch.Tensor] = {}
    for shard in shard_files:
        with safe_open(str(shard), framework="pt", device=str(device)) as f:
            for k in f.keys():
                weights[k] = f.get_tensor(k)
    return weights, level, version


def load_into(model, base_path: str | Path, subdir: str = "transformer", requested_bits: int | None = None) -> int | None:
    """Loads a saved component into a model built with the matching quantization. The stored level wins over a
    different requested one (with a warning), as QuantizationResolution does; keys the model does not have (other
    components' tensors saved next to it) are skipped, shape or dtype mismatches raise."""
    from . import resolution

    weights, stored, _ = load_weights(Path(base_path) / subdir, device=next(model.parameters()).device)
    if weights is None:
        raise ValueError(f"{Path(base_path) / subdir} does not hold mflux-format weights")
    bits, warning = resolution.resolve(stored, requested_bits)
    if warning:
        print(f"Warning: {warning}")
    model_bits = getattr(model, "bits", None)
    if model_bits != bits:
        raise ValueError(f"the checkpoint is quantized to {bits} bits but the model was built for {model_bits}")
    model.update(weights, strict=False)
    return bits
