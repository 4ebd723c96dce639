"""Stored-vs-requested quantization level resolution.

Same four rules, priorities, return values and warning text as the reference's
QuantizationResolution.resolve (src/mflux/models/common/resolution/quantization_resolution.py:8-52):
none/none -> no quantization; none/any -> quantize on the fly at the requested bits; any/none -> use the
stored bits; any/any -> the stored bits win, with a warning when they differ.
"""
from __future__ import annotations

SUPPORTED_BITS = (3, 4, 5, 6, 8)


def resolve(stored: int | None, requested: int | None) -> tuple[int | None, str | None]:
    if stored is None and requested is None:
        return None, None
    if stored is None:
        return requested, None
    if requested is None:
        return stored, None
    warning = None
    if stored != requested:
        warning = f"Model is pre-quantized at {stored}-bit. Ignoring -q {requested} flag."
    return stored, warning


def check_supported(bits: int | None) -> None:
    """The widths the reference's CLI accepts (cli/defaults/defaults.py:63): 3, 4, 5, 6, 8."""
    if bits is not None and bits not in SUPPORTED_BITS:
        raise ValueError(f"quantize={bits} is not implemented on this backend (supported: {SUPPORTED_BITS})")
