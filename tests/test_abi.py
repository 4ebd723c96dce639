"""The C-ABI library builds for sm_100a, loads without a GPU and exports every declared symbol."""
import re
from pathlib import Path

from mflux_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = header.read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mfx_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(lib_built):
    lib = _lib.load()
    declared = _declared()
    assert declared, "no declarations found in include/*.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signature table out of sync with include/*.h"


def test_version_and_status_strings(lib_built):
    lib = _lib.load()
    assert lib.mfx_version() == 100
    assert lib.mfx_status_str(0) == b"ok"
    for code in range(-9, 0):
        assert lib.mfx_status_str(code) != b"unknown status"


def test_argument_validation_needs_no_gpu(lib_built):
    """Host-side validation rejects bad calls before anything touches a device."""
    lib = _lib.load()
    assert lib.mfx_quantize_affine(None, 0, 4, 64, 4, 64, 0, None, None, None, None) == -7
    assert lib.mfx_quantize_affine(16, 0, 4, 64, 3, 64, 0, 16, 16, 16, None) == -3
    assert lib.mfx_quantize_affine(16, 0, 4, 96, 4, 64, 0, 16, 16, 16, None) == -1
    assert lib.mfx_quantize_affine(16, 0, 4, 64, 4, 32, 0, 16, 16, 16, None) == -3
    assert lib.mfx_quantize_affine(8, 0, 4, 64, 4, 64, 0, 16, 16, 16, None) == -2
    a = _lib.QLinearArgs()
    assert lib.mfx_qlinear_ex(a, None) == -7
    assert lib.mfx_qlinear_ex(None, None) == -7
    a.x = a.wq = a.scales = a.biases = a.y = a.workspace = 1024
    a.rows, a.batch, a.K, a.N, a.bits, a.group_size = 128, 1, 96, 64, 4, 64
    assert lib.mfx_qlinear_ex(a, None) == -1  # K % 64
    a.K = 128
    a.bits = 5
    assert lib.mfx_qlinear_ex(a, None) == -3
    a.bits = 4
    a.workspace_bytes = 16  # too small for the prepared form of the weight
    assert lib.mfx_qlinear_ex(a, None) == -1
    assert lib.mfx_qlinear_prepared_bytes(12288, 3072, 4, 64) == 12288 * 3072 // 2 + 12288 * 48 * 4
    assert lib.mfx_qlinear_prepared_bytes(12288, 3000, 4, 64) == 0
    assert lib.mfx_qlinear_prepared_bytes(10, 64, 4, 64) == 512 + 40  # 320 code bytes padded to 256s + pairs
