"""CPU tests of the host-side mirror: quantization resolution rules and sigma schedules against the
reference's own golden vectors (tests/schedulers/test_linear_scheduler.py:41-73,
tests/resolution/test_quantization_resolution.py:7-70)."""
import io
import json
from pathlib import Path

import numpy as np
import pytest

from mflux_b200 import resolution
from mflux_b200.schedulers import LinearScheduler

GOLDEN = Path(__file__).parent / "golden" / "linear_scheduler_sigmas.json"


def _vec(hexstr):
    return np.load(io.BytesIO(bytes.fromhex(hexstr)))


def test_sigmas_dev_match_reference_golden():
    g = json.loads(GOLDEN.read_text())
    s = LinearScheduler(14, 1024, 1024, requires_sigma_shift=True)
    want = _vec(g["dev_requires_sigma_shift_true"])
    assert s.sigmas.shape == (15,) and s.sigmas.dtype == np.float32
    np.testing.assert_allclose(s.sigmas, want, rtol=1e-5, atol=1e-8)  # mx.allclose defaults


def test_sigmas_schnell_match_reference_golden():
    g = json.loads(GOLDEN.read_text())
    s = LinearScheduler(14, 1024, 1024, requires_sigma_shift=False)
    np.testing.assert_allclose(s.sigmas, _vec(g["schnell_requires_sigma_shift_false"]), rtol=1e-5, atol=1e-8)


def test_euler_step():
    import torch

    s = LinearScheduler(4, 1024, 1024, requires_sigma_shift=False)
    lat = torch.ones(2, 3)
    out = s.step(torch.full((2, 3), 2.0), 0, lat)
    np.testing.assert_allclose(out.numpy(), 1.0 + 2.0 * (0.75 - 1.0))


LEVELS = [None, 3, 4, 5, 6, 8]


@pytest.mark.parametrize("stored", LEVELS)
@pytest.mark.parametrize("requested", LEVELS)
def test_resolution_rules(stored, requested):
    bits, warning = resolution.resolve(stored, requested)
    if stored is None:
        assert bits == requested and warning is None
    else:
        assert bits == stored
        if requested is not None and requested != stored:
            assert warning == f"Model is pre-quantized at {stored}-bit. Ignoring -q {requested} flag."
        else:
            assert warning is None


def test_unsupported_bits_rejected():
    for b in (3, 5, 6):
        with pytest.raises(ValueError):
            resolution.check_supported(b)
    resolution.check_supported(None)
    resolution.check_supported(4)
    resolution.check_supported(8)
