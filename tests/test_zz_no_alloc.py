"""The allocation-free entry point mfx_qlinear_static_scratch (collected last on purpose).

Some callers cannot allocate device memory when they call into the library (all of HBM already belongs
to their own allocator, or an allocation's implicit synchronisation is not acceptable where they call
from), so they cannot supply the workspace mfx_qlinear wants. This entry point keeps that scratch in a
fixed array inside the library instead. The test calls it through the C ABI several times in a row, with
different weights, and compares each result with what the workspace-taking entry point returns for the same
inputs (the kernels are the same, so the outputs must be identical, and a call must not see anything of the
one before) and with the float32 CPU oracle (rel-L2 <= 1e-2, the tolerance of the other quantized-linear
tests). The cases cover both kernels behind the entry point: the tensor-core kernel (more than 16 rows) and the
weight-streaming kernel (at most 16 rows). It also checks the documented size limit.
"""
import pytest
import torch

from oracle import quant
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu


def _case(m, n, k, bits, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    b = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    return w, x, b


def test_static_scratch_matches_workspace_entry_point_and_oracle(lib_built):
    from mflux_b200 import ops

    cases = [(300, 1024, 512, 4), (129, 520, 1024, 8), (16, 768, 512, 4), (1, 264, 256, 8), (300, 1024, 512, 4)]
    for call, (m, n, k, bits) in enumerate(cases):
        w, x, b = _case(m, n, k, bits, 40 + call)
        wq, s, bi = ops.quantize_affine(w.cuda(), 64, bits)
        want = ops.qlinear_plain(x.cuda(), wq, s, bi, b.cuda(), bits=bits, static_scratch=False)
        got = ops.qlinear_plain(x.cuda(), wq, s, bi, b.cuda(), bits=bits, static_scratch=True)
        torch.cuda.synchronize()
        assert ops.poll_device_status() == 0
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)  # same kernels, same inputs: bit-identical
        ref = quant.qlinear(x, wq.cpu().numpy(), s.float().cpu().numpy(), bi.float().cpu().numpy(), b, 64, bits)
        assert rel_l2(got, ref) <= 1e-2


def test_static_scratch_rejects_weights_beyond_its_limit(lib_built):
    from mflux_b200 import _lib, ops

    n, k = 16384, 8192  # 64 MiB of 4-bit codes: twice the built-in scratch
    assert _lib.load().mfx_qlinear_prepared_bytes(n, k, 4, 64) > _lib.STATIC_SCRATCH_BYTES
    wq = torch.zeros(n, k // 8, dtype=torch.uint32, device="cuda")
    s = torch.zeros(n, k // 64, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(8, k, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="fixed limit"):
        ops.qlinear_plain(x, wq, s, s.clone(), None, bits=4, static_scratch=True)
