"""Finite-difference gradient checks of the CUDA backward functions through the C ABI: the same cases, method and gate as
the CPU oracle's check (tests/gradcheck.py; the reference's GradCheckTests.cs, RecurrentGradTests.cs, SpatialGradTests.cs,
GraphOpsGradTests.cs and CtcLossTests.cs), with fp32 products so the forward being differenced is the fp32 one."""
import pytest

import gradcheck
from backends import GpuBackend

pytestmark = pytest.mark.gpu

CASES = gradcheck.cases()


@pytest.mark.parametrize("name,f,arrays,wrt", CASES, ids=[c[0] for c in CASES])
def test_gpu_gradients_match_central_differences(ctx, name, f, arrays, wrt):
    ctx.set_flags(0)
    errs = gradcheck.grad_check(GpuBackend(ctx), f, [a.copy() for a in arrays], wrt)
    for i, e in errs.items():
        assert e <= gradcheck.GATE, (name, i, e)
