"""Finite-difference gradient checks of the CPU oracle's backward functions: the reference's own method and gate
(tests/OneModel.Tests/Tensors/GradCheckTests.cs:11-177, RecurrentGradTests.cs, SpatialGradTests.cs, GraphOpsGradTests.cs,
CtcLossTests.cs:41-64 of the reference), so the oracle's gradients are checked against its own forward, independent of
any fixture."""
import pytest

import gradcheck
from backends import OracleBackend

CASES = gradcheck.cases()


@pytest.mark.parametrize("name,f,arrays,wrt", CASES, ids=[c[0] for c in CASES])
def test_oracle_gradients_match_central_differences(oracle_built, name, f, arrays, wrt):
    errs = gradcheck.grad_check(OracleBackend(), f, [a.copy() for a in arrays], wrt)
    for i, e in errs.items():
        assert e <= gradcheck.GATE, (name, i, e)
