"""Pins the CPU oracle against every known-answer vector the reference's tests hold."""
import numpy as np
import pytest

from oracle.oracle import OracleFunction
from tests.golden import reference_vectors as rv


@pytest.mark.parametrize("case", rv.CASES, ids=[c.name for c in rv.CASES])
def test_oracle_matches_reference_vector(case):
    f = OracleFunction()
    out = case.build(f, *case.inputs)
    assert rv.check(out, case) == []


@pytest.mark.parametrize("name,cite,shape,layout", rv.SHAPE_CASES, ids=[c[0] for c in rv.SHAPE_CASES])
def test_oracle_sdpa_shapes(name, cite, shape, layout):
    f = OracleFunction()
    data = np.array([1, 0, 0, 1], dtype=np.float32).reshape(shape)
    out = f.FusedScaledDotProductAttention(data, data, data, None, 1, 1, layout, 1.0 / np.sqrt(2.0), False)
    assert out.shape == shape
    assert ((out > -0.1) & (out < 1.1)).all()
