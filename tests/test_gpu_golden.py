"""The reference's own known-answer vectors, replayed through the C ABI on the GPU."""
import numpy as np
import pytest

from tests.golden import reference_vectors as rv
from tests.util import run_backend

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", rv.CASES, ids=[c.name for c in rv.CASES])
def test_backend_matches_reference_vector(b200, backend, case):
    out = run_backend(b200, backend, case.build, case.inputs)
    assert rv.check(out, case) == []


@pytest.mark.parametrize("name,cite,shape,layout", rv.SHAPE_CASES, ids=[c[0] for c in rv.SHAPE_CASES])
def test_sdpa_shapes(b200, backend, name, cite, shape, layout):
    data = np.array([1, 0, 0, 1], dtype=np.float32).reshape(shape)
    out = run_backend(b200, backend,
                      lambda f, q, k, v: f.FusedScaledDotProductAttention(q, k, v, None, 1, 1, layout, 1.0 / np.sqrt(2.0), False),
                      [data, data, data])[0]
    assert out.shape == shape
    assert ((out > -0.1) & (out < 1.1)).all()
