"""IQ2_S expert tensors: the stand-alone matvec (integer partials bit-exact) and whole blocks with IQ2_S
experts, alone and mixed with IQ3_S, against the oracle."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


@pytest.mark.parametrize("cols", [256, 512, 2048])
def test_iq2s_matvec_partials_and_rows(wd, oracle, cols):
    rng = np.random.Generator(np.random.PCG64(2200 + cols))
    rows = 64
    w = ol.random_blocks(rng, ol.TYPE_IQ2_S, rows * cols // 256)
    x = rng.standard_normal(cols).astype(np.float32)
    y, part = wd.matvec(ol.TYPE_IQ2_S, w, rows, cols, x, partials=True)
    xq = oracle.quantize_q8_K(x)
    rb = cols // 256 * 82
    for r in range(rows):
        v, p = oracle.row(ol.TYPE_IQ2_S, w[r * rb:(r + 1) * rb], xq, cols, partials=True)
        assert np.array_equal(part[r].reshape(-1), p), r
        assert bits(y[r:r + 1])[0] == bits(np.array([v]))[0], r
