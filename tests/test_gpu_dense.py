"""Dense Q4_0 matvec (the plain decoder's operator) against the oracle's ggml-order row dot, bit for bit."""
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


def _ref_rows(oracle, w, rows, cols, x):
    xq = oracle.quantize_q8_0(x)
    rb = cols // 32 * 18
    return np.array([oracle.row(ol.TYPE_Q4_0, w[r * rb:(r + 1) * rb], xq, cols) for r in range(rows)], np.float32)


@pytest.mark.parametrize("rows,cols", [(32, 256), (64, 2048), (96, 8192), (1024, 512), (19200, 256), (20480, 1024)])
def test_q4_0_matvec_random_blocks(wd, oracle, rows, cols):
    rng = np.random.Generator(np.random.PCG64(700 + rows + cols))
    w = ol.random_blocks(rng, ol.TYPE_Q4_0, rows * cols // 32)
    x = (rng.standard_normal(cols) * rng.choice([1e-3, 1.0, 50.0])).astype(np.float32)
    y = wd.matvec(ol.TYPE_Q4_0, w, rows, cols, x)
    assert np.array_equal(bits(y), bits(_ref_rows(oracle, w, rows, cols, x)))


def test_q4_0_matvec_quantised_weights_and_edge_inputs(wd, oracle):
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(71))
    rows, cols = 64, 2048
    w = synth.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)).reshape(-1)
    for x in (np.zeros(cols, np.float32), rng.standard_normal(cols).astype(np.float32),
              np.where(np.arange(cols) % 97 == 0, 1e4, 1e-4).astype(np.float32)):
        y = wd.matvec(ol.TYPE_Q4_0, w, rows, cols, x)
        assert np.array_equal(bits(y), bits(_ref_rows(oracle, w, rows, cols, x)))
    # against the dequantised float product: the quantisation error budget, not a bit check
    x = rng.standard_normal(cols).astype(np.float32)
    y = wd.matvec(ol.TYPE_Q4_0, w, rows, cols, x)
    exact = synth.dequantize(ol.TYPE_Q4_0, w, rows, cols).astype(np.float64) @ x.astype(np.float64)
    assert np.max(np.abs(y - exact)) < 0.02 * np.max(np.abs(exact)) + 1e-3


def test_q4_0_matvec_refuses_odd_shapes(wd):
    with pytest.raises(wd.WdError, match="multiple of 32"):
        wd.matvec(ol.TYPE_Q4_0, np.zeros(33 * 8 * 18, np.uint8), 33, 256, np.zeros(256, np.float32))

