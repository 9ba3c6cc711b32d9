"""Output head: Q8_0 matvec with the arg-max fused, against the oracle's Q8_0 rows and the reference's
arg-max rule (largest finite value, lowest index on ties, token 0 when nothing is finite)."""
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


def _ref_argmax(logits):
    """q38_argmax_kernel's rule: largest finite value, lowest index on ties, 0 when nothing is finite."""
    best, tok = None, 0
    for i, v in enumerate(logits):
        if not np.isfinite(v):
            continue
        if best is None or v > best:
            best, tok = v, i
    return tok, int(not np.all(np.isfinite(logits)))


@pytest.mark.parametrize("rows,cols", [(64, 128), (4096, 512), (19200, 256)])
def test_q8_0_head_logits_and_argmax(wd, oracle, rows, cols):
    import torch
    rng = np.random.Generator(np.random.PCG64(800 + rows))
    w = ol.random_blocks(rng, ol.TYPE_Q8_0, rows * cols // 32)
    head = wd.HeadQ8_0(rows, cols, ggml_host=w)
    rb = cols // 32 * 34
    for rep in range(3):
        x = (rng.standard_normal(cols) * [1.0, 1e-3, 30.0][rep]).astype(np.float32)
        xd = torch.from_numpy(x).cuda()
        logits = torch.zeros(rows, dtype=torch.float32, device="cuda")
        tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        nf = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        head.argmax(xd.data_ptr(), tok.data_ptr(), logits.data_ptr(), nf.data_ptr())
        torch.cuda.synchronize()
        xq = oracle.quantize_q8_0(x)
        ref = np.array([oracle.row(ol.TYPE_Q8_0, w[r * rb:(r + 1) * rb], xq, cols) for r in range(rows)], np.float32)
        assert np.array_equal(bits(logits.cpu().numpy()), bits(ref))
        want_tok, want_nf = _ref_argmax(ref)
        assert int(tok[0]) == want_tok and int(nf[0]) == want_nf
    head.close()


def test_q8_0_head_argmax_ties_zeros_and_nonfinite(wd):
    import torch
    from warpdecode_b200 import synth
    rows, cols = 64, 128
    # rows 5 and 9 identical and largest: the lower index wins; a row with an infinite scale gives a non-finite logit
    wf = np.zeros((rows, cols), np.float32)
    wf[5, :] = 1.0
    wf[9, :] = 1.0
    wf[3, :] = -1.0
    w = synth.quantize_q8_0(wf).reshape(rows, -1).copy()
    w[7, 0:2] = np.frombuffer(np.float16(np.inf).tobytes(), np.uint8)
    w[7, 2:34] = 1
    head = wd.HeadQ8_0(rows, cols, ggml_host=w.reshape(-1))
    x = torch.ones(cols, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    nf = torch.zeros(1, dtype=torch.int32, device="cuda")
    head.argmax(x.data_ptr(), tok.data_ptr(), None, nf.data_ptr())
    torch.cuda.synchronize()
    assert int(tok[0]) == 5 and int(nf[0]) == 1
    # all-zero input: every finite logit is +-0, the lowest finite index wins
    x0 = torch.zeros(cols, device="cuda")
    head.argmax(x0.data_ptr(), tok.data_ptr(), None, nf.data_ptr())
    torch.cuda.synchronize()
    assert int(tok[0]) == 0
    head.close()
