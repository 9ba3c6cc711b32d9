"""Token batches (speculative verify, up to 4 tokens per call) through the per-layer forward."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
H, F, E, K, SF = 512, 256, 32, 4, 256


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


@pytest.mark.parametrize("cache_mib", [0, 2])
def test_batch_of_tokens_equals_single_token_calls_and_oracle(wd, oracle, cache_mib):
    from warpdecode_b200 import synth
    m = synth.make_moe_block(640, H, F, E, K, SF)
    eng = wd.Engine(H, F, E, K, SF, 1, max_tokens=4, cache_mib=cache_mib)
    eng.load_block(0, m)
    rng = np.random.Generator(np.random.PCG64(641))
    for n in (1, 2, 3, 4):
        x = rng.standard_normal((n, H)).astype(np.float32)
        x[n - 1] = x[0]                                   # a repeated token: same experts, same bits
        out = eng.forward_host(0, x if n > 1 else x[0])
        out = out.reshape(n, H)
        for t in range(n):
            r = oracle.moe_block(m, x[t])
            assert np.array_equal(eng.tap("ids", t), r["ids"]), (n, t)                 # pair (t, j) -> expert
            assert np.array_equal(bits(eng.tap("weights", t)), bits(r["weights"])), (n, t)
            assert np.array_equal(bits(out[t]), bits(r["out"])), (n, t)
        assert np.array_equal(bits(eng.tap("routed")), bits(oracle.moe_block(m, x[n - 1])["routed"]))
        if n > 1:
            with pytest.raises(wd.WdError, match="earlier tokens"):
                eng.tap("logits", 0)
    assert eng.device_status() == 0
    with pytest.raises(wd.WdError, match="max_tokens"):
        eng.forward_host(0, np.zeros((5, H), np.float32))
    eng.close()


def test_max_tokens_out_of_range_is_refused(wd):
    with pytest.raises(wd.WdError, match="max_tokens"):
        wd.Engine(H, F, E, K, SF, 1, max_tokens=5)
