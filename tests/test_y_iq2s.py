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


@pytest.mark.parametrize("gu,down", [(ol.TYPE_IQ2_S, ol.TYPE_IQ2_S), (ol.TYPE_IQ2_S, ol.TYPE_IQ3_S),
                                     (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S)])
def test_blocks_with_iq2s_experts(wd, oracle, gu, down):
    from warpdecode_b200 import synth
    H, F, E, K, SF = 1024, 512, 32, 6, 256
    m = synth.make_moe_block(2300 + gu + 3 * down, H, F, E, K, SF, expert_type=gu, down_type=down)
    eng = wd.Engine(H, F, E, K, SF, 1, expert_type=gu, down_type=down)
    eng.load_block(0, m)
    rng = np.random.Generator(np.random.PCG64(2301))
    for rep in range(4):
        x = rng.standard_normal(H).astype(np.float32)
        out = eng.forward_host(0, x)
        r = oracle.moe_block(m, x)
        assert np.array_equal(eng.tap("ids"), r["ids"])
        assert np.array_equal(bits(eng.tap("act")), bits(r["act"]))
        assert np.array_equal(bits(eng.tap("expert_out")), bits(r["expert_out"]))
        assert np.array_equal(bits(out), bits(r["out"]))
    assert eng.device_status() == 0
    eng.close()


def test_iq2s_experts_through_a_capped_cache_and_a_stack(wd, oracle):
    from warpdecode_b200 import synth
    H, F, E, K, SF, L = 512, 256, 32, 4, 256, 2
    ms = [synth.make_moe_block(2400 + l, H, F, E, K, SF, expert_type=ol.TYPE_IQ2_S) for l in range(L)]
    full = wd.Engine(H, F, E, K, SF, L, expert_type=ol.TYPE_IQ2_S)
    capped = wd.Engine(H, F, E, K, SF, L, expert_type=ol.TYPE_IQ2_S, cache_mib=1)
    for l in range(L):
        full.load_block(l, ms[l])
        capped.load_block(l, ms[l])
    assert capped.slot_count() < L * E
    rng = np.random.Generator(np.random.PCG64(2402))
    res = rng.standard_normal(H).astype(np.float32)
    for step in range(3):
        ref = res.copy()
        for l in range(L):
            ref = (ref + oracle.moe_block(ms[l], oracle.rmsnorm(ref, None, 1e-6))["out"]).astype(np.float32)
        a, b = full.stack_step_host(res), capped.stack_step_host(res)
        assert np.array_equal(bits(a), bits(ref)) and np.array_equal(bits(b), bits(ref))
        res = a
    full.close(), capped.close()
