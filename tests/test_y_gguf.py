"""Model load from GGUF through the library's own reader: the engine built from the file gives the bits of
the engine loaded tensor by tensor (and of the oracle), resident and with a capped cache that streams its
misses straight from the mapping."""
import numpy as np
import pytest

import oracle_lib as ol
from test_host_cpu import _tiny_gguf

pytestmark = pytest.mark.gpu


def bits(a):
    return ol.fbits(a)


@pytest.mark.parametrize("cache_mib", [0, 1])
def test_engine_from_gguf_matches_oracle(tmp_path, oracle, cache_mib):
    import warpdecode_b200 as wd
    wd.lib()
    path, ms = _tiny_gguf(tmp_path, layers=2)
    g = wd.Gguf(path)
    eng = wd.Engine.from_gguf(g, cache_mib=cache_mib)
    if cache_mib:
        assert eng.slot_count() < 2 * 8
    rng = np.random.Generator(np.random.PCG64(88))
    for l, m in enumerate(ms):
        x = rng.standard_normal(256).astype(np.float32)
        r = oracle.moe_block(m, x)
        assert np.array_equal(bits(eng.forward_host(l, x)), bits(r["out"]))
        assert np.array_equal(eng.tap("ids"), r["ids"])
    # the stack uses the file's ffn_norm weights and epsilon
    res = rng.standard_normal(256).astype(np.float32)
    ref = res.copy()
    for l, m in enumerate(ms):
        ref = (ref + oracle.moe_block(m, oracle.rmsnorm(ref, np.full(256, 1.0 + l, np.float32), 1e-5))["out"]).astype(np.float32)
    assert np.array_equal(bits(eng.stack_step_host(res)), bits(ref))
    eng.close()
    g.close()
