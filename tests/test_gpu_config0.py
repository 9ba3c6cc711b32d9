"""Headline block shape on the GPU: hidden 2048, 512 routed experts (IQ3_S, ffn 512), top-10, one
Q8_0 shared expert, weights N(0, 0.02) generated on the device from seed 0, 64 inputs N(0, 1)
from seed 1. Expert indices must be bit-exact and outputs within 1e-3 relative of the CPU oracle
fed the same block bytes (they are in fact bit-identical)."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def test_config0_block_64_inputs():
    import warpdecode_b200 as wd
    oracle = ol.Oracle()
    H, F, E, K, SF = 2048, 512, 512, 10, 512
    eng = wd.Engine(H, F, E, K, SF, 1)
    eng.synth_model(0, 0.02, 0.0)
    dense = eng.synth_dense_host(0, 0.02, 0.0, 0)
    gb = db = F * (H // 256) * 110
    gate, up, down = np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8), np.zeros(E * db, np.uint8)
    have = set()
    xs = np.random.Generator(np.random.PCG64(1)).standard_normal((64, H)).astype(np.float32)
    worst = 0.0
    for x in xs:
        out = eng.forward_host(0, x)
        ids = eng.tap("ids")
        for e in map(int, ids):
            if e not in have:
                g, u, d = eng.synth_expert_host(0, 0.02, 0, e)
                gate[e * gb:(e + 1) * gb], up[e * gb:(e + 1) * gb], down[e * db:(e + 1) * db] = g, u, d
                have.add(e)
        m = dict(hidden=H, expert_ffn=F, shared_ffn=SF, n_experts=E, top_k=K, gate_type=21, up_type=21,
                 down_type=21, w_scale=1.0, gate=gate, up=up, down=down, **dense)
        r = oracle.moe_block(m, x)
        assert np.array_equal(ids, r["ids"])
        worst = max(worst, float(np.max(np.abs(out - r["out"]) / np.maximum(np.abs(r["out"]), 1e-30))))
        assert np.array_equal(ol.fbits(out), ol.fbits(r["out"]))
    assert worst <= 1e-3
    assert len(have) > 100          # routing really spreads over the expert table
    assert eng.device_status() == 0
    eng.close()
