"""GPU parity of the plain-layout path: the geometries and tensor types of the reference's own model
(src/qwen38_moe.cuh:2181-2211, :2252-2258: hidden 2560, expert_ffn 640, IQ4_NL down tensors fed by a Q8_0 activation,
an F32 router), which the tiled kernels do not take. Same bar as everywhere else: every intermediate and the output
equal to the CPU oracle bit for bit, and to the golden outputs the reference composition produced."""
import os

import numpy as np
import pytest

import make_golden as mg
import oracle_lib as ol
from warpdecode_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_pins.npz"))
bits = ol.fbits


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def _engine_for(wd, m, **kw):
    return wd.Engine(m["hidden"], m["expert_ffn"], m["n_experts"], m["top_k"], m["shared_ffn"], 1,
                     expert_type=m["gate_type"], down_type=m["down_type"], w_scale=m.get("w_scale", 1.0),
                     router_f32="router_f32" in m, **kw)


def _compare(eng, r, out, token=None):
    assert np.array_equal(bits(eng.tap("logits", token)), bits(r["logits"]))
    assert np.array_equal(eng.tap("ids", token), r["ids"])
    assert np.array_equal(bits(eng.tap("weights", token)), bits(r["weights"]))
    assert np.array_equal(bits(eng.tap("act", token)), bits(r["act"]))
    assert np.array_equal(bits(eng.tap("expert_out", token)), bits(r["expert_out"]))
    assert np.array_equal(bits(eng.tap("routed", token)), bits(r["routed"]))
    if eng.cfg.shared_ffn:
        assert np.array_equal(bits(eng.tap("shared_gate", token)), bits(r["shared_gate"]))
        assert np.array_equal(bits(eng.tap("shared", token)), bits(r["shared"]))
    assert np.array_equal(bits(out), bits(r["out"]))


@pytest.mark.parametrize("bi", [4, 5, 6])
def test_blocks_outside_the_tiled_geometries_match_oracle_and_golden(wd, oracle, bi):
    m, xs = mg.block_cases()[bi]
    eng = _engine_for(wd, m)
    assert eng.kernel_name() == "plain_gate_up_kernel"
    eng.load_block(0, m)
    for xi, x in enumerate(xs):
        out = eng.forward_host(0, x)
        _compare(eng, oracle.moe_block(m, x), out)
        assert np.array_equal(bits(out), GOLD[f"block{bi}_out"][xi])
        assert np.array_equal(eng.tap("ids"), GOLD[f"block{bi}_ids"][xi])
    H = m["hidden"]
    spike = np.zeros(H, np.float32); spike[7] = 1000.0
    for x in (np.zeros(H, np.float32), spike, (xs[0] * 1e-30).astype(np.float32), (xs[0] * 1e4).astype(np.float32)):
        _compare(eng, oracle.moe_block(m, x), eng.forward_host(0, x))
    assert eng.device_status() == 0
    eng.close()


@pytest.mark.parametrize("bi", [4, 5])
def test_token_batch_equals_single_calls(wd, oracle, bi):
    m, xs = mg.block_cases()[bi]
    eng = _engine_for(wd, m, max_tokens=4)
    eng.load_block(0, m)
    outs = eng.forward_host(0, xs)
    for t in range(4):
        r = oracle.moe_block(m, xs[t])
        assert np.array_equal(bits(outs[t]), bits(r["out"]))
        assert np.array_equal(eng.tap("ids", t), r["ids"])
        assert np.array_equal(bits(eng.tap("expert_out", t)), bits(r["expert_out"]))
    eng.close()


def test_reference_model_block_shape_512_experts(wd, oracle):
    """hidden 2560, expert_ffn 640, 512 experts, top 10, IQ2_S gate/up, IQ4_NL down, F32 router with a bias, shared
    expert of 640: the block of the reference's model. Expert tensors are random block bytes with sane scales, the way
    the reference's host tests fill rows (tests/qwen38_cpu_moe_host_test.cpp:72-119); the oracle reads the same bytes."""
    H, F, E, K, SF = 2560, 640, 512, 10, 640
    rng = np.random.Generator(np.random.PCG64(77))
    m = synth.make_moe_block(5, H, F, 8, 8, SF, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=True)   # the shared expert
    m.update(n_experts=E, top_k=K, w_scale=1.25)
    m["router_f32"] = (rng.standard_normal(E * H) * 0.02).astype(np.float32)
    m["router_bias"] = (rng.standard_normal(E) * 0.5).astype(np.float32)
    m["gate"] = ol.random_blocks(rng, ol.TYPE_IQ2_S, E * F * H // 256)
    m["up"] = ol.random_blocks(rng, ol.TYPE_IQ2_S, E * F * H // 256)
    m["down"] = ol.random_blocks(rng, ol.TYPE_IQ4_NL, E * H * F // 32)
    eng = _engine_for(wd, m, max_tokens=4)
    eng.load_block(0, m)
    xs = rng.standard_normal((4, H)).astype(np.float32)
    outs = eng.forward_host(0, xs)
    for t in range(4):
        r = oracle.moe_block(m, xs[t])
        assert np.array_equal(eng.tap("ids", t), r["ids"])
        assert np.array_equal(bits(eng.tap("act", t)), bits(r["act"]))
        assert np.array_equal(bits(outs[t]), bits(r["out"]))
    _compare(eng, oracle.moe_block(m, xs[0]), eng.forward_host(0, xs[0]))
    eng.close()


def test_layers_of_different_expert_types_and_a_gguf_file(wd, oracle, tmp_path):
    """The reference model mixes IQ2_S and IQ3_S layers (src/qwen38_moe.cuh:2185-2190); the loader gives each layer
    the types the file holds."""
    m0 = synth.make_moe_block(31, 768, 192, 16, 4, 128, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=True)
    m1 = synth.make_moe_block(32, 768, 192, 16, 4, 128, ol.TYPE_IQ3_S, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=True)
    path = str(tmp_path / "plain.gguf")
    meta = {"general.architecture": "qwen4exp", "qwen4exp.embedding_length": 768, "qwen4exp.expert_count": 16,
            "qwen4exp.expert_used_count": 4, "qwen4exp.expert_feed_forward_length": 192,
            "qwen4exp.expert_shared_feed_forward_length": 128, "qwen4exp.expert_weights_scale": 1.0}
    # layer 0 stores its gate and up rows as one fused tensor (the other form the reference's loader reads); the file's
    # geometry is then read from that tensor
    synth.write_gguf(path, meta, synth.moe_block_tensors(m0, 0, fused=True) + synth.moe_block_tensors(m1, 1))
    g = wd.Gguf(path)
    eng = wd.Engine.from_gguf(g)
    x = np.random.Generator(np.random.PCG64(9)).standard_normal(768).astype(np.float32)
    for layer, m in ((0, m0), (1, m1)):
        out = eng.forward_host(layer, x)
        assert np.array_equal(bits(out), bits(oracle.moe_block(m, x)["out"]))
    eng.close()
    g.close()


def test_what_the_plain_layout_path_refuses(wd):
    """Call order and configuration errors come back as messages, not as wrong results."""
    m, xs = mg.block_cases()[5]
    with pytest.raises(wd.WdError, match="expert parallelism"):
        _engine_for(wd, m, ep_size=2, ep_rank=0)
    with pytest.raises(wd.WdError, match="resident"):           # 8 experts of this shape are 16 MiB
        _engine_for(wd, m, cache_mib=8)
    _engine_for(wd, m, cache_mib=64).close()                     # room for all of them: accepted, nothing is cached
    with pytest.raises(wd.WdError, match="4096"):
        wd.Engine(8192, 640, 64, 4, 0, 1, expert_type=ol.TYPE_IQ2_S, down_type=ol.TYPE_IQ4_NL)
    eng = _engine_for(wd, m)
    with pytest.raises(wd.WdError, match="not all set"):
        eng.forward_host(0, xs[0])
    with pytest.raises(wd.WdError, match="wd_set_router_f32"):          # the Q8_0 setter on an engine made for an F32 router
        wd._check(wd.lib().wd_set_router(eng.h, 0, np.zeros(8 * 2560 // 32 * 34, np.uint8).ctypes.data, None))
    eng.load_block(0, m)
    out = eng.forward_host(0, xs[0])
    assert np.array_equal(bits(out), GOLD["block5_out"][0])
    for call in (lambda: eng.synth_model(1), lambda: eng.set_profiling(True)):
        with pytest.raises(wd.WdError, match="plain-layout"):
            call()
    assert eng.device_status() == 0
    eng.close()
    # an engine of a tiled geometry does not take an F32 router through the Q8_0 path either
    tiled = wd.Engine(256, 256, 16, 4, 0)
    with pytest.raises(wd.WdError, match="router_f32"):
        wd._check(wd.lib().wd_set_router_f32(tiled.h, 0, np.zeros(16 * 256, np.float32).ctypes.data, None))
    tiled.close()


@pytest.mark.parametrize("shape", [(768, 192, 16, 4, 128, ol.TYPE_IQ3_S, False), (2560, 640, 8, 4, 640, ol.TYPE_IQ2_S, True)])
def test_stack_step_matches_oracle_chain(wd, oracle, shape):
    """wd_stack_step on the plain-layout path: per layer x = RMSNorm(residual) * w, residual += block(x), three layers,
    three tokens; hidden 768 and 2560 make the RMSNorm tree pad to 1024 and 4096 leaves."""
    H, F, E, K, SF, et, rf32 = shape
    L = 3
    ms = [synth.make_moe_block(60 + l, H, F, E, K, SF, et, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=rf32) for l in range(L)]
    eng = wd.Engine(H, F, E, K, SF, L, expert_type=et, down_type=ol.TYPE_IQ4_NL, router_f32=rf32, rms_eps=1e-6)
    rng = np.random.Generator(np.random.PCG64(61))
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    for l in range(L):
        eng.load_block(l, ms[l])
        eng.set_norm(l, norms[l] if l != 1 else None)        # a layer without a norm weight scales only
    res = rng.standard_normal(H).astype(np.float32)
    for step in range(3):
        got = eng.stack_step_host(res)
        ref = res.copy()
        for l in range(L):
            x = oracle.rmsnorm(ref, norms[l] if l != 1 else None, 1e-6)
            ref = (ref + oracle.moe_block(ms[l], x)["out"]).astype(np.float32)
        assert np.array_equal(bits(got), bits(ref)), step
        res = got
    assert eng.device_status() == 0
    eng.close()


@pytest.mark.parametrize("shape", [(4096, 64, 1024, 16, 128, ol.TYPE_IQ3_S, True, 4), (256, 64, 8, 1, 0, ol.TYPE_IQ2_S, False, 2),
                                   (1024, 512, 64, 8, 256, ol.TYPE_IQ2_S, True, 3)])
def test_limits_of_the_plain_layout_geometry(wd, oracle, shape):
    """The ends of what the path accepts: the widest hidden (16 superblocks, four tokens: the largest shared-memory plan of
    the rows kernel), 1,024 experts with an F32 router, top 16, the smallest expert_ffn (two IQ4_NL blocks per down row), a
    single expert per token without a shared expert; and a tiled-looking geometry (1024 / 512) that is here only because
    its down tensors are IQ4_NL. Random block bytes for the experts; every token of the batch against the oracle."""
    H, F, E, K, SF, et, rf32, T = shape
    rng = np.random.Generator(np.random.PCG64(H + E))
    m = synth.make_moe_block(71, H, F, 8, 1, SF, et, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=rf32)     # shared expert, types
    m.update(n_experts=E, top_k=K, w_scale=1.0)
    if rf32:
        m["router_f32"] = (rng.standard_normal(E * H) * 0.05).astype(np.float32)
    else:
        m["router"] = synth.quantize_q8_0((rng.standard_normal((E, H)) * 0.05).astype(np.float32)).reshape(-1)
    m["router_bias"] = (rng.standard_normal(E) * 0.3).astype(np.float32)
    m["gate"] = ol.random_blocks(rng, et, E * F * H // 256)
    m["up"] = ol.random_blocks(rng, et, E * F * H // 256)
    m["down"] = ol.random_blocks(rng, ol.TYPE_IQ4_NL, E * H * F // 32)
    eng = _engine_for(wd, m, max_tokens=T)
    eng.load_block(0, m)
    xs = rng.standard_normal((T, H)).astype(np.float32)
    outs = eng.forward_host(0, xs)
    for t in range(T):
        r = oracle.moe_block(m, xs[t])
        assert np.array_equal(eng.tap("ids", t), r["ids"])
        assert np.array_equal(bits(eng.tap("weights", t)), bits(r["weights"]))
        assert np.array_equal(bits(eng.tap("act", t)), bits(r["act"]))
        assert np.array_equal(bits(outs[t]), bits(r["out"]))
    assert eng.device_status() == 0
    eng.close()
