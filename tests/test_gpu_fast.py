"""The layer kernel compiled for fixed geometries (the one the 48-layer model's block runs on).

Its expert ids come from a threshold on the LOGITS, checked afterwards against the probabilities, with the
exact rungs as the fallback. The adversarial router rows of the reference's tests
(tests/router_parallel_exact_test.cu:36-76, tests/qwen38_router_host_test.cpp:181-295) must come out bit for
bit through either route: they are fed in through the router bias (a router of zero blocks gives logits =
0 + bias), at the full shape (512 experts, top-10), against the oracle's router on the same logits.
An engine runs this kernel when WD_COMPILED_KERNEL=1 is set while it is created (the generic kernel is the
default: it is the faster of the two on the 48-layer model); the stack test runs on both.
"""
import os

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
H, F, E, K, SF = 2048, 512, 512, 10, 512


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def _engine(wd, compiled, *a, **kw):
    old = os.environ.get("WD_COMPILED_KERNEL")
    os.environ["WD_COMPILED_KERNEL"] = "1" if compiled else "0"
    try:
        eng = wd.Engine(*a, **kw)
    finally:
        if old is None:
            os.environ.pop("WD_COMPILED_KERNEL", None)
        else:
            os.environ["WD_COMPILED_KERNEL"] = old
    assert eng.kernel_name() == ("moe_fast_kernel" if compiled else "moe_layer_kernel")
    return eng


@pytest.fixture(scope="module", params=["compiled", "generic"])
def head_engine(wd, request):
    """One block at the model shape on the compiled kernel, and on the generic kernel (whose ids come from the same
    threshold on the logits with the same proof)."""
    eng = _engine(wd, request.param == "compiled", H, F, E, K, SF, 1)
    eng.synth_model(11, 0.02, 0.0)
    yield eng
    eng.close()


def _set_logits(wd, eng, logits):
    zero_router = np.zeros(E * (H // 32) * 34, np.uint8)
    wd._check(wd.lib().wd_set_router(eng.h, 0, zero_router.ctypes.data, np.ascontiguousarray(logits, np.float32).ctypes.data))


def test_selection_on_adversarial_logits_matches_the_oracle_router(wd, oracle, head_engine):
    eng = head_engine
    x = np.random.Generator(np.random.PCG64(5)).standard_normal(H).astype(np.float32)
    taken = {}
    for ki, kind in enumerate(ol.ADVERSARIAL_KINDS):
        for rep in range(6):
            rng = np.random.Generator(np.random.PCG64(77000 + 40 * ki + rep))
            bias = ol.adversarial_logits(rng, E, kind)
            logits = (np.float32(0.0) + bias).astype(np.float32)          # what the kernel's 0 + bias gives
            _set_logits(wd, eng, bias)
            before = eng.fallbacks()
            eng.forward_host(0, x)
            assert eng.device_status() == 0
            _, ids, w = oracle.router(logits, K, 1.0)
            assert np.array_equal(bits(eng.tap("logits")), bits(logits)), (kind, rep)
            assert np.array_equal(eng.tap("ids"), ids), (kind, rep)
            assert np.array_equal(bits(eng.tap("weights")), bits(w)), (kind, rep)
            taken[kind] = taken.get(kind, 0) + (eng.fallbacks() - before)
    # both routes were exercised: ordinary rows stay on the threshold path, degenerate ones take the exact rungs
    assert taken["normal"] == 0 and taken["small_normal"] == 0 and taken["model_range"] == 0
    assert taken["const"] > 0 and taken["all_neg_inf"] > 0 and taken["all_underflow"] > 0


def test_crowded_and_tied_rows(wd, oracle, head_engine):
    """Rows whose winners sit in one warp's 32 experts, exact ties across the threshold, and more than 32
    candidates above the threshold."""
    eng = head_engine
    x = np.random.Generator(np.random.PCG64(6)).standard_normal(H).astype(np.float32)
    rng = np.random.Generator(np.random.PCG64(99))
    rows = []
    a = (rng.standard_normal(E) * 0.01).astype(np.float32)
    a[64:96] += 5.0                                     # all winners in one warp
    rows.append(a)
    b = np.zeros(E, np.float32)
    b[::3] = 1.0                                        # 171 equal maxima: lowest indices win, > 32 candidates
    rows.append(b)
    c = (rng.standard_normal(E)).astype(np.float32)
    c[np.argsort(c)[-12:]] = c.max()                    # a 12-way tie at the top around the cut
    rows.append(c)
    d = (rng.standard_normal(E) * 1e-4).astype(np.float32)   # probabilities collide although the logits differ
    rows.append(d)
    for i, bias in enumerate(rows):
        _set_logits(wd, eng, bias)
        eng.forward_host(0, x)
        assert eng.device_status() == 0
        _, ids, w = oracle.router((np.float32(0.0) + bias).astype(np.float32), K, 1.0)
        assert np.array_equal(eng.tap("ids"), ids), i
        assert np.array_equal(bits(eng.tap("weights")), bits(w)), i


@pytest.mark.parametrize("generic", [False, True])
def test_stack_at_the_model_shape_matches_the_oracle_chain(wd, oracle, generic):
    """Eight layers of the 48-layer model's block shape, weights generated on the device, four tokens: the final
    residual must equal the oracle chain bit for bit (the oracle needs the selected experts' bytes only). Runs on
    the compiled kernel and on the generic one."""
    L, n_tok, seed = 8, 4, 21
    eng = _engine(wd, not generic, H, F, E, K, SF, L)
    eng.synth_model(seed, 0.02, 1.0)
    rng = np.random.Generator(np.random.PCG64(8))
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    for l in range(L):
        eng.set_norm(l, norms[l])
    dense = [eng.synth_dense_host(seed, 0.02, 1.0, l) for l in range(L)]
    gb = F * (H // 256) * 110
    res = rng.standard_normal(H).astype(np.float32)
    ref = res.copy()
    for t in range(n_tok):
        res = eng.stack_step_host(res)
        assert eng.device_status() == 0
        for l in range(L):
            x = oracle.rmsnorm(ref, norms[l], 1e-6)
            xq = oracle.quantize_q8_0(x)
            rb = H // 32 * 34
            logits = np.array([oracle.row(ol.TYPE_Q8_0, dense[l]["router"][e * rb:(e + 1) * rb], xq, H) for e in range(E)],
                              np.float32) + dense[l]["router_bias"]
            _, ids, _ = oracle.router(logits.astype(np.float32), K, 1.0)
            gate, up, down = np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8)
            for e in map(int, ids):
                g, u, d = eng.synth_expert_host(seed, 0.02, l, e)
                gate[e * gb:(e + 1) * gb], up[e * gb:(e + 1) * gb], down[e * gb:(e + 1) * gb] = g, u, d
            m = dict(hidden=H, expert_ffn=F, shared_ffn=SF, n_experts=E, top_k=K, gate_type=21, up_type=21, down_type=21,
                     w_scale=1.0, gate=gate, up=up, down=down, **dense[l])
            ref = (ref + oracle.moe_block(m, x)["out"]).astype(np.float32)
        assert np.array_equal(bits(res), bits(ref)), t
    eng.close()


def test_small_block_and_taps_on_the_compiled_kernel(wd, oracle):
    """One small block with every tap, and a capped expert cache (selection pass, fill, full pass), on the compiled
    kernel: bit-equal to the oracle."""
    from warpdecode_b200 import synth
    h, f, e, k, sf = 512, 256, 32, 6, 256
    m = synth.make_moe_block(4100, h, f, e, k, sf, bias_sigma=1.0, w_scale=2.5)
    rng = np.random.Generator(np.random.PCG64(41))
    for cache_mib in (0, 1):
        eng = _engine(wd, True, h, f, e, k, sf, 1, w_scale=2.5, cache_mib=cache_mib)
        eng.load_block(0, m)
        for _ in range(3):
            x = rng.standard_normal(h).astype(np.float32)
            out = eng.forward_host(0, x)
            ref = oracle.moe_block(m, x)
            assert np.array_equal(eng.tap("ids"), ref["ids"])
            assert np.array_equal(bits(eng.tap("weights")), bits(ref["weights"]))
            assert np.array_equal(bits(eng.tap("logits")), bits(ref["logits"]))
            assert np.array_equal(bits(eng.tap("act")), bits(ref["act"]))
            assert np.array_equal(bits(eng.tap("expert_out")), bits(ref["expert_out"]))
            assert np.array_equal(bits(eng.tap("routed")), bits(ref["routed"]))
            assert np.array_equal(bits(eng.tap("shared")), bits(ref["shared"]))
            assert np.array_equal(bits(eng.tap("shared_gate")), bits(ref["shared_gate"]))
            assert np.array_equal(bits(out), bits(ref["out"]))
            assert eng.device_status() == 0
        eng.close()
