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


@pytest.mark.parametrize("cache_mib", [0, 2, 4])
def test_batch_of_tokens_equals_single_token_calls_and_oracle(wd, oracle, cache_mib):
    """cache 0: every expert resident (batch kernel); 2 MiB: 12 slots, fewer than one batch's 16 picks (the layer kernel
    walks the tokens, the host placing each token's experts); 4 MiB: 24 of the 32 experts fit (the batch kernel stops when
    a pick has no slot, the host places the batch's experts, the batch runs again)."""
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
        if n > 1 and cache_mib != 2:
            # the batch kernel keeps every token's intermediate values (all but the routed sum, which is the last token's)
            assert eng.last_kernel_name() == "moe_batch_kernel"
            r0 = oracle.moe_block(m, x[0])
            assert np.array_equal(bits(eng.tap("logits", 0)), bits(r0["logits"]))
            assert np.array_equal(bits(eng.tap("act", 0)), bits(r0["act"]))
            assert np.array_equal(bits(eng.tap("expert_out", 0)), bits(r0["expert_out"]))
            assert np.array_equal(bits(eng.tap("shared", 0)), bits(r0["shared"]))
            assert np.array_equal(bits(eng.tap("shared_gate", 0)), bits(r0["shared_gate"]))
            with pytest.raises(wd.WdError, match="earlier tokens"):
                eng.tap("routed", 0)
        elif n > 1:
            # the token walk of the layer kernel (capped cache) keeps the earlier tokens' ids and weights only
            with pytest.raises(wd.WdError, match="earlier tokens"):
                eng.tap("logits", 0)
    assert eng.device_status() == 0
    if cache_mib:
        hits, misses, evictions = eng.cache_stats()[:3]
        assert misses > 0 and hits > 0
        assert (evictions > 0) == (cache_mib == 2) or cache_mib == 4
    with pytest.raises(wd.WdError, match="max_tokens"):
        eng.forward_host(0, np.zeros((5, H), np.float32))
    eng.close()


def test_max_tokens_out_of_range_is_refused(wd):
    with pytest.raises(wd.WdError, match="max_tokens"):
        wd.Engine(H, F, E, K, SF, 1, max_tokens=5)


@pytest.mark.parametrize("batch_kernel", [True, False])
def test_batch_of_four_at_the_model_shape(wd, oracle, batch_kernel, monkeypatch):
    """Four tokens x ten experts = forty (token, slot) pairs at the 48-layer model's block shape (hidden 2048, 512
    experts, top-10), weights generated on the device. Token 3 repeats token 0, so ten of the pairs share their
    experts. One call (one launch: of the batch kernel, or with WD_BATCH_KERNEL=0 of the layer kernel walking the
    tokens) must give, for every token, the oracle's ids, weights and output bit for bit, and the same bits as four
    single-token calls. The pair map follows the reference's batch verify (p = t * k + j;
    tests/moe_batch_verify_host_test.cpp:137-186): swapping two tokens' activations must change the result (negative
    control). Batches of two and three tokens must agree with the same single-token results."""
    Hh, Fh, Eh, Kh, SFh = 2048, 512, 512, 10, 512
    monkeypatch.setenv("WD_BATCH_KERNEL", "1" if batch_kernel else "0")
    eng = wd.Engine(Hh, Fh, Eh, Kh, SFh, 1, max_tokens=4)
    assert eng.kernel_name() == "moe_layer_kernel"
    assert eng.batch_kernel_name() == ("moe_batch_kernel" if batch_kernel else "moe_layer_kernel")
    eng.synth_model(31, 0.02, 1.0)
    dense = eng.synth_dense_host(31, 0.02, 1.0, 0)
    gb = Fh * (Hh // 256) * 110
    gate, up, down = np.zeros(Eh * gb, np.uint8), np.zeros(Eh * gb, np.uint8), np.zeros(Eh * gb, np.uint8)
    x = np.random.Generator(np.random.PCG64(32)).standard_normal((4, Hh)).astype(np.float32)
    x[3] = x[0]
    out = eng.forward_host(0, x)
    ids = [eng.tap("ids", t) for t in range(4)]
    wts = [eng.tap("weights", t) for t in range(4)]
    assert eng.device_status() == 0
    for e in sorted({int(v) for t in range(4) for v in ids[t]}):
        g, u, d = eng.synth_expert_host(31, 0.02, 0, e)
        gate[e * gb:(e + 1) * gb], up[e * gb:(e + 1) * gb], down[e * gb:(e + 1) * gb] = g, u, d
    m = dict(hidden=Hh, expert_ffn=Fh, shared_ffn=SFh, n_experts=Eh, top_k=Kh, gate_type=21, up_type=21, down_type=21,
             w_scale=1.0, gate=gate, up=up, down=down, **dense)
    for t in range(4):
        r = oracle.moe_block(m, x[t])
        assert np.array_equal(ids[t], r["ids"]), t
        assert np.array_equal(bits(wts[t]), bits(r["weights"])), t
        assert np.array_equal(bits(out[t]), bits(r["out"])), t
        single = eng.forward_host(0, x[t])
        assert np.array_equal(bits(single), bits(out[t])), t
    assert np.array_equal(ids[0], ids[3]) and not np.array_equal(ids[0], ids[1])
    swapped = eng.forward_host(0, x[[1, 0, 2, 3]])
    assert np.array_equal(bits(swapped[0]), bits(out[1])) and not np.array_equal(bits(swapped[0]), bits(out[0]))
    for n in (2, 3):
        part = eng.forward_host(0, x[:n]).reshape(n, Hh)
        assert np.array_equal(bits(part), bits(out[:n])), n
        assert np.array_equal(eng.tap("ids", n - 1), ids[n - 1])
    assert eng.device_status() == 0
    eng.close()
