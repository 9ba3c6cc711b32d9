"""GPU parity tests: the CUDA path through the C ABI against the CPU oracle on the same bytes.

Integer and index work must be bit-exact. The float outputs are also compared bit for bit
(NaNs canonicalised): the kernels keep the oracle's operation order, which is stricter than the
1e-3 relative tolerance the path's contract asks for; `REL_TOL` documents that contract and is
what a deliberate re-ordering would be held to.
"""
import os

import numpy as np
import pytest

import make_golden as mg
import oracle_lib as ol

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_pins.npz"))


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()          # raises when the library is missing: there is no fallback to test instead
    return w


def bits(a):
    return ol.fbits(a)


def test_activation_quantisers_match_oracle_bytes(wd, oracle):
    x = mg.quantizer_inputs()
    assert np.array_equal(wd.quantize_q8_0(x), oracle.quantize_q8_0(x))
    assert np.array_equal(wd.quantize_q8_K(x), oracle.quantize_q8_K(x))
    assert np.array_equal(wd.quantize_q8_0(x), GOLD["q8_0"])
    assert np.array_equal(wd.quantize_q8_K(x), GOLD["q8_K"])
    rng = np.random.Generator(np.random.PCG64(5))
    for scale in (1e-6, 1.0, 300.0):
        x = (rng.standard_normal(4096) * scale).astype(np.float32)
        assert np.array_equal(wd.quantize_q8_0(x), oracle.quantize_q8_0(x))
        assert np.array_equal(wd.quantize_q8_K(x), oracle.quantize_q8_K(x))


def test_router_topk_bit_exact_on_adversarial_rows(wd, oracle):
    for ci, (kind, rep, logits, k, s) in enumerate(mg.router_cases()):
        p, ids, w = wd.router_topk(logits, k, s)
        assert np.array_equal(ids, GOLD["router_ids"][ci][:k]), (kind, rep)
        assert np.array_equal(bits(w), GOLD["router_w"][ci][:k]), (kind, rep)
        po, io, wo = oracle.router(logits, k, s)
        assert np.array_equal(bits(p), bits(po)), (kind, rep)


def test_router_topk_many_seeds(wd, oracle):
    for ki, kind in enumerate(ol.ADVERSARIAL_KINDS):
        for rep in range(12):
            rng = np.random.Generator(np.random.PCG64(91000 + 40 * ki + rep))
            logits = ol.adversarial_logits(rng, 512, kind)
            k, s = 1 + rep % 16, [1.0, 2.5, 0.5][rep % 3]
            p, ids, w = wd.router_topk(logits, k, s)
            po, io, wo = oracle.router(logits, k, s)
            assert np.array_equal(ids, io) and np.array_equal(bits(w), bits(wo)), (kind, rep)


def test_router_topk_when_one_warp_holds_most_of_the_winners(wd, oracle):
    """The selection first lists four candidates per 32 consecutive experts and repeats with full lists when
    the merge would have needed a fifth: rows whose winners crowd into one such group (0..k of them, with and
    without ties) must give the oracle's ids and weights either way."""
    for e in (512, 256, 1024):
        for rep in range(40):
            rng = np.random.Generator(np.random.PCG64(77000 + rep))
            k = [10, 8, 16, 5, 3][rep % 5]
            logits = rng.standard_normal(e).astype(np.float32)
            group = int(rng.integers(0, e // 32))
            crowd = rep % (k + 1)                                   # how many winners sit in the group
            lanes = rng.choice(32, size=min(crowd, 32), replace=False)
            boost = 6.0 + rng.standard_normal(len(lanes)).astype(np.float32)
            if rep % 4 == 3:
                boost[:] = 6.0                                       # equal winners: the lower index first
            logits[group * 32 + lanes] = boost
            if rep % 7 == 6:                                         # and the same value once outside the group
                logits[(group * 32 + 40) % e] = 6.0
            p, ids, w = wd.router_topk(logits, k, 1.0)
            po, io, wo = oracle.router(logits, k, 1.0)
            assert np.array_equal(ids, io) and np.array_equal(bits(w), bits(wo)), (e, rep)


@pytest.mark.parametrize("cols", [256, 512, 1024, 2048])
def test_iq3s_matvec_partials_and_rows(wd, oracle, cols):
    rng = np.random.Generator(np.random.PCG64(300 + cols))
    rows = 64
    w = ol.random_blocks(rng, ol.TYPE_IQ3_S, rows * cols // 256)
    x = rng.standard_normal(cols).astype(np.float32)
    y, part = wd.matvec(ol.TYPE_IQ3_S, w, rows, cols, x, partials=True)
    xq = oracle.quantize_q8_K(x)
    rb = cols // 256 * 110
    for r in range(rows):
        v, p = oracle.row(ol.TYPE_IQ3_S, w[r * rb:(r + 1) * rb], xq, cols, partials=True)
        assert np.array_equal(part[r].reshape(-1), p), r          # integer partials: bit-exact
        assert bits(y[r:r + 1])[0] == bits(np.array([v]))[0], r


def test_iq3s_matvec_negative_control(wd, oracle):
    # one flipped sign bit in one block must change exactly that row
    rng = np.random.Generator(np.random.PCG64(17))
    rows, cols = 32, 512
    w = ol.random_blocks(rng, ol.TYPE_IQ3_S, rows * cols // 256)
    x = rng.standard_normal(cols).astype(np.float32)
    y0 = wd.matvec(ol.TYPE_IQ3_S, w, rows, cols, x)
    w2 = w.copy()
    w2[5 * 220 + 110 + 74 + 3] ^= 0x10
    y1 = wd.matvec(ol.TYPE_IQ3_S, w2, rows, cols, x)
    diff = np.nonzero(bits(y0) != bits(y1))[0]
    assert list(diff) == [5]


@pytest.mark.parametrize("cols", [128, 512, 2048])
def test_q8_0_matvec_rows(wd, oracle, cols):
    rng = np.random.Generator(np.random.PCG64(400 + cols))
    rows = 64
    w = ol.random_blocks(rng, ol.TYPE_Q8_0, rows * cols // 32)
    x = rng.standard_normal(cols).astype(np.float32)
    y = wd.matvec(ol.TYPE_Q8_0, w, rows, cols, x)
    xq = oracle.quantize_q8_0(x)
    rb = cols // 32 * 34
    ref = np.array([oracle.row(ol.TYPE_Q8_0, w[r * rb:(r + 1) * rb], xq, cols) for r in range(rows)], np.float32)
    assert np.array_equal(bits(y), bits(ref))


@pytest.fixture(params=["batch_kernel", "layer_kernel"])
def single_path(request, monkeypatch):
    """One-token calls of the per-layer forward run on the batch kernel where the geometry fits it (the default) and on
    the layer kernel otherwise or with WD_BATCH_SINGLE=0: the block tests run on both."""
    monkeypatch.setenv("WD_BATCH_SINGLE", "1" if request.param == "batch_kernel" else "0")
    return request.param


def _engine_for(wd, m, n_layers=1, **kw):
    return wd.Engine(m["hidden"], m["expert_ffn"], m["n_experts"], m["top_k"], m["shared_ffn"], n_layers,
                     w_scale=m.get("w_scale", 1.0), **kw)


def _compare_block(eng, oracle, m, x, golden_out=None, path=None):
    out = eng.forward_host(0, x)
    if path is not None:
        assert eng.last_kernel_name() == ("moe_batch_kernel" if path == "batch_kernel" else "moe_layer_kernel")
    r = oracle.moe_block(m, x)
    assert np.array_equal(bits(eng.tap("logits")), bits(r["logits"]))
    assert np.array_equal(eng.tap("ids"), r["ids"])                      # expert indices: bit-exact
    assert np.array_equal(bits(eng.tap("weights")), bits(r["weights"]))
    assert np.array_equal(bits(eng.tap("act")), bits(r["act"]))
    assert np.array_equal(bits(eng.tap("expert_out")), bits(r["expert_out"]))
    assert np.array_equal(bits(eng.tap("routed")), bits(r["routed"]))
    if m["shared_ffn"]:
        assert np.array_equal(bits(eng.tap("shared_gate")), bits(r["shared_gate"]))
        assert np.array_equal(bits(eng.tap("shared")), bits(r["shared"]))
    assert np.array_equal(bits(out), bits(r["out"]))
    ok = np.isfinite(r["out"])                # an overflowing input gives the same inf/nan on both sides
    if ok.any():
        denom = np.maximum(np.abs(r["out"][ok]), 1e-30)
        assert float(np.max(np.abs(out[ok] - r["out"][ok]) / denom)) <= REL_TOL
    if golden_out is not None:
        assert np.array_equal(bits(out), golden_out)


@pytest.mark.parametrize("bi", [0, 1])
def test_moe_block_small_against_oracle_and_golden(wd, oracle, bi, single_path):
    m, xs = mg.block_cases()[bi]
    eng = _engine_for(wd, m)
    eng.load_block(0, m)
    for xi, x in enumerate(xs):
        _compare_block(eng, oracle, m, x, GOLD[f"block{bi}_out"][xi], path=single_path)
    assert eng.device_status() == 0
    eng.close()


def test_moe_block_edge_inputs(wd, oracle, single_path):
    m, xs = mg.block_cases()[0]
    eng = _engine_for(wd, m)
    eng.load_block(0, m)
    H = m["hidden"]
    zero = np.zeros(H, np.float32)                      # all-zero activations: every logit ties at 0
    spike = np.zeros(H, np.float32); spike[7] = 1000.0  # single-peak blocks
    tiny = (xs[0] * 1e-30).astype(np.float32)
    big = (xs[0] * 1e4).astype(np.float32)
    for x in (zero, spike, tiny, big):
        _compare_block(eng, oracle, m, x, path=single_path)
    eng.close()


def test_moe_block_baseline_row_shapes(wd, oracle, single_path):
    # hidden 2048 / ffn 512 / top-10 as in the headline configuration, 32 experts to keep the CPU side short
    from warpdecode_b200 import synth
    m = synth.make_moe_block(7, 2048, 512, 32, 10, 512)
    eng = _engine_for(wd, m)
    eng.load_block(0, m)
    rng = np.random.Generator(np.random.PCG64(8))
    for _ in range(3):
        _compare_block(eng, oracle, m, rng.standard_normal(2048).astype(np.float32), path=single_path)
    eng.close()


def test_moe_block_router_bias_and_scale(wd, oracle, single_path):
    from warpdecode_b200 import synth
    m = synth.make_moe_block(9, 512, 256, 64, 10, 128, bias_sigma=1.0, w_scale=2.5)
    eng = _engine_for(wd, m)
    eng.load_block(0, m)
    rng = np.random.Generator(np.random.PCG64(10))
    for _ in range(4):
        _compare_block(eng, oracle, m, rng.standard_normal(512).astype(np.float32), path=single_path)
    eng.close()


def test_moe_block_without_shared_expert(wd, oracle, single_path):
    from warpdecode_b200 import synth
    m = synth.make_moe_block(11, 256, 256, 16, 4, 0)
    eng = _engine_for(wd, m)
    eng.load_block(0, m)
    rng = np.random.Generator(np.random.PCG64(12))
    _compare_block(eng, oracle, m, rng.standard_normal(256).astype(np.float32), path=single_path)
    eng.close()


def test_stack_of_layers_matches_oracle_chain(wd, oracle):
    from warpdecode_b200 import synth
    L, H = 3, 512
    ms = [synth.make_moe_block(20 + l, H, 256, 32, 6, 256) for l in range(L)]
    eng = _engine_for(wd, ms[0], n_layers=L, rms_eps=1e-6)
    rng = np.random.Generator(np.random.PCG64(21))
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    for l in range(L):
        eng.load_block(l, ms[l])
        eng.set_norm(l, norms[l])
    res = rng.standard_normal(H).astype(np.float32)
    for step in range(3):
        got = eng.stack_step_host(res)
        ref = res.copy()
        for l in range(L):
            x = oracle.rmsnorm(ref, norms[l], 1e-6)
            ref = (ref + oracle.moe_block(ms[l], x)["out"]).astype(np.float32)
        assert np.array_equal(bits(got), bits(ref)), step
        res = got
    assert eng.device_status() == 0
    eng.close()


def test_device_generated_model_round_trips_through_oracle(wd, oracle):
    # weights generated on the GPU, copied back as ggml blocks, fed to the oracle
    H, F, E, K, SF = 1024, 256, 64, 8, 256
    eng = wd.Engine(H, F, E, K, SF, 2)
    eng.synth_model(3, 0.02, 1.0)
    rng = np.random.Generator(np.random.PCG64(31))
    for layer in (0, 1):
        dense = eng.synth_dense_host(3, 0.02, 1.0, layer)
        gb, db = F * (H // 256) * 110, H * (F // 256) * 110
        gate, up, down = np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8), np.zeros(E * db, np.uint8)
        x = rng.standard_normal(H).astype(np.float32)
        out = eng.forward_host(layer, x)
        ids = eng.tap("ids")
        for e in ids:
            g, u, d = eng.synth_expert_host(3, 0.02, layer, int(e))
            gate[e * gb:(e + 1) * gb], up[e * gb:(e + 1) * gb], down[e * db:(e + 1) * db] = g, u, d
        m = dict(hidden=H, expert_ffn=F, shared_ffn=SF, n_experts=E, top_k=K, gate_type=21, up_type=21,
                 down_type=21, w_scale=1.0, gate=gate, up=up, down=down, **dense)
        r = oracle.moe_block(m, x)
        assert np.array_equal(ids, r["ids"])
        assert np.array_equal(bits(out), bits(r["out"]))
    eng.close()


def test_unsupported_geometry_is_refused_with_a_message(wd):
    with pytest.raises(wd.WdError, match="hidden"):
        wd.Engine(2500, 512, 64, 10, 512)
    with pytest.raises(wd.WdError, match="expert_ffn"):       # 640 columns are not whole superblocks for an IQ3_S down tensor
        wd.Engine(2560, 640, 64, 10, 640)
    with pytest.raises(wd.WdError, match="top_k"):
        wd.Engine(2048, 512, 64, 32, 512)
    eng = wd.Engine(256, 256, 16, 4, 0)
    with pytest.raises(wd.WdError, match="no weights"):
        eng.forward_host(0, np.zeros(256, np.float32))
    eng.close()
