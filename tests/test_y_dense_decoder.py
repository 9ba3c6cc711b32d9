"""The plain (dense) Q4_0 decoder: greedy decode on the device (one CUDA-graph replay per token) against the CPU
restatement of the same step, bit for bit, on a small Llama-style model (64 generated tokens after an 8-token prompt,
as the reference's dense benchmark runs) and on layers of the benchmark model's own width."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def _oracle_for(wd, oracle, dec, cfg, rope_theta):
    tensors = {"token_embd": dec.get_tensor(0, wd.DT_TOKEN_EMBD), "output_norm": dec.get_tensor(0, wd.DT_OUTPUT_NORM),
               "output": dec.get_tensor(0, wd.DT_OUTPUT)}
    layers = []
    for l in range(cfg["n_layers"]):
        layers.append({"attn_norm": dec.get_tensor(l, wd.DT_ATTN_NORM), "wqkv": dec.get_tensor(l, wd.DT_WQKV),
                       "wo": dec.get_tensor(l, wd.DT_WO), "ffn_norm": dec.get_tensor(l, wd.DT_FFN_NORM),
                       "w_gate_up": dec.get_tensor(l, wd.DT_W_GATE_UP), "w_down": dec.get_tensor(l, wd.DT_W_DOWN)})
    return ol.DenseOracle(oracle, cfg, tensors, layers, rope_theta)


@pytest.mark.parametrize("hidden,token_kernel", [(256, False), (512, True), (512, False)])
def test_greedy_64_tokens_of_a_small_model_from_host_tensors(wd, oracle, hidden, token_kernel, monkeypatch):
    """Tensors quantised on the host by gguf-py's Q4_0 encoder and handed over in ggml layout; norms random. On the
    graph of per-operation kernels and (hidden >= 512) on the one-launch-per-token kernel."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    cfg = dict(hidden=hidden, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=1024, n_layers=2, max_ctx=96, rms_eps=1e-5)
    theta = 500000.0
    monkeypatch.setenv("WD_DENSE_TOKEN_KERNEL", "1" if token_kernel else "0")
    dec = wd.DenseDecoder(cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                          cfg["n_layers"], cfg["max_ctx"], cfg["rms_eps"], theta)
    assert (dec.kernel_name() == "dense_token_kernel") == token_kernel
    rng = np.random.Generator(np.random.PCG64(2024))

    def q4(which, layer, sigma):
        rows, cols = dec.shape(which)
        w = (rng.standard_normal((rows, cols)) * sigma).astype(np.float32)
        dec.set_tensor(layer, which, quants.quantize(w, gguf.GGMLQuantizationType.Q4_0).reshape(-1))

    def norm(which, layer):
        dec.set_tensor(layer, which, (1.0 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32))

    q4(wd.DT_TOKEN_EMBD, 0, 1.0)
    q4(wd.DT_OUTPUT, 0, 0.05)
    norm(wd.DT_OUTPUT_NORM, 0)
    for l in range(cfg["n_layers"]):
        norm(wd.DT_ATTN_NORM, l)
        norm(wd.DT_FFN_NORM, l)
        q4(wd.DT_WQKV, l, 0.08)
        q4(wd.DT_WO, l, 0.08)
        q4(wd.DT_W_GATE_UP, l, 0.08)
        q4(wd.DT_W_DOWN, l, 0.08)
    prompt = rng.integers(0, cfg["vocab"], 8)
    got, ms = dec.decode(prompt, 64)
    logits, hidden = dec.read()
    ref = _oracle_for(wd, oracle, dec, cfg, theta)
    want = ref.decode(prompt, 64)
    assert np.array_equal(got, want)                                   # 8 prompt tokens + 64 generated
    assert len(set(want[8:].tolist())) > 8                             # not a fixed point
    assert np.array_equal(ol.fbits(logits), ol.fbits(ref.logits))      # the last step's logits, bit for bit
    assert np.array_equal(ol.fbits(hidden), ol.fbits(ref.hidden))
    # a second run from position 0 gives the same tokens (the caches are rewritten, the graph is replayed)
    again, _ = dec.decode(prompt, 64)
    assert np.array_equal(again, got)
    with pytest.raises(wd.WdError, match="max_ctx"):
        dec.decode(prompt, 96)
    dec.close()


@pytest.mark.parametrize("token_kernel", [True, False])
def test_layers_of_the_benchmark_width_match_the_oracle(wd, oracle, token_kernel, monkeypatch):
    """Two layers of the dense benchmark model's shape (hidden 2048, 32 query / 8 KV heads of 64, SwiGLU 8192, RoPE
    theta 5e5), vocabulary cut to 4096 so that the oracle finishes in seconds; weights N(0, 0.02) generated on the
    device, norms 1, as the benchmark configuration says. 8 prompt tokens + 8 generated."""
    cfg = dict(hidden=2048, n_heads=32, n_kv_heads=8, head_dim=64, ffn=8192, vocab=4096, n_layers=2, max_ctx=128, rms_eps=1e-5)
    theta = 500000.0
    monkeypatch.setenv("WD_DENSE_TOKEN_KERNEL", "1" if token_kernel else "0")
    dec = wd.DenseDecoder(cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                          cfg["n_layers"], cfg["max_ctx"], cfg["rms_eps"], theta)
    assert (dec.kernel_name() == "dense_token_kernel") == token_kernel
    dec.synth(2, 0.02)
    prompt = np.random.Generator(np.random.PCG64(2)).integers(0, cfg["vocab"], 8)
    got, _ = dec.decode(prompt, 8)
    logits, hidden = dec.read()
    ref = _oracle_for(wd, oracle, dec, cfg, theta)
    want = ref.decode(prompt, 8)
    assert np.array_equal(got, want)
    assert np.array_equal(ol.fbits(logits), ol.fbits(ref.logits))
    assert np.array_equal(ol.fbits(hidden), ol.fbits(ref.hidden))
    dec.close()


def test_bad_geometry_is_refused(wd):
    with pytest.raises(wd.WdError, match="hidden"):
        wd.DenseDecoder(2560, 32, 8, 64, 8192, 1024, 1, 64)
    with pytest.raises(wd.WdError, match="n_kv_heads"):
        wd.DenseDecoder(2048, 32, 5, 64, 8192, 1024, 1, 64)
