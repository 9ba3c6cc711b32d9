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
    """The CPU restatement fed with the decoder's own tensors (bytes and block types as it holds them)."""
    tensors = {"token_embd": dec.get_tensor(0, wd.DT_TOKEN_EMBD), "output_norm": dec.get_tensor(0, wd.DT_OUTPUT_NORM),
               "output": dec.get_tensor(0, wd.DT_OUTPUT), "token_embd_type": dec.tensor_type(0, wd.DT_TOKEN_EMBD),
               "output_type": dec.tensor_type(0, wd.DT_OUTPUT)}
    layers = []
    for l in range(cfg["n_layers"]):
        layers.append({"attn_norm": dec.get_tensor(l, wd.DT_ATTN_NORM), "wqkv": dec.get_tensor(l, wd.DT_WQKV),
                       "wo": dec.get_tensor(l, wd.DT_WO), "ffn_norm": dec.get_tensor(l, wd.DT_FFN_NORM),
                       "w_gate_up": dec.get_tensor(l, wd.DT_W_GATE_UP), "w_down": dec.get_tensor(l, wd.DT_W_DOWN),
                       "wqkv_type": dec.tensor_type(l, wd.DT_WQKV), "wo_type": dec.tensor_type(l, wd.DT_WO),
                       "w_gate_up_type": dec.tensor_type(l, wd.DT_W_GATE_UP), "w_down_type": dec.tensor_type(l, wd.DT_W_DOWN)})
        for key, which in (("bqkv", wd.DT_BQKV), ("q_norm", wd.DT_Q_NORM), ("k_norm", wd.DT_K_NORM)):
            try:
                layers[-1][key] = dec.get_tensor(l, which)       # the optional vectors, when the model has them
            except wd.WdError:
                pass
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


@pytest.mark.parametrize("style", ["llama", "qwen2", "qwen3"])
def test_model_file_in_the_reference_loaders_tensor_names(wd, oracle, tmp_path, style):
    """A Llama-style Q4_0 GGUF as the reference's dense loader reads it (load_model, src/warodecode.cu:1255-1345): separate
    attn_q / attn_k / attn_v and ffn_gate / ffn_up tensors, no output.weight (tied to the embedding table). The decoder
    built from the file decodes the same 40 tokens as the CPU restatement fed with the same bytes."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from warpdecode_b200 import synth
    H, nh, nkv, hd, F, V, L = 256, 4, 2, 64, 512, 768, 2
    rng = np.random.Generator(np.random.PCG64(77))
    q4 = lambda rows, cols, sigma: quants.quantize((rng.standard_normal((rows, cols)) * sigma).astype(np.float32),
                                                   gguf.GGMLQuantizationType.Q4_0).reshape(-1)
    vec = lambda: (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    tensors = [("token_embd.weight", [H, V], ol.TYPE_Q4_0, q4(V, H, 0.3)), ("output_norm.weight", [H], ol.TYPE_F32, vec())]
    for l in range(L):
        p = f"blk.{l}."
        tensors += [(p + "attn_norm.weight", [H], ol.TYPE_F32, vec()), (p + "ffn_norm.weight", [H], ol.TYPE_F32, vec()),
                    (p + "attn_q.weight", [H, nh * hd], ol.TYPE_Q4_0, q4(nh * hd, H, 0.08)),
                    (p + "attn_k.weight", [H, nkv * hd], ol.TYPE_Q4_0, q4(nkv * hd, H, 0.08)),
                    (p + "attn_v.weight", [H, nkv * hd], ol.TYPE_Q4_0, q4(nkv * hd, H, 0.08)),
                    (p + "attn_output.weight", [H, H], ol.TYPE_Q4_0, q4(H, nh * hd, 0.08)),
                    (p + "ffn_gate.weight", [H, F], ol.TYPE_Q4_0, q4(F, H, 0.08)),
                    (p + "ffn_up.weight", [H, F], ol.TYPE_Q4_0, q4(F, H, 0.08)),
                    (p + "ffn_down.weight", [F, H], ol.TYPE_Q4_0, q4(H, F, 0.08))]
    # Qwen2-style files carry q/k/v biases (here: k's is absent, which reads as zeros), Qwen3-style ones RMSNorm weights
    # for the q and k heads (load_model, src/warodecode.cu:1305-1309)
    if style == "qwen2":
        for l in range(L):
            tensors += [(f"blk.{l}.attn_q.bias", [nh * hd], ol.TYPE_F32, (0.2 * rng.standard_normal(nh * hd)).astype(np.float32)),
                        (f"blk.{l}.attn_v.bias", [nkv * hd], ol.TYPE_F32, (0.2 * rng.standard_normal(nkv * hd)).astype(np.float32))]
    if style == "qwen3":
        for l in range(L):
            tensors += [(f"blk.{l}.attn_q_norm.weight", [hd], ol.TYPE_F32, (1.0 + 0.2 * rng.standard_normal(hd)).astype(np.float32)),
                        (f"blk.{l}.attn_k_norm.weight", [hd], ol.TYPE_F32, (1.0 + 0.2 * rng.standard_normal(hd)).astype(np.float32))]
    meta = {"general.architecture": style, f"{style}.embedding_length": H, f"{style}.block_count": L,
            f"{style}.attention.head_count": nh, f"{style}.attention.head_count_kv": nkv, f"{style}.feed_forward_length": F,
            f"{style}.attention.layer_norm_rms_epsilon": 1e-5, f"{style}.rope.freq_base": 500000.0}
    path = str(tmp_path / "dense.gguf")
    synth.write_gguf(path, meta, tensors)
    g = wd.Gguf(path)
    dec = wd.DenseDecoder.from_gguf(g, 64)
    g.close()                                   # every tensor was copied to the device
    c = dec.cfg
    assert (c.hidden, c.n_heads, c.n_kv_heads, c.head_dim, c.ffn, c.vocab, c.n_layers) == (H, nh, nkv, hd, F, V, L)
    by_name = {n: d for n, _, _, d in tensors}
    assert np.array_equal(dec.get_tensor(0, wd.DT_OUTPUT), by_name["token_embd.weight"])         # tied
    assert np.array_equal(dec.get_tensor(1, wd.DT_WQKV), np.concatenate([by_name["blk.1.attn_q.weight"], by_name["blk.1.attn_k.weight"],
                                                                         by_name["blk.1.attn_v.weight"]]))
    cfg = dict(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, ffn=F, vocab=V, n_layers=L, max_ctx=64, rms_eps=c.rms_eps)
    prompt = rng.integers(0, V, 8)
    got, _ = dec.decode(prompt, 32)
    want = _oracle_for(wd, oracle, dec, cfg, 500000.0).decode(prompt, 32)
    assert np.array_equal(got, want) and len(set(want[8:].tolist())) > 1
    dec.close()
    # what the step does not have is refused by name
    synth.write_gguf(path, dict(meta, **{f"{style}.rope.scaling.type": "yarn"}), tensors)
    g = wd.Gguf(path)
    with pytest.raises(wd.WdError, match="yarn"):
        wd.DenseDecoder.from_gguf(g, 64)
    g.close()
    synth.write_gguf(path, dict(meta, **{"general.architecture": "qwen4exp"}), tensors)
    g = wd.Gguf(path)
    with pytest.raises(wd.WdError, match="architecture"):
        wd.DenseDecoder.from_gguf(g, 64)
    g.close()


def _random_q6_k(rng, rows, cols):
    """Q6_K blocks (210 bytes per 256 values) with random quants, small int8 sub-scales and f16 scales: valid input for
    the decoder of that type; gguf-py has no encoder for it."""
    n = rows * cols // 256
    blk = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
    blk[:, 192:208] = rng.integers(-24, 25, size=(n, 16)).astype(np.int8).view(np.uint8)
    blk[:, 208:210] = rng.uniform(2e-4, 1e-3, n).astype(np.float16).view(np.uint8).reshape(n, 2)
    return blk.reshape(-1)


def test_model_file_with_q6_k_and_q8_0_tensors(wd, oracle, tmp_path):
    """The Q4_0 files that llama.cpp writes keep the output head in Q6_K and some ffn_down tensors in Q8_0; the
    reference's dense loader requantises every 2-D tensor that is not Q4_0 to Q8_0 on the host and multiplies with that
    (planarize_q4, src/warodecode.cu:1027-1075; ggml_requantize_row_to_q8_0, src/ggml_dequant.hpp:362-392). Here: a tied
    Q6_K embedding table (so the embedding row comes from Q8_0 blocks too), Q8_0 ffn_down in layer 1, Q8_0 q/k/v in
    layer 0. The tensors the decoder holds equal the oracle's requantiser on the file's bytes; 32 tokens equal the oracle."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from warpdecode_b200 import synth
    H, nh, nkv, hd, F, V, L = 256, 4, 2, 64, 512, 640, 2
    rng = np.random.Generator(np.random.PCG64(99))
    enc = lambda rows, cols, sigma, t: quants.quantize((rng.standard_normal((rows, cols)) * sigma).astype(np.float32), t).reshape(-1)
    q4 = lambda rows, cols, sigma=0.08: enc(rows, cols, sigma, gguf.GGMLQuantizationType.Q4_0)
    q8 = lambda rows, cols, sigma=0.08: enc(rows, cols, sigma, gguf.GGMLQuantizationType.Q8_0)
    vec = lambda: (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    emb = _random_q6_k(rng, V, H)
    tensors = [("token_embd.weight", [H, V], ol.TYPE_Q6_K, emb), ("output_norm.weight", [H], ol.TYPE_F32, vec())]
    for l in range(L):
        p = f"blk.{l}."
        qt, qf = (ol.TYPE_Q8_0, q8) if l == 0 else (ol.TYPE_Q4_0, q4)
        dt, df = (ol.TYPE_Q8_0, q8) if l == 1 else (ol.TYPE_Q4_0, q4)
        tensors += [(p + "attn_norm.weight", [H], ol.TYPE_F32, vec()), (p + "ffn_norm.weight", [H], ol.TYPE_F32, vec()),
                    (p + "attn_q.weight", [H, nh * hd], qt, qf(nh * hd, H)), (p + "attn_k.weight", [H, nkv * hd], qt, qf(nkv * hd, H)),
                    (p + "attn_v.weight", [H, nkv * hd], qt, qf(nkv * hd, H)),
                    (p + "attn_output.weight", [H, H], ol.TYPE_Q4_0, q4(H, nh * hd)),
                    (p + "ffn_gate.weight", [H, F], ol.TYPE_Q4_0, q4(F, H)), (p + "ffn_up.weight", [H, F], ol.TYPE_Q4_0, q4(F, H)),
                    (p + "ffn_down.weight", [F, H], dt, df(H, F))]
    meta = {"general.architecture": "llama", "llama.embedding_length": H, "llama.block_count": L,
            "llama.attention.head_count": nh, "llama.attention.head_count_kv": nkv, "llama.feed_forward_length": F,
            "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0}
    path = str(tmp_path / "mixed.gguf")
    synth.write_gguf(path, meta, tensors)
    g = wd.Gguf(path)
    dec = wd.DenseDecoder.from_gguf(g, 64)
    g.close()
    by_name = {n: d for n, _, _, d in tensors}
    assert dec.tensor_type(0, wd.DT_TOKEN_EMBD) == ol.TYPE_Q8_0 and dec.tensor_type(0, wd.DT_OUTPUT) == ol.TYPE_Q8_0
    assert dec.tensor_type(0, wd.DT_WQKV) == ol.TYPE_Q8_0 and dec.tensor_type(1, wd.DT_WQKV) == ol.TYPE_Q4_0
    assert dec.tensor_type(1, wd.DT_W_DOWN) == ol.TYPE_Q8_0 and dec.tensor_type(0, wd.DT_W_DOWN) == ol.TYPE_Q4_0
    assert np.array_equal(dec.get_tensor(0, wd.DT_TOKEN_EMBD), oracle.requantize_rows_to_q8_0(ol.TYPE_Q6_K, emb, V, H))
    assert np.array_equal(dec.get_tensor(1, wd.DT_W_DOWN), oracle.requantize_rows_to_q8_0(ol.TYPE_Q8_0, by_name["blk.1.ffn_down.weight"], H, F))
    cfg = dict(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, ffn=F, vocab=V, n_layers=L, max_ctx=64, rms_eps=dec.cfg.rms_eps)
    prompt = rng.integers(0, V, 8)
    got, _ = dec.decode(prompt, 32)
    logits, hidden = dec.read()
    ref = _oracle_for(wd, oracle, dec, cfg, 10000.0)
    want = ref.decode(prompt, 32)
    assert np.array_equal(got, want)
    assert np.array_equal(ol.fbits(logits), ol.fbits(ref.logits)) and np.array_equal(ol.fbits(hidden), ol.fbits(ref.hidden))
    dec.close()
    # q/k/v parts of different types are refused by name
    bad = [(n, d, (ol.TYPE_Q4_0 if n == "blk.0.attn_k.weight" else t), (q4(nkv * hd, H) if n == "blk.0.attn_k.weight" else a))
           for n, d, t, a in tensors]
    synth.write_gguf(path, meta, bad)
    g = wd.Gguf(path)
    with pytest.raises(wd.WdError, match="differ in type"):
        wd.DenseDecoder.from_gguf(g, 64)
    g.close()


def test_cpp_runtime_wrapper_decodes_a_model_file(wd, oracle, tmp_path):
    """include/warpdecode_b200.hpp's Model / load_model / Runtime (the reference's dense entry points,
    src/warodecode.cu:1255, :2011-2150) run a small model file end to end from C++; the hash of the 64 generated tokens
    equals the one of the tokens the Python binding decodes from the same file."""
    import os
    import shutil
    import subprocess
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    from warpdecode_b200 import synth
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    H, nh, nkv, hd, F, V, L = 256, 4, 2, 64, 512, 512, 2
    rng = np.random.Generator(np.random.PCG64(5))
    q4 = lambda rows, cols, sigma: quants.quantize((rng.standard_normal((rows, cols)) * sigma).astype(np.float32),
                                                   gguf.GGMLQuantizationType.Q4_0).reshape(-1)
    vec = lambda: (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    tensors = [("token_embd.weight", [H, V], ol.TYPE_Q4_0, q4(V, H, 0.3)), ("output_norm.weight", [H], ol.TYPE_F32, vec()),
               ("output.weight", [H, V], ol.TYPE_Q4_0, q4(V, H, 0.05))]
    for l in range(L):
        p = f"blk.{l}."
        tensors += [(p + "attn_norm.weight", [H], ol.TYPE_F32, vec()), (p + "ffn_norm.weight", [H], ol.TYPE_F32, vec()),
                    (p + "attn_q.weight", [H, H], ol.TYPE_Q4_0, q4(H, H, 0.08)), (p + "attn_k.weight", [H, nkv * hd], ol.TYPE_Q4_0, q4(nkv * hd, H, 0.08)),
                    (p + "attn_v.weight", [H, nkv * hd], ol.TYPE_Q4_0, q4(nkv * hd, H, 0.08)),
                    (p + "attn_output.weight", [H, H], ol.TYPE_Q4_0, q4(H, H, 0.08)), (p + "ffn_gate.weight", [H, F], ol.TYPE_Q4_0, q4(F, H, 0.08)),
                    (p + "ffn_up.weight", [H, F], ol.TYPE_Q4_0, q4(F, H, 0.08)), (p + "ffn_down.weight", [F, H], ol.TYPE_Q4_0, q4(H, F, 0.08))]
    meta = {"general.architecture": "llama", "llama.embedding_length": H, "llama.block_count": L, "llama.attention.head_count": nh,
            "llama.attention.head_count_kv": nkv, "llama.feed_forward_length": F, "llama.attention.layer_norm_rms_epsilon": 1e-5,
            "llama.rope.freq_base": 10000.0}
    path = str(tmp_path / "rt.gguf")
    synth.write_gguf(path, meta, tensors)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe, libdir = str(tmp_path / "boundary_check"), os.path.dirname(wd.LIB_PATH)
    r = subprocess.run(["g++", "-std=c++17", "-I", os.path.join(root, "include"), "-o", exe, os.path.join(root, "tests", "boundary_check.cpp"),
                        "-L", libdir, "-lwarpdecode_b200", f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe, "/nonexistent.gguf", path], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("dense:")][0]
    g = wd.Gguf(path)
    dec = wd.DenseDecoder.from_gguf(g, 128)
    g.close()
    toks, _ = dec.decode(np.array([1]), 64)
    h = 1469598103934665603
    for t in toks[1:]:
        for b in range(4):
            h = ((h ^ ((int(t) >> (8 * b)) & 0xff)) * 1099511628211) & 0xffffffffffffffff
    assert line.startswith("dense: 2 layers") and line.endswith("hash %x" % h), (line, hex(h))
    want = _oracle_for(wd, oracle, dec, dict(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, ffn=F, vocab=V, n_layers=L, max_ctx=128,
                                             rms_eps=dec.cfg.rms_eps), 10000.0).decode(np.array([1]), 64)
    assert np.array_equal(toks, want)
    dec.close()
