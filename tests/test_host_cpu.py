"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, the
synthetic encoders produce blocks their own decoders (and gguf-py's, when importable) read back,
and the GGUF writer round-trips."""
import ctypes
import os
import re

import numpy as np
import pytest

import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_every_declared_symbol():
    import warpdecode_b200 as wd
    path = wd.build()
    L = ctypes.CDLL(path)
    header = open(os.path.join(ROOT, "include", "warpdecode_b200.h")).read()
    names = set(re.findall(r"\b(wd_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 25
    for n in sorted(names):
        assert hasattr(L, n), n
    assert L.wd_version() >= 1


def test_default_cache_rule_and_env_override(monkeypatch):
    import warpdecode_b200 as wd
    L = wd.lib()
    monkeypatch.delenv("WARODECODE_EXPERT_CACHE_MIB", raising=False)
    assert L.wd_default_cache_mib(40 * 1024) == 40 * 1024 * 3 // 4 - 8192          # 22 GiB on a 40 GB card
    assert L.wd_default_cache_mib(183359) == 65536                                  # clamp high
    assert L.wd_default_cache_mib(8 * 1024) == 512                                  # clamp low
    monkeypatch.setenv("WARODECODE_EXPERT_CACHE_MIB", "8192")
    assert L.wd_default_cache_mib(183359) == 8192
    monkeypatch.setenv("WARODECODE_EXPERT_CACHE_MIB", "-3")
    assert L.wd_default_cache_mib(183359) == 65536


@pytest.mark.parametrize("t", [ol.TYPE_Q8_0, ol.TYPE_Q4_0, ol.TYPE_IQ3_S, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL])
def test_synth_encoders_decode_close_to_the_weights(t):
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(3))
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    blob = synth.QUANTIZERS[t](w)
    assert blob.shape == (8, synth.row_bytes(t, 512))
    back = synth.dequantize(t, blob, 8, 512)
    rel = np.linalg.norm(back - w) / np.linalg.norm(w)
    assert rel < {ol.TYPE_Q8_0: 0.01, ol.TYPE_Q4_0: 0.12, ol.TYPE_IQ3_S: 0.35, ol.TYPE_IQ2_S: 0.6, ol.TYPE_IQ4_NL: 0.12}[t]
    try:
        import gguf
        from gguf import quants
    except Exception:
        return
    qt = {ol.TYPE_Q8_0: gguf.GGMLQuantizationType.Q8_0, ol.TYPE_Q4_0: gguf.GGMLQuantizationType.Q4_0,
          ol.TYPE_IQ3_S: gguf.GGMLQuantizationType.IQ3_S, ol.TYPE_IQ2_S: gguf.GGMLQuantizationType.IQ2_S,
          ol.TYPE_IQ4_NL: gguf.GGMLQuantizationType.IQ4_NL}[t]
    theirs = quants.dequantize(blob, qt)
    assert np.array_equal(theirs.astype(np.float32), back.astype(np.float32))


def test_oracle_rows_agree_with_dequantised_weights(oracle):
    # the row dot of the oracle equals sum(dequant(w) * dequant(q8k(x))) up to float rounding
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(4))
    w = (rng.standard_normal((4, 512)) * 0.02).astype(np.float32)
    x = rng.standard_normal(512).astype(np.float32)
    for t in (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S):
        blob = synth.QUANTIZERS[t](w)
        wf = synth.dequantize(t, blob, 4, 512).astype(np.float64)
        xq = oracle.quantize_q8_K(x)
        xf = np.concatenate([xq[i * 292 + 4:i * 292 + 260].view(np.int8).astype(np.float64) *
                             float(xq[i * 292:i * 292 + 4].view(np.float32)[0]) for i in range(2)])
        for r in range(4):
            got = float(oracle.row(t, blob[r], xq, 512))
            assert abs(got - float(wf[r] @ xf)) <= 1e-4 * max(1.0, abs(got))


def test_gguf_writer_round_trip(tmp_path):
    from warpdecode_b200 import synth
    m = synth.make_moe_block(5, 256, 256, 8, 2, 128)
    path = str(tmp_path / "tiny.gguf")
    meta = {"general.architecture": "qwen4exp", "qwen4exp.block_count": 1, "qwen4exp.expert_count": 8,
            "qwen4exp.expert_used_count": 2, "qwen4exp.embedding_length": 256,
            "qwen4exp.expert_feed_forward_length": 256, "qwen4exp.expert_weights_scale": 1.0}
    synth.write_gguf(path, meta, synth.moe_block_tensors(m, 0))
    try:
        import gguf
    except Exception:
        pytest.skip("gguf-py not importable")
    r = gguf.GGUFReader(path)
    names = {t.name: t for t in r.tensors}
    t = names["blk.0.ffn_gate_exps.weight"]
    assert list(map(int, t.shape)) == [256, 256, 8]
    assert int(t.tensor_type) == ol.TYPE_IQ3_S
    assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), m["gate"])
    assert np.array_equal(np.asarray(names["blk.0.ffn_gate_inp_shexp.weight"].data).reshape(-1), m["shared_gate_vec"])


def _tiny_gguf(tmp_path, layers=2, expert_type=None, bias=True, name="m.gguf"):
    from warpdecode_b200 import synth
    kw = {} if expert_type is None else {"expert_type": expert_type}
    ms = [synth.make_moe_block(60 + l, 256, 256, 8, 2, 128, bias_sigma=1.0 if bias else 0.0, w_scale=2.5, **kw)
          for l in range(layers)]
    meta = {"general.architecture": "qwen4exp", "qwen4exp.block_count": layers, "qwen4exp.expert_count": 8,
            "qwen4exp.expert_used_count": 2, "qwen4exp.embedding_length": 256,
            "qwen4exp.expert_feed_forward_length": 256, "qwen4exp.expert_shared_feed_forward_length": 128,
            "qwen4exp.expert_weights_scale": 2.5, "qwen4exp.attention.layer_norm_rms_epsilon": 1e-5,
            "general.name": "tiny", "qwen4exp.rope.dimension_sections": [1, 2, 3]}
    tensors = []
    for l, m in enumerate(ms):
        tensors += synth.moe_block_tensors(m, l)
        tensors.append((f"blk.{l}.ffn_norm.weight", [256], ol.TYPE_F32, np.full(256, 1.0 + l, np.float32)))
    path = str(tmp_path / name)
    synth.write_gguf(path, meta, tensors)
    return path, ms


def test_gguf_reader_geometry_and_tensors_without_a_gpu(tmp_path):
    """The C++ GGUF reader of the library (no CUDA call involved): geometry from keys and tensors, tensor
    pointers into the mapping equal to the bytes that were written."""
    import warpdecode_b200 as wd
    path, ms = _tiny_gguf(tmp_path)
    g = wd.Gguf(path)
    c = g.config()
    assert (c.hidden, c.expert_ffn, c.shared_ffn, c.n_experts, c.top_k, c.n_layers) == (256, 256, 128, 8, 2, 2)
    assert (c.gate_type, c.up_type, c.down_type) == (ol.TYPE_IQ3_S,) * 3
    assert c.w_scale == 2.5 and abs(c.rms_eps - 1e-5) < 1e-12
    for l, m in enumerate(ms):
        data, t, dims = g.tensor(f"blk.{l}.ffn_down_exps.weight")
        assert (t, dims) == (ol.TYPE_IQ3_S, [256, 256, 8]) and np.array_equal(data, m["down"])
        data, t, dims = g.tensor(f"blk.{l}.ffn_gate_inp.weight")
        assert (t, dims) == (ol.TYPE_Q8_0, [256, 8]) and np.array_equal(data, m["router"])
        data, t, dims = g.tensor(f"blk.{l}.ffn_gate_inp.bias")
        assert t == ol.TYPE_F32 and np.array_equal(data.view(np.float32), m["router_bias"])
    with pytest.raises(wd.WdError, match="no tensor"):
        g.tensor("blk.9.ffn_gate_inp.weight")
    g.close()
    # IQ2_S experts are recognised by their tensor type
    path2, _ = _tiny_gguf(tmp_path, layers=1, expert_type=ol.TYPE_IQ2_S, name="iq2.gguf")
    g2 = wd.Gguf(path2)
    assert g2.config().gate_type == ol.TYPE_IQ2_S and g2.config().n_layers == 1
    g2.close()


def test_gguf_reader_takes_the_reference_models_tensor_forms(tmp_path):
    """A file shaped like the reference's own model (src/qwen38_moe.cuh:601-612, :2181-2258): F32 router, IQ4_NL down
    tensors, hidden that is not a power of two, expert_ffn a multiple of 64, gate and up rows fused into one tensor in
    the first layer. The geometry comes out of the fused tensor; no CUDA call is involved."""
    import warpdecode_b200 as wd
    from warpdecode_b200 import synth
    ms = [synth.make_moe_block(40 + l, 768, 192, 8, 2, 128, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=True)
          for l in range(2)]
    path = str(tmp_path / "ref_forms.gguf")
    meta = {"general.architecture": "qwen4exp", "qwen4exp.embedding_length": 768, "qwen4exp.expert_count": 8,
            "qwen4exp.expert_used_count": 2, "qwen4exp.expert_feed_forward_length": 192,
            "qwen4exp.expert_shared_feed_forward_length": 128}
    synth.write_gguf(path, meta, synth.moe_block_tensors(ms[0], 0, fused=True) + synth.moe_block_tensors(ms[1], 1))
    g = wd.Gguf(path)
    c = g.config()
    assert (c.hidden, c.expert_ffn, c.shared_ffn, c.n_experts, c.top_k, c.n_layers) == (768, 192, 128, 8, 2, 2)
    assert (c.gate_type, c.up_type, c.down_type, c.router_f32) == (ol.TYPE_IQ2_S, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, 1)
    data, t, dims = g.tensor("blk.0.ffn_gate_up_exps.weight")
    assert (t, dims) == (ol.TYPE_IQ2_S, [768, 384, 8])
    rb = 192 * 3 * 82                    # one expert's gate (or up) rows
    fused = data.reshape(8, 2 * rb)
    assert np.array_equal(fused[:, :rb].reshape(-1), ms[0]["gate"]) and np.array_equal(fused[:, rb:].reshape(-1), ms[0]["up"])
    data, t, dims = g.tensor("blk.1.ffn_gate_inp.weight")
    assert (t, dims) == (ol.TYPE_F32, [768, 8]) and np.array_equal(data.view(np.float32), ms[1]["router_f32"])
    data, t, dims = g.tensor("blk.1.ffn_down_exps.weight")
    assert (t, dims) == (ol.TYPE_IQ4_NL, [192, 768, 8]) and np.array_equal(data, ms[1]["down"])
    g.close()


def test_oracle_f32_router_block_against_the_reference_any_thread_count(oracle, reference):
    """The reference composition run live (when its sources are present): F32 router, IQ4_NL down, hidden 2560."""
    from warpdecode_b200 import synth
    m = synth.make_moe_block(9, 2560, 640, 8, 4, 640, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, sigma=0.02, router_f32=True, w_scale=1.25)
    x = np.random.Generator(np.random.PCG64(10)).standard_normal(2560).astype(np.float32)
    o = oracle.moe_block(m, x)
    for th in (1, 3, 8):
        r = reference.moe_block(m, x, threads=th)
        assert np.array_equal(r["ids"], o["ids"]) and np.array_equal(ol.fbits(r["out"]), ol.fbits(o["out"]))


def test_gguf_reader_refuses_broken_files(tmp_path):
    import warpdecode_b200 as wd
    path, _ = _tiny_gguf(tmp_path, layers=1)
    blob = open(path, "rb").read()
    cases = {"magic": b"GGXX" + blob[4:], "version": blob[:4] + (9).to_bytes(4, "little") + blob[8:],
             "short": blob[:200], "data": blob[:len(blob) // 2]}
    for name, b in cases.items():
        p = str(tmp_path / (name + ".gguf"))
        open(p, "wb").write(b)
        with pytest.raises(wd.WdError, match="GGUF|too short"):
            wd.Gguf(p)
    with pytest.raises(wd.WdError, match="cannot open"):
        wd.Gguf(str(tmp_path / "missing.gguf"))
    # a key that disagrees with the tensors
    from warpdecode_b200 import synth
    m = synth.make_moe_block(5, 256, 256, 8, 2, 128)
    p = str(tmp_path / "liar.gguf")
    synth.write_gguf(p, {"general.architecture": "qwen4exp", "qwen4exp.expert_used_count": 2,
                         "qwen4exp.expert_count": 16}, synth.moe_block_tensors(m, 0))
    g = wd.Gguf(p)
    with pytest.raises(wd.WdError, match="disagrees"):
        g.config()
    g.close()


def test_cpp_wrappers_with_the_reference_signatures_compile_link_and_report_errors(tmp_path):
    """include/warpdecode_b200.hpp (the reference's C++ entry points over the C ABI) meets a compiler: the call sites
    of tests/boundary_check.cpp, written like the reference decoder's, compile with -Wall -Wextra against stand-ins
    for the CUDA names, link against the built library, and a load that cannot succeed here (no file, or no GPU)
    ends in std::runtime_error with the library's message, as the reference's callers expect."""
    import shutil
    import subprocess
    import warpdecode_b200 as wd
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    wd.build()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "boundary_check")
    libdir = os.path.dirname(wd.LIB_PATH)
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(root, "include"), "-o", exe,
                        os.path.join(root, "tests", "boundary_check.cpp"), "-L", libdir, "-lwarpdecode_b200",
                        f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "runtime_error: warpdecode_b200: cannot open" in r.stdout
    assert r.stdout.count("runtime_error: warpdecode_b200: cannot open") == 2       # the MoE runtime and the dense load_model


def test_dense_model_file_refusals_need_no_gpu(tmp_path):
    """What wd_dense_decoder_load_gguf refuses is decided from the file's keys before any CUDA call (load_model,
    src/warodecode.cu:1255-1284): another architecture, missing geometry, partial or scaled rotary embeddings."""
    import ctypes as C
    import warpdecode_b200 as wd
    from warpdecode_b200 import synth
    emb = np.zeros(64 * (256 // 32) * 18, np.uint8)
    base = {"general.architecture": "llama", "llama.embedding_length": 256, "llama.block_count": 1, "llama.attention.head_count": 4,
            "llama.attention.head_count_kv": 2, "llama.feed_forward_length": 512}
    cases = [(dict(base, **{"general.architecture": "qwen4exp"}), "architecture"),
             ({k: v for k, v in base.items() if k != "llama.feed_forward_length"}, "missing or inconsistent"),
             (dict(base, **{"llama.attention.head_count": 3}), "missing or inconsistent"),
             (dict(base, **{"llama.rope.dimension_count": 32}), "partial rotary"),
             (dict(base, **{"llama.rope.scaling.type": "linear"}), "linear")]
    for i, (meta, msg) in enumerate(cases):
        path = str(tmp_path / f"d{i}.gguf")
        synth.write_gguf(path, meta, [("token_embd.weight", [256, 64], ol.TYPE_Q4_0, emb)])
        g = wd.Gguf(path)
        h = C.c_void_p()
        rc = wd.lib().wd_dense_decoder_load_gguf(g.h, 64, 0, C.byref(h))
        assert rc != 0 and msg in wd.lib().wd_last_error().decode(), (msg, wd.lib().wd_last_error())
        g.close()
