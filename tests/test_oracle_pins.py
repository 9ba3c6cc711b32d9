"""Pins oracle/wd_oracle.c: bit for bit against the golden vectors the reference's own host
code produced (tests/golden/oracle_pins.npz, made by tests/golden/make_golden.py) and, when
oracle/_ref/libwd_ref.so is present, against that code live on further seeded inputs."""
import hashlib
import os

import numpy as np
import pytest

import make_golden as mg
import oracle_lib as ol

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_pins.npz"))


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def bits(a):
    return ol.fbits(a)


def test_codebooks_match_reference_tables(oracle):
    g3, g2 = oracle.grids()
    assert np.array_equal(g3, GOLD["grid3"]) and np.array_equal(g2, GOLD["grid2"])


def test_codebook_crc_constants():
    import zlib
    txt = open(os.path.join(ol.ROOT, "warpdecode_b200", "csrc", "wd_grids.h")).read()
    assert f"0x{zlib.crc32(GOLD['grid3'].astype('<u4').tobytes()):08x}u" in txt
    assert f"0x{zlib.crc32(GOLD['grid2'].astype('<u8').tobytes()):08x}u" in txt


def test_half_conversions(oracle):
    assert np.array_equal(sha(oracle.f16_to_f32(np.arange(65536)).view(np.uint32)), GOLD["f16_to_f32_sha"])
    assert np.array_equal(oracle.f32_to_f16(mg.f32_inputs_for_f16()), GOLD["f32_to_f16"])


@pytest.mark.parametrize("name", ["exp_ggml", "silu_ggml", "sigmoid_ggml"])
def test_transcendentals(oracle, name):
    assert np.array_equal(bits(oracle.unary(name, mg.unary_inputs())), GOLD[name])


def test_activation_quantisers_incl_edge_blocks(oracle):
    x = mg.quantizer_inputs()
    assert np.array_equal(oracle.quantize_q8_0(x), GOLD["q8_0"])
    assert np.array_equal(oracle.quantize_q8_K(x), GOLD["q8_K"])


def test_row_dots_all_types(oracle):
    got = []
    for t, cols in mg.ROW_CASES:
        for i in range(mg.ROWS_PER_CASE):
            w, x = mg.row_case(t, cols, i)
            y = oracle.quantize_q8_K(x) if t in (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S) else oracle.quantize_q8_0(x)
            got.append(oracle.row(t, w, y, cols))
    assert np.array_equal(bits(np.array(got)), GOLD["rows"])


def _exact_partials(t, w, yq, cols):
    """Independent int64 reconstruction of the per-(superblock, chunk-lane) integer sums."""
    g3, g2 = GOLD["grid3"], GOLD["grid2"]
    nb = cols // 256
    bb = ol.BLOCK_BYTES[t]
    out = np.zeros(nb * 8, np.int64)
    for sb in range(nb):
        blk = w[sb * bb:(sb + 1) * bb]
        a = yq[sb * ol.Q8K_BYTES + 4: sb * ol.Q8K_BYTES + 260].view(np.int8).astype(np.int64)
        for ib in range(8):
            for c in range(8):
                if t == ol.TYPE_IQ3_S:
                    qs, qh, sg, sc = blk[2:66], blk[66:74], blk[74:106], blk[106:110]
                    idx = int(qs[ib * 8 + c]) | (((int(qh[ib]) >> c) & 1) << 8)
                    mags = [(int(g3[idx]) >> (8 * j)) & 255 for j in range(4)]
                    nib = (int(sc[ib >> 1]) >> 4) if (ib & 1) else (int(sc[ib >> 1]) & 15)
                else:
                    qs, sg, qh, sc = blk[2:34], blk[34:66], blk[66:74], blk[74:82]
                    idx = int(qs[ib * 4 + (c >> 1)]) | (((int(qh[ib]) >> (2 * (c >> 1))) & 3) << 8)
                    mags = [(int(g2[idx]) >> (8 * (4 * (c & 1) + j))) & 255 for j in range(4)]
                    nib = (int(sc[ib]) & 15) if c < 4 else (int(sc[ib]) >> 4)
                sbits = int(sg[ib * 4 + (c >> 1)]) >> (4 * (c & 1))
                dot = sum(int(a[ib * 32 + c * 4 + j]) * (-mags[j] if (sbits >> j) & 1 else mags[j]) for j in range(4))
                out[sb * 8 + c] += dot * (1 + 2 * nib)
    return out


@pytest.mark.parametrize("t", [ol.TYPE_IQ3_S, ol.TYPE_IQ2_S])
def test_integer_partials_are_exact(oracle, t):
    for i in range(6):
        w, x = mg.row_case(t, 512, i)
        y = oracle.quantize_q8_K(x)
        _, part = oracle.row(t, w, y, 512, partials=True)
        assert np.array_equal(part.astype(np.int64), _exact_partials(t, w, y, 512))


def test_dot_f32(oracle):
    rng = np.random.Generator(np.random.PCG64(14))
    got = []
    for n in (32, 2048, 2560, 100, 31, 2049):
        a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        got.append(oracle.dot_f32(a, b))
    assert np.array_equal(bits(np.array(got)), GOLD["dot_f32"])


def test_router_adversarial_rows(oracle):
    for ci, (kind, rep, logits, k, s) in enumerate(mg.router_cases()):
        p, ids, w = oracle.router(logits, k, s)
        assert np.array_equal(ids, GOLD["router_ids"][ci][:k]), (kind, rep)
        assert np.array_equal(bits(w), GOLD["router_w"][ci][:k]), (kind, rep)
        assert np.array_equal(sha(bits(p)), GOLD["router_probs_sha"][ci]), (kind, rep)


def test_moe_block_composition(oracle):
    for bi, (m, xs) in enumerate(mg.block_cases()):
        for xi, x in enumerate(xs):
            r = oracle.moe_block(m, x)
            assert np.array_equal(r["ids"], GOLD[f"block{bi}_ids"][xi])
            assert np.array_equal(bits(r["weights"]), GOLD[f"block{bi}_w"][xi])
            assert np.array_equal(bits(r["out"]), GOLD[f"block{bi}_out"][xi])


def test_combine_is_mul_then_add_not_fma(oracle):
    # negative control from the reference's host test (tests/qwen38_cpu_moe_host_test.cpp:315-324)
    a, b, c = np.float32(1.1109310388565063), np.float32(1.1190425157546997), np.float32(-1.3467210531234741)
    two_step = np.float32(np.float32(a * b) + c)
    fused = np.float32(np.float64(a) * np.float64(b) + np.float64(c))
    assert two_step != fused


def test_expert_parallel_partials_cover_the_block(oracle):
    m, xs = mg.block_cases()[1]
    full = oracle.moe_block(m, xs[0])
    E = m["n_experts"]
    lo = oracle.moe_block(m, xs[0], 0, E // 2)
    hi = oracle.moe_block(m, xs[0], E // 2, E // 2)
    assert np.array_equal(lo["ids"], full["ids"]) and np.array_equal(hi["ids"], full["ids"])
    # every selected expert's down output appears in exactly one partial
    assert np.array_equal(bits(lo["expert_out"] + hi["expert_out"]), bits(full["expert_out"]))


# ---- live comparison with the reference build (skipped where it is absent) -----------------
def test_live_rows_against_reference(oracle, reference):
    rng = np.random.Generator(np.random.PCG64(99))
    for t in (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S, ol.TYPE_Q8_0, ol.TYPE_IQ4_NL):
        for cols in (256, 1024, 2048):
            for _ in range(8):
                w = ol.random_blocks(rng, t, cols // ol.BLOCK_ELEMS[t])
                x = (rng.standard_normal(cols) * rng.uniform(0.01, 30)).astype(np.float32)
                if t in (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S):
                    y = oracle.quantize_q8_K(x)
                    assert np.array_equal(y, reference.quantize_q8_K(x))
                else:
                    y = oracle.quantize_q8_0(x)
                    assert np.array_equal(y, reference.quantize_q8_0(x))
                assert bits(oracle.row(t, w, y, cols)) == bits(reference.row(t, w, y, cols))


def test_live_router_against_reference(oracle, reference):
    for ki, kind in enumerate(ol.ADVERSARIAL_KINDS):
        for rep in range(10):
            rng = np.random.Generator(np.random.PCG64(77000 + 50 * ki + rep))
            logits = ol.adversarial_logits(rng, 512, kind)
            k, s = 1 + rep % 16, [1.0, 2.5, 0.5][rep % 3]
            po, io, wo = oracle.router(logits, k, s)
            pr, ir, wr = reference.router(logits, k, s)
            assert np.array_equal(io, ir) and np.array_equal(bits(wo), bits(wr)) and np.array_equal(bits(po), bits(pr))


def test_live_block_against_reference_any_thread_count(oracle, reference):
    m, xs = mg.block_cases()[0]
    o = oracle.moe_block(m, xs[1])
    for th in (1, 3, 8):
        r = reference.moe_block(m, xs[1], threads=th)
        assert np.array_equal(r["ids"], o["ids"]) and np.array_equal(bits(r["out"]), bits(o["out"]))


def test_q4_0_row_dot_against_gguf_py_decoder_and_exact_integers(oracle):
    """The reference has no host twin and no golden vector for its plain Q4_0 matvec (src/warodecode.cu:1535-1562),
    so the oracle's Q4_0 row is pinned against an independent decoder instead: gguf-py dequantises the same block
    bytes, the integer side (sum of (q - 8) * q_x per chunk of four values) is rebuilt in int64, and the float side
    replays ggml's order (one fmaf per block and chunk-lane, then the 8-lane tree) with every step rounded once."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.Generator(np.random.PCG64(404))
    cols, rows = 2048, 48
    nb = cols // 32
    w = rng.integers(0, 256, (rows * nb, 18), dtype=np.uint8)
    w[:, 0:2] = (rng.random(rows * nb) * 0.01 + 0.001).astype(np.float16).view(np.uint8).reshape(-1, 2)
    x = rng.standard_normal(cols).astype(np.float32)
    xq = oracle.quantize_q8_0(x).reshape(nb, 34)
    wf = quants.dequantize(w.reshape(rows, nb * 18), gguf.GGMLQuantizationType.Q4_0).reshape(rows, nb, 32)
    xf = quants.dequantize(xq.reshape(1, nb * 34), gguf.GGMLQuantizationType.Q8_0).reshape(nb, 32)
    d_w = w[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(rows, nb)
    d_x = xq[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(nb)
    qw = np.rint(wf.astype(np.float64) / d_w[:, :, None]).astype(np.int64)          # (q - 8), exact
    qx = xq[:, 2:].view(np.int8).astype(np.int64)
    assert np.array_equal(np.rint(xf.astype(np.float64) / np.where(d_x == 0, 1, d_x)[:, None]).astype(np.int64) * (d_x != 0)[:, None],
                          qx * (d_x != 0)[:, None])
    assert qw.min() >= -8 and qw.max() <= 7
    part = (qw.reshape(rows, nb, 8, 4) * qx.reshape(1, nb, 8, 4)).sum(-1)           # [row][block][chunk-lane], int64
    for r in range(rows):
        lane = np.zeros(8, np.float32)
        for b in range(nb):
            d = np.float32(d_w[r, b] * d_x[b])
            lane = (d.astype(np.float64) * part[r, b].astype(np.float64) + lane.astype(np.float64)).astype(np.float32)   # fmaf
        s = [np.float32(lane[i] + lane[i + 4]) for i in range(4)]
        want = np.float32(np.float32(s[0] + s[2]) + np.float32(s[1] + s[3]))
        got = oracle.row(ol.TYPE_Q4_0, w[r * nb:(r + 1) * nb].reshape(-1), xq.reshape(-1), cols)
        assert ol.fbits(np.array([got]))[0] == ol.fbits(np.array([want]))[0], r


def test_q4_0_row_dot_in_lane_order_against_gguf_py_decoder(oracle):
    """The dense decoder's row dot (a warp splits a row's blocks over its 32 lanes, one fmaf per block, then a
    butterfly) pinned the same way: gguf-py's decoder gives the block values, the integer dot of every block is
    rebuilt in int64, the float side replays the stated order with every step rounded once."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.Generator(np.random.PCG64(405))
    for cols in (256, 2048, 8192):
        rows, nb = 12, cols // 32
        w = rng.integers(0, 256, (rows * nb, 18), dtype=np.uint8)
        w[:, 0:2] = (rng.random(rows * nb) * 0.01 + 0.001).astype(np.float16).view(np.uint8).reshape(-1, 2)
        x = rng.standard_normal(cols).astype(np.float32)
        xq = oracle.quantize_q8_0(x).reshape(nb, 34)
        wf = quants.dequantize(w.reshape(rows, nb * 18), gguf.GGMLQuantizationType.Q4_0).reshape(rows, nb, 32)
        d_w = w[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(rows, nb)
        d_x = xq[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(nb)
        qw = np.rint(wf.astype(np.float64) / d_w[:, :, None]).astype(np.int64)
        qx = xq[:, 2:].view(np.int8).astype(np.int64)
        dots = (qw * qx[None]).sum(-1)                                                  # [row][block], int64
        f = oracle.lib.wdo_row_q4_0_q8_0_lanes
        for r in range(rows):
            lane = np.zeros(32, np.float32)
            for b in range(nb):
                d = np.float32(d_w[r, b] * d_x[b])
                lane[b & 31] = np.float32(np.float64(d) * np.float64(dots[r, b]) + np.float64(lane[b & 31]))    # fmaf
            for sft in (16, 8, 4, 2, 1):
                lane = np.array([np.float32(lane[l] + lane[l ^ sft]) for l in range(32)], np.float32)
            wr = np.ascontiguousarray(w[r * nb:(r + 1) * nb].reshape(-1))
            xr = np.ascontiguousarray(xq.reshape(-1))
            got = np.float32(f(wr.ctypes.data, xr.ctypes.data, cols))
            assert ol.fbits(np.array([got]))[0] == ol.fbits(np.array([lane[0]]))[0], (cols, r)


def test_dense_loader_requantiser_and_q6_k_values(oracle):
    """Non-Q4_0 tensors of a dense model file become Q8_0 on the host, by the reference's rule (src/ggml_dequant.hpp:
    362-392): golden bytes from the reference's function; Q6_K values also against gguf-py's decoder."""
    qk, q8 = mg.requant_inputs()
    assert np.array_equal(oracle.requantize_rows_to_q8_0(ol.TYPE_Q6_K, qk, 8, 512), GOLD["requant_q6_k"])
    assert np.array_equal(oracle.requantize_rows_to_q8_0(ol.TYPE_Q8_0, q8, 8, 512), GOLD["requant_q8_0"])
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    theirs = quants.dequantize(qk.reshape(8, -1), gguf.GGMLQuantizationType.Q6_K).astype(np.float32)
    mine = np.array([[oracle.lib.wdo_q6_k_value(qk.ctypes.data + (r * 2 + i // 256) * 210, i % 256) for i in range(512)]
                     for r in range(8)], np.float32)
    assert np.array_equal(bits(theirs), bits(mine))
