"""Generates tests/golden/oracle_pins.npz from the REFERENCE's own host code.

Run in a container that has the reference tree (so that oracle/build_ref.sh can build
oracle/_ref/libwd_ref.so):

    python tests/golden/make_golden.py

Every input is derived from a fixed seed by `cases()` below, which the tests import, so
the file only stores the reference's outputs. The outputs come from libwd_ref.so, i.e.
from src/qwen38_cpu_moe.cuh and the router block of src/qwen38_moe.cuh of the reference,
never from this repository's oracle.
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle_lib as ol  # noqa: E402
from warpdecode_b200 import synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_pins.npz")


def digest(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


def unary_inputs():
    rng = np.random.Generator(np.random.PCG64(11))
    xs = [rng.uniform(-100, 100, 4000), rng.uniform(-1, 1, 2000), rng.standard_normal(2000) * 10,
          np.array([0.0, -0.0, 1e-38, -1e-38, 87.0, 88.5, 89.0, -87.0, -88.0, -103.0, -104.0, -126.0,
                    -127.0, -150.0, -192.5, 126.5, 127.5, 191.0, 193.0, np.inf, -np.inf])]
    return np.concatenate(xs).astype(np.float32)


def f32_inputs_for_f16():
    rng = np.random.Generator(np.random.PCG64(12))
    bits = rng.integers(0, 2 ** 32, 20000, dtype=np.uint64).astype(np.uint32)
    edge = np.array([0x00000000, 0x80000000, 0x33000000, 0x33000001, 0x33800000, 0x387fc000, 0x387fe000,
                     0x38800000, 0x477fe000, 0x477ff000, 0x47800000, 0x7f800000, 0xff800000, 0x3f801000,
                     0x3f803000, 0x3f802000, 0x38000000, 0x37ffffff], np.uint32)
    v = np.concatenate([bits, edge]).view(np.float32)
    return v[~np.isnan(v)]


def quantizer_inputs():
    rng = np.random.Generator(np.random.PCG64(13))
    x = rng.uniform(-1.5, 1.5, 2048).astype(np.float32)
    x[256:512] = 0.0                       # zero superblock
    x[512:544] = 0.0
    x[519] = 3.0                           # single-peak block
    x[768:1024] = rng.standard_normal(256).astype(np.float32) * 1e-3
    x[1024] = -7.5                         # negative peak picks the scale
    x[1300:1332] = np.float32(65504.0)     # saturating scale
    x[1400:1432] = np.float32(1e-8)        # subnormal fp16 scale
    half = np.float32(0.5) * np.float32(1.5) / np.float32(127)
    x[1500:1532] = np.arange(32, dtype=np.float32) * half  # ties for rint
    return x


ROW_CASES = [(ol.TYPE_IQ3_S, c) for c in (256, 512, 768, 2048, 2560)] + \
            [(ol.TYPE_IQ2_S, c) for c in (256, 512, 2048, 2560)] + \
            [(ol.TYPE_Q8_0, c) for c in (32, 224, 512, 640, 2048, 2560)] + \
            [(ol.TYPE_IQ4_NL, c) for c in (32, 96, 224, 640)]
ROWS_PER_CASE = 24


def row_case(t, cols, i):
    rng = np.random.Generator(np.random.PCG64(1000 + 17 * t + cols + 7919 * i))
    w = ol.random_blocks(rng, t, cols // ol.BLOCK_ELEMS[t])
    x = rng.uniform(-1.5, 1.5, cols).astype(np.float32) if i % 3 else rng.standard_normal(cols).astype(np.float32)
    return w, x


ROUTER_K = [10, 1, 4, 16, 7]
ROUTER_SCALES = [1.0, 2.5, 0.5, 0.0]


def router_cases():
    out = []
    for ki, kind in enumerate(ol.ADVERSARIAL_KINDS):
        for rep in range(6):
            rng = np.random.Generator(np.random.PCG64(5000 + 100 * ki + rep))
            n = 512 if rep < 4 else (64 if rep == 4 else 1024)
            out.append((kind, rep, ol.adversarial_logits(rng, n, kind), ROUTER_K[rep % 5],
                        ROUTER_SCALES[rep % 4]))
    return out


def requant_inputs():
    """Rows of Q6_K (210 B / 256 values) and Q8_0 blocks with random bytes and f16 scales in [1e-4, 2e-2], for the host
    requantiser of the reference's dense loader (ggml_requantize_row_to_q8_0, src/ggml_dequant.hpp:362-392): 8 rows of
    512 columns each; one Q6_K block and one Q8_0 block are all zeros (d = 0)."""
    rng = np.random.Generator(np.random.PCG64(606))
    qk = rng.integers(0, 256, size=(16, 210), dtype=np.uint8)
    qk[:, 208:210] = rng.uniform(1e-4, 2e-2, 16).astype(np.float16).view(np.uint8).reshape(16, 2)
    qk[3] = 0
    q8 = rng.integers(0, 256, size=(128, 34), dtype=np.uint8)
    q8[:, 0:2] = rng.uniform(1e-4, 2e-2, 128).astype(np.float16).view(np.uint8).reshape(128, 2)
    q8[17] = 0
    return qk.reshape(-1), q8.reshape(-1)


def block_cases():
    """(model dict, inputs [n, H]) for small MoE blocks. The last three have the geometry rules of the reference's own
    model (src/qwen38_moe.cuh:2181-2211, :2252-2258): hidden a multiple of 256 that is not a power of two, expert_ffn
    a multiple of 64, IQ4_NL down tensors with a Q8_0 activation, and (two of them) an F32 router."""
    out = []
    for i, (H, F, E, K, SF, et, dt, bias, rf32) in enumerate([
            (256, 256, 16, 4, 256, ol.TYPE_IQ3_S, ol.TYPE_IQ3_S, 0.0, False),
            (512, 256, 32, 10, 128, ol.TYPE_IQ3_S, ol.TYPE_IQ3_S, 1.0, False),
            (512, 512, 16, 6, 256, ol.TYPE_IQ2_S, ol.TYPE_IQ2_S, 0.0, False),
            (256, 512, 24, 8, 64, ol.TYPE_IQ2_S, ol.TYPE_IQ3_S, 0.0, False),
            (768, 192, 16, 4, 128, ol.TYPE_IQ3_S, ol.TYPE_IQ4_NL, 0.5, False),
            (2560, 640, 8, 4, 640, ol.TYPE_IQ2_S, ol.TYPE_IQ4_NL, 0.0, True),
            (1280, 256, 24, 10, 0, ol.TYPE_IQ3_S, ol.TYPE_IQ2_S, 1.0, True)]):
        m = synth.make_moe_block(100 + i, H, F, E, K, SF, et, dt, sigma=0.02, bias_sigma=bias,
                                 w_scale=1.0 if i not in (2, 5) else 1.25, router_f32=rf32)
        rng = np.random.Generator(np.random.PCG64(200 + i))
        out.append((m, rng.standard_normal((4, H)).astype(np.float32)))
    return out


def main():
    ol.build_oracle()
    if not ol.Reference.available():
        raise SystemExit("oracle/_ref/libwd_ref.so missing: the reference tree is needed to make goldens")
    ref = ol.Reference()
    g = {}
    g3, g2 = ref.grids()
    g["grid3"], g["grid2"] = g3, g2
    g["f16_to_f32_sha"] = digest(ref.f16_to_f32(np.arange(65536)).view(np.uint32))
    g["f32_to_f16"] = ref.f32_to_f16(f32_inputs_for_f16())
    ux = unary_inputs()
    for name in ("exp_ggml", "silu_ggml", "sigmoid_ggml"):
        g[name] = ol.fbits(ref.unary(name, ux))
    qx = quantizer_inputs()
    g["q8_0"] = ref.quantize_q8_0(qx)
    g["q8_K"] = ref.quantize_q8_K(qx)
    rows = []
    for t, cols in ROW_CASES:
        for i in range(ROWS_PER_CASE):
            w, x = row_case(t, cols, i)
            y = ref.quantize_q8_K(x) if t in (ol.TYPE_IQ3_S, ol.TYPE_IQ2_S) else ref.quantize_q8_0(x)
            rows.append(ref.row(t, w, y, cols, 0))
            assert rows[-1].view(np.uint32) == ref.row(t, w, y, cols, 1).view(np.uint32)
    g["rows"] = np.array(rows, np.float32).view(np.uint32)
    rng = np.random.Generator(np.random.PCG64(14))
    dots = []
    for n in (32, 2048, 2560, 100, 31, 2049):
        a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        dots.append(ref.dot_f32(a, b))
    g["dot_f32"] = np.array(dots, np.float32).view(np.uint32)
    ids, wts, psha = [], [], []
    for kind, rep, logits, k, s in router_cases():
        p, i_, w_ = ref.router(logits, k, s)
        ids.append(np.pad(i_, (0, 16 - k), constant_values=-1))
        wts.append(np.pad(ol.fbits(w_), (0, 16 - k)))
        psha.append(digest(ol.fbits(p)))
    g["router_ids"], g["router_w"], g["router_probs_sha"] = np.array(ids, np.int32), np.array(wts, np.uint32), np.array(psha)
    qk, q8 = requant_inputs()
    g["requant_q6_k"] = ref.requantize_rows_to_q8_0(ol.TYPE_Q6_K, qk, 8, 512)
    g["requant_q8_0"] = ref.requantize_rows_to_q8_0(ol.TYPE_Q8_0, q8, 8, 512)
    for bi, (m, xs) in enumerate(block_cases()):
        outs, sel, sw = [], [], []
        for x in xs:
            r = ref.moe_block(m, x, threads=4)
            r1 = ref.moe_block(m, x, threads=1)
            assert np.array_equal(r["out"].view(np.uint32), r1["out"].view(np.uint32))
            outs.append(r["out"].view(np.uint32)); sel.append(r["ids"]); sw.append(r["weights"].view(np.uint32))
        g[f"block{bi}_out"], g[f"block{bi}_ids"], g[f"block{bi}_w"] = np.array(outs), np.array(sel), np.array(sw)
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
