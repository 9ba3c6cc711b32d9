"""Small, self-ending measurement cases beside bench.py: the workloads that the profile summaries under profiles/
were captured from (ncu wants a short program with few launches), and the kernel's own phase stamps.

    python bench_cases.py profile [--layers 2] [--iters 4] [--stamps] [--stack] [--compiled]
        a few forward calls of the MoE layer kernel at the 48-layer model's block shape, direct launches, about
        0.7 GB per layer on the device; --stamps prints the kernel's per-phase timestamps (mean over CTAs)
        instead (generic kernel), which needs no profiler; --compiled runs the kernel compiled for the geometry
    python bench_cases.py batch [--layers 2] [--tokens 4] [--iters 4] [--stamps]
        token batches (speculative verify) through the per-layer forward on the batch kernel; --stamps prints the
        kernel's own step times (median over CTAs)
    python bench_cases.py plain [--layers 2] [--tokens 1] [--iters 20]
        the plain-layout path at the block shape of the reference's own model (hidden 2560, expert_ffn 640, 512
        experts, top 10, IQ2_S gate/up, IQ4_NL down, F32 router, shared expert 640; random block bytes): per-layer
        forward calls, time per call from CUDA events on the launching stream
    python bench_cases.py decoder
        the IQ3_S tile decoder alone, tiles resident in shared memory: cycles per round of tiles for 16, 8, 4 and 1
        active warps per SM (the issue bound of the expert GEMVs)
    python bench_cases.py dense-decode [--layers 16] [--vocab 128256] [--gen 64] [--runs 3]
        the plain Q4_0 decoder on the dense benchmark model (Llama-style, hidden 2048, 32 query / 8 KV heads of 64,
        SwiGLU 8192, RoPE theta 5e5, weights N(0, 0.02) generated on the device): greedy decode of 64 tokens after an
        8-token prompt, one CUDA-graph replay per token; fastest of the runs, with the token hash
    python bench_cases.py dense [--rows 128256] [--cols 2048] [--mats 2] [--iters 20]
        streams Q4_0 matrices of the plain decoder's output-head size through the dense matvec kernel
    python bench_cases.py head [--rows 151936] [--cols 2048] [--iters 20]
        the Q8_0 output head with fused arg-max
    python bench_cases.py load [--layers 2] [--dir /tmp]
        model load from a GGUF file: open + engine create + load for a few layers of the model's shape
"""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import warpdecode_b200 as wd          # noqa: E402


def measured_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


# ---- profile: the MoE layer kernel ---------------------------------------------------------------------------------


# stamp indices in the order the kernel passes them, and the name of the span that ends at each
ORDER = [0, 1, 2, 3, 4, 13, 5, 6, 11, 7, 9, 8, 10]
PHASES = ["issue_p1", "x_wait_quant", "q8_rows", "gather_logits", "select.router", "select.rest",
          "issue_tiles", "first_tile_wait", "gate_up", "gather_act_quant", "down", "combine"]


def phase_row(st, with_period):
    ok = st[:, 11] >= st[:, 6]          # CTAs without a gate/up tile in this layer leave stamp 11 unset
    d = [(st[ok, ORDER[i + 1]] - st[ok, ORDER[i]]).mean() for i in range(len(ORDER) - 1)]
    d.append((st[:, 10] - st[:, 0]).mean())                         # a CTA's time inside the layer
    d.append((st[:, 14] - st[:, 0]).mean() if with_period else 0)   # start of this layer to start of the next
    return d


def profile_case(a):
    os.environ["WD_BATCH_SINGLE"] = "0"          # this case is about the layer kernel, also for one-layer calls
    if a.compiled:
        os.environ["WD_COMPILED_KERNEL"] = "1"
    eng = wd.Engine(2048, 512, 512, 10, 512, a.layers)
    print("kernel:", eng.kernel_name())
    eng.synth_model(3, 0.02, 0.0)
    rng = np.random.Generator(np.random.PCG64(1))
    rows = []
    if a.stack:
        # all layers in one launch; the profiled layer sits in the middle, where the code is cache-warm
        eng.set_profiling(1 + a.layers // 2 if a.stamps else 0)
        res = rng.standard_normal(2048).astype(np.float32)
        for it in range(a.iters + 1):
            t0 = time.perf_counter()
            res = eng.stack_step_host(res)
            wall = time.perf_counter() - t0
            if a.stamps:
                rows.append(phase_row(eng.stamps().astype(np.int64), a.layers // 2 + 1 < a.layers))
        print("last stack step, host wall clock: %.1f us per layer" % (wall * 1e6 / a.layers))
        skip = 1
    else:
        eng.set_profiling(a.stamps)
        for it in range(a.iters):
            for layer in range(a.layers):
                eng.forward_host(layer, rng.standard_normal(2048).astype(np.float32))
                if a.stamps:
                    rows.append(phase_row(eng.stamps().astype(np.int64), False))
        skip = a.layers
    assert eng.device_status() == 0
    if a.stamps:
        m = np.array(rows[skip:]).mean(0)          # skip the first pass (cold)
        names = PHASES + ["cta_in_layer", "layer_period"]
        print("mean ns per phase:", {n: int(v) for n, v in zip(names, m)})
    print("done")


# ---- dense: Q4_0 matvec and the Q8_0 head ---------------------------------------------------------------------------


# ---- batch: the batch kernel ---------------------------------------------------------------------------------------
BATCH_STEPS = [(1, "copies_issued_tables"), (2, "activations_quantised"), (3, "row_tasks"), (4, "block_sync"),
               (5, "picks_gathered"), (6, "first_tiles_issued"), (9, "tile_tasks"), (10, "shared_down"), (11, "combine"),
               (12, "end")]


def batch_case(a):
    import torch
    H = 2048
    eng = wd.Engine(H, 512, 512, 10, 512, a.layers, max_tokens=4)
    print("kernel:", eng.batch_kernel_name())
    eng.synth_model(3, 0.02, 1.0)
    x = torch.randn(4, H, generator=torch.Generator().manual_seed(2), dtype=torch.float32).cuda()
    out = torch.zeros_like(x)
    ts = torch.cuda.Stream()
    sp = ts.cuda_stream
    if a.stamps:
        eng.set_profiling(True)
    with torch.cuda.stream(ts):
        for _ in range(2):
            for l in range(a.layers):
                eng.forward_device(l, x.data_ptr(), out.data_ptr(), sp, a.tokens)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ts):
        e0.record(ts)
        for _ in range(a.iters):
            for l in range(a.layers):
                eng.forward_device(l, x.data_ptr(), out.data_ptr(), sp, a.tokens)
        e1.record(ts)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.iters * a.layers)
    print("%d tokens per call: %.2f us per call, %.2f us per token and layer, status %d" % (a.tokens, us, us / a.tokens, eng.device_status()))
    if a.stamps:
        st = eng.stamps().astype(np.int64)
        mhz = 1965.0          # the stamps are SM clock cycles; the bench box runs the SMs at their maximum under this load
        prev = 0
        for idx, name in BATCH_STEPS:
            d = np.median(st[:, idx] - st[:, 0]) / mhz
            print("  %-24s ends at %6.2f us (+%.2f)" % (name, d, d - prev))
            prev = d
    eng.close()


def plain_case(a):
    import torch
    from warpdecode_b200 import synth
    H, F, E, K, SF = 2560, 640, 512, 10, 640
    eng = wd.Engine(H, F, E, K, SF, a.layers, expert_type=synth.TYPE_IQ2_S, down_type=synth.TYPE_IQ4_NL, w_scale=1.25,
                    router_f32=True, max_tokens=4)
    print("kernel:", eng.kernel_name())
    rng = np.random.Generator(np.random.PCG64(4))
    small = synth.make_moe_block(5, H, F, 8, 8, SF, synth.TYPE_IQ2_S, synth.TYPE_IQ4_NL, sigma=0.02, router_f32=True)
    for l in range(a.layers):
        m = dict(small)
        m.update(n_experts=E, top_k=K, w_scale=1.25)
        m["router_f32"] = (rng.standard_normal(E * H) * 0.02).astype(np.float32)
        m["router_bias"] = (rng.standard_normal(E) * 0.5).astype(np.float32)
        m["gate"] = synth.random_blocks(rng, synth.TYPE_IQ2_S, E * F * H // 256)
        m["up"] = synth.random_blocks(rng, synth.TYPE_IQ2_S, E * F * H // 256)
        m["down"] = synth.random_blocks(rng, synth.TYPE_IQ4_NL, E * H * F // 32)
        eng.load_block(l, m)
    x = torch.randn(4, H, generator=torch.Generator().manual_seed(2), dtype=torch.float32).cuda()
    out = torch.zeros_like(x)
    ts = torch.cuda.Stream()
    sp = ts.cuda_stream
    with torch.cuda.stream(ts):
        for _ in range(3):
            for l in range(a.layers):
                eng.forward_device(l, x.data_ptr(), out.data_ptr(), sp, a.tokens)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(ts):
        e0.record(ts)
        for _ in range(a.iters):
            for l in range(a.layers):
                eng.forward_device(l, x.data_ptr(), out.data_ptr(), sp, a.tokens)
        e1.record(ts)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.iters * a.layers)
    # bytes one token reads in a layer: ten experts' gate, up and down rows, the F32 router, the shared expert
    layer_bytes = K * (2 * F * (H // 256) * 82 + H * (F // 32) * 18) + E * H * 4 + 3 * SF * (H // 32) * 34
    peak = measured_peak()
    if os.environ.get("WD_PLAIN_STAMPS") == "1":
        import ctypes as C
        st = np.zeros(2 * 512 * 8, np.uint64)
        wd._check(wd.lib().wd_read_tap(eng.h, 9, -1, st.ctypes.data, st.nbytes))
        st = st.reshape(2, 512, 8).astype(np.int64)
        for k, (name, n, steps) in enumerate((("gate_up", K * F // 16, ["tables", "wait for select", "issue + activation", "wait for chunks", "rows"]),
                                              ("down", H // 16, ["issue", "wait for gate_up", "load act", "quantise", "wait for chunks", "rows", "shared + combine"]))):
            v = st[k, :min(n, 512)]
            t0 = v[:, 0].min()
            print(name, "first CTA starts 0, last CTA starts %.2f us, last CTA ends %.2f us" % ((v[:, 0].max() - t0) / 1e3, (v[:, len(steps)].max() - t0) / 1e3))
            for i, sname in enumerate(steps):
                print("   %-22s median %.2f us" % (sname, np.median(v[:, i + 1] - v[:, i]) / 1e3))
    print("%d tokens per call: %.2f us per call, %.2f us per token and layer; %.1f MB per token and layer -> %.0f GB/s = %.3f of "
          "the measured HBM peak (%.0f GB/s); status %d" % (a.tokens, us, us / a.tokens, layer_bytes / 1e6,
                                                          layer_bytes * a.tokens / us / 1e3, layer_bytes * a.tokens / us / 1e3 / peak, peak,
                                                          eng.device_status()))
    eng.close()


def decoder_case(a):
    mhz = 1965.0
    for unroll in (1, 8):
        for nsb in (8, 2):
            for warps in (16, 8, 4, 1):
                c = wd.measure_tile_decoder(nsb, warps, unroll)
                print("unroll %d, %d superblocks per row, %2d warps: %6.0f cycles per round, %5.1f cycles per tile and SM, "
                      "%.2f us per 16 tiles at %.0f MHz" % (unroll, nsb, warps, c, c / warps, c / warps * 16 / mhz, mhz))


def dense_decode_case(a):
    H, nh, nkv, hd, F = 2048, 32, 8, 64, 8192
    dec = wd.DenseDecoder(H, nh, nkv, hd, F, a.vocab, a.layers, 128, 1e-5, 500000.0)
    t0 = time.perf_counter()
    dec.synth(2, 0.02)
    gen_s = time.perf_counter() - t0
    prompt = np.random.Generator(np.random.PCG64(2)).integers(0, a.vocab, 8)
    q4 = lambda r, c: r * (c // 32) * 18
    layer_bytes = q4((nh + 2 * nkv) * hd, H) + q4(H, nh * hd) + q4(2 * F, H) + q4(H, F)
    token_bytes = a.layers * layer_bytes + q4(a.vocab, H)
    best, toks = None, None
    for _ in range(a.runs):
        toks, ms = dec.decode(prompt, a.gen)
        best = ms if best is None else min(best, ms)
    steps = len(prompt) + a.gen - 1
    h = 0xcbf29ce484222325
    for t in toks.tolist():
        for k in range(4):
            h = ((h ^ ((t >> (8 * k)) & 0xff)) * 0x100000001b3) & 0xffffffffffffffff
    us = best * 1e3 / steps
    peak = measured_peak()
    print("model generated in %.2f s; %d layers, vocab %d; %d bytes of weights per token" % (gen_s, a.layers, a.vocab, token_bytes))
    print("%d steps in %.3f ms: %.1f us per token, %.1f tok/s, %.0f GB/s = %.3f of the measured HBM peak (%.0f GB/s)"
          % (steps, best, us, 1e6 / us, token_bytes / us / 1e3, token_bytes / us / 1e3 / peak, peak))
    print("token_hash %016x, %d distinct generated tokens" % (h, len(set(toks[len(prompt):].tolist()))))
    dec.close()


def head_case(a):
    """Q8_0 matrix [rows][cols] (default: the 48-layer decoder's head, 151936 x 2048 = 331 MB) + arg-max."""
    import torch
    nb = a.cols // 32
    g = torch.Generator(device="cuda").manual_seed(7)
    blocks = torch.randint(0, 256, (a.rows * nb, 34), dtype=torch.uint8, device="cuda", generator=g)
    scale = (torch.rand(a.rows * nb, device="cuda", generator=g) * 0.01 + 0.001).to(torch.float16)
    blocks[:, 0:2] = scale.view(torch.uint8).reshape(-1, 2)
    torch.cuda.synchronize()
    head = wd.HeadQ8_0(a.rows, a.cols, ggml_dev_ptr=blocks.data_ptr())
    torch.cuda.synchronize()
    del blocks
    x = torch.randn(a.cols, device="cuda", generator=g)
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        head.argmax(x.data_ptr(), tok.data_ptr(), None, None, s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        head.argmax(x.data_ptr(), tok.data_ptr(), None, None, s)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    nbytes = a.rows * nb * 34
    peak = measured_peak()
    gbs = nbytes / us / 1e3
    print(json.dumps({"kernel": "q8_0_head_kernel (+ memset, finish)", "rows": a.rows, "cols": a.cols,
                      "bytes_per_call": nbytes, "us_per_call": us, "achieved_gbs": gbs, "peak_gbs": peak,
                      "frac": gbs / peak, "token": int(tok[0])}))


def dense_case(a):
    import torch
    wd.lib()
    nb = a.cols // 32
    g = torch.Generator(device="cuda").manual_seed(7)
    mats = []
    for m in range(a.mats):
        blocks = torch.randint(0, 256, (a.rows * nb, 18), dtype=torch.uint8, device="cuda", generator=g)
        scale = (torch.rand(a.rows * nb, device="cuda", generator=g) * 0.01 + 0.001).to(torch.float16)
        blocks[:, 0:2] = scale.view(torch.uint8).reshape(-1, 2)
        torch.cuda.synchronize()
        mats.append(wd.DenseQ4_0(a.rows, a.cols, ggml_dev_ptr=blocks.data_ptr()))
        torch.cuda.synchronize()
        del blocks
    x = torch.randn(a.cols, device="cuda", generator=g)
    y = torch.zeros(a.rows, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for i in range(3 * a.mats):
        mats[i % a.mats].matvec(x.data_ptr(), y.data_ptr(), s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters * a.mats):
        mats[i % a.mats].matvec(x.data_ptr(), y.data_ptr(), s)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.iters * a.mats)
    nbytes = a.rows * nb * 18
    peak = measured_peak()
    gbs = nbytes / us / 1e3
    print(json.dumps({"kernel": "q4_0_gemv_kernel", "rows": a.rows, "cols": a.cols, "bytes_per_launch": nbytes,
                      "us_per_launch": us, "achieved_gbs": gbs, "peak_gbs": peak, "frac": gbs / peak,
                      "finite": bool(torch.isfinite(y).all())}))


# ---- load: GGUF file -> repacked HBM slots --------------------------------------------------------------------------


def load_case(a):
    from warpdecode_b200 import synth
    H, F, E, K, SF = 2048, 512, 512, 10, 512
    rng = np.random.Generator(np.random.PCG64(9))
    gb = F * (H // 256) * 110
    meta = {"general.architecture": "qwen4exp", "qwen4exp.block_count": a.layers, "qwen4exp.expert_count": E,
            "qwen4exp.expert_used_count": K, "qwen4exp.embedding_length": H, "qwen4exp.expert_feed_forward_length": F,
            "qwen4exp.expert_shared_feed_forward_length": SF}
    tensors = []
    for l in range(a.layers):
        m = dict(hidden=H, expert_ffn=F, n_experts=E, shared_ffn=SF, gate_type=21, up_type=21, down_type=21,
                 router=rng.integers(0, 256, E * (H // 32) * 34, dtype=np.uint8),
                 gate=rng.integers(0, 256, E * gb, dtype=np.uint8), up=rng.integers(0, 256, E * gb, dtype=np.uint8),
                 down=rng.integers(0, 256, E * gb, dtype=np.uint8),
                 shared_gate_vec=rng.standard_normal(H).astype(np.float32),
                 shared_gate=rng.integers(0, 256, SF * (H // 32) * 34, dtype=np.uint8),
                 shared_up=rng.integers(0, 256, SF * (H // 32) * 34, dtype=np.uint8),
                 shared_down=rng.integers(0, 256, H * (SF // 32) * 34, dtype=np.uint8))
        tensors += synth.moe_block_tensors(m, l)
    path = os.path.join(a.dir, "wd_load_case.gguf")
    synth.write_gguf(path, meta, tensors)
    del tensors
    size = os.path.getsize(path)
    with open(path, "rb") as f:                  # page-cache warm, as the reference's own protocol does
        while f.read(1 << 26):
            pass
    wd.lib()
    wd.Engine(256, 256, 8, 2, 0, 1).close()      # CUDA context and module load happen here, outside the timing
    t0 = time.perf_counter()
    g = wd.Gguf(path)
    c = g.config()
    eng = wd.Engine(c.hidden, c.expert_ffn, c.n_experts, c.top_k, c.shared_ffn, c.n_layers, expert_type=c.gate_type,
                    down_type=c.down_type, w_scale=c.w_scale, rms_eps=c.rms_eps)
    t1 = time.perf_counter()
    wd._check(wd.lib().wd_engine_load_gguf(eng.h, g.h))
    t2 = time.perf_counter()
    expert_bytes = a.layers * E * 3 * gb
    print(json.dumps({"layers": a.layers, "file_bytes": size, "expert_bytes": expert_bytes, "open_create_s": t1 - t0,
                      "load_s": t2 - t1, "expert_gb_per_s": expert_bytes / (t2 - t1) / 1e9,
                      "status": eng.device_status()}))
    eng.close()
    g.close()
    os.remove(path)


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("profile")
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--iters", type=int, default=4)
    p.add_argument("--stamps", action="store_true")
    p.add_argument("--stack", action="store_true", help="run every layer in one launch (wd_stack_step)")
    p.add_argument("--compiled", action="store_true", help="the kernel compiled for the geometry (WD_COMPILED_KERNEL=1)")
    p.set_defaults(fn=profile_case)
    p = sub.add_parser("batch")
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--tokens", type=int, default=4)
    p.add_argument("--iters", type=int, default=4)
    p.add_argument("--stamps", action="store_true")
    p.set_defaults(fn=batch_case)
    p = sub.add_parser("plain")
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--tokens", type=int, default=1)
    p.add_argument("--iters", type=int, default=20)
    p.set_defaults(fn=plain_case)
    p = sub.add_parser("dense-decode")
    p.add_argument("--layers", type=int, default=16)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--gen", type=int, default=64)
    p.add_argument("--runs", type=int, default=3)
    p.set_defaults(fn=dense_decode_case)
    p = sub.add_parser("decoder")
    p.set_defaults(fn=decoder_case)
    p = sub.add_parser("dense")
    p.add_argument("--rows", type=int, default=128256)
    p.add_argument("--cols", type=int, default=2048)
    p.add_argument("--mats", type=int, default=2)
    p.add_argument("--iters", type=int, default=20)
    p.set_defaults(fn=dense_case)
    p = sub.add_parser("head")
    p.add_argument("--rows", type=int, default=151936)
    p.add_argument("--cols", type=int, default=2048)
    p.add_argument("--iters", type=int, default=20)
    p.set_defaults(fn=head_case)
    p = sub.add_parser("load")
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--dir", default="/tmp")
    p.set_defaults(fn=load_case)
    a = ap.parse_args()
    a.fn(a)


if __name__ == "__main__":
    main()
