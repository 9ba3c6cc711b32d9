"""Bench of the batch-1 MoE decode hot path (48-layer, 512-expert IQ3_S MoE stack).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl reference]
                  [--cache-mib M] [--no-decode] [--no-verify] [--no-dense] [--no-plain]

One step = one decode token through the 48 MoE blocks of the synthetic model (hidden 2048, 512
routed experts of ffn 512 in IQ3_S, top-10, one Q8_0 shared expert per layer, every expert resident
in HBM; weights N(0, 0.02) generated on the device from seed 3; the router logits carry a per-expert
N(0, 1) bias at every N, so that 1, 2, 4 and 8 GPUs run the SAME model). Each layer reads different
weights (863 MB per token, far beyond the 126 MB L2), so no cache flush is needed between steps.
With N > 1 (one process per GPU under torchrun) the same single token stream runs expert-parallel:
rank r holds experts [r*512/N, (r+1)*512/N) of every layer, router and shared expert are replicated,
and the ranks' kernels exchange expert output rows over NVLink inside the layer kernel. The job still
decodes ONE stream, so scaling is "strong".

The K timed steps are repeated R times (each repeat bracketed by a synchronise + barrier); `value` is
K / median repeat time, `repeats` holds the spread. Before the timing a fixed validation pass (8 steps
from the seeded start vector) leaves `residual_sha`, the hash of the final residual bits: it does not
depend on --steps/--warmup, and it is the same at every N when expert parallelism reproduces one GPU.
Besides the MoE-stack value the line carries `decode`: the device-resident greedy loop (embedding row
-> 48 MoE blocks -> Q8_0 head over 151,936 rows -> arg-max, no host synchronisation inside), so that
the head's 331 MB per token count too.

Prints ONE JSON line (rank 0) as the last line of stdout; a failing run prints {"error": ...} there.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CFG = dict(hidden=2048, expert_ffn=512, n_experts=512, top_k=10, shared_ffn=512, n_layers=48)
VOCAB = 151936
SEED, SIGMA, BIAS_SIGMA = 3, 0.02, 1.0
EXPERT_BYTES = 3 * 450560
REPLICATED_BYTES = 3 * 1114112 + 8192 + 1114112                      # shared expert + gate vector + router
LAYER_BYTES = 10 * EXPERT_BYTES + REPLICATED_BYTES
HEAD_BYTES = VOCAB * (CFG["hidden"] // 32) * 34
# dram__bytes_read + dram__bytes_write of the layer kernel per layer, from an ncu capture of a two-layer
# launch of the same shape; every layer reads its own weights once, so a launch of n layers moves n times this.
TRAFFIC_PER_LAYER = 18_137_000
METRIC = "batch-1 decode tok/s (48L 512-expert IQ3_S MoE)"
WORKLOAD = ("cfg2/cfg3 MoE stack: 48 layers x (router top-10 of 512 IQ3_S experts + Q8_0 shared expert), "
            "hidden 2048, all experts resident, router bias N(0,1) at every N; per token x=RMSNorm(residual), "
            "residual+=moe(x); attention/GDN mixers are not part of the path (`decode` adds embedding + head)")
DTYPE = "int8 x IQ3_S/Q8_0 blocks, f32 accumulate"


def emit(line):
    """The JSON line must be the LAST line on stdout: native libraries (NCCL's version banner) write through
    C stdio, which is block-buffered on a pipe, so that buffer is emptied first."""
    import ctypes
    try:
        ctypes.CDLL(None).fflush(None)
    except Exception:
        pass
    print(json.dumps(line), flush=True)


def config_dict(args, world, timed_on):
    return {"workload": WORKLOAD, "layers": args.layers, "timed_on": timed_on,
            "parallelism": f"ep{world} (experts sharded contiguously)" if world > 1 else "1 GPU",
            "l2": "863 MB of distinct weights per step, no flush needed",
            "timing": f"median over repeats (at least {args.repeats}, about 3 s in all) of {args.steps} steps each"}


def sample_clocks(stop, out):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    while not stop.is_set():
        try:
            r = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                os.environ.get("LOCAL_RANK", "0")], capture_output=True, text=True, timeout=5)
            for line in r.stdout.strip().splitlines():
                out.append([c.strip() for c in line.split(",")])
        except Exception:
            pass
        stop.wait(0.2)


def clocks_summary(samples):
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
    sm = sorted(float(s[1]) for s in samples if s[1].replace(".", "").isdigit())
    reasons = set()
    for s in samples:
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
            if v.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": float(samples[0][2]) if samples[0][2].replace(".", "").isdigit() else None,
            "reasons": sorted(reasons), "samples": len(samples)}


def cpu_reference_run(steps, warmup, budget_s=20.0, n_blocks=8):
    """Times the reference's own host MoE code (oracle/_ref) on the box's host cores: `n_blocks` distinct
    whole blocks of the config's shape (weights from the same encoders), all the threads the reference
    would use. Returns (tok/s, description)."""
    import oracle_lib as ol
    from warpdecode_b200 import synth
    ol.build_oracle()
    use_ref = ol.Reference.available()
    ref = ol.Reference() if use_ref else None
    orc = ol.Oracle()
    threads = ref.threads() if use_ref else 1
    H, F, E, K, SF = CFG["hidden"], CFG["expert_ffn"], CFG["n_experts"], CFG["top_k"], CFG["shared_ffn"]
    rng = np.random.Generator(np.random.PCG64(SEED))
    layers = []
    gb = F * (H // 256) * 110
    for l in range(n_blocks):
        normal = lambda shape: (rng.standard_normal(shape, dtype=np.float32) * np.float32(SIGMA))
        m = dict(hidden=H, expert_ffn=F, shared_ffn=SF, n_experts=E, top_k=K, gate_type=21, up_type=21,
                 down_type=21, w_scale=1.0)
        m["router"] = synth.quantize_q8_0(normal((E, H))).reshape(-1)
        m["router_bias"] = (rng.standard_normal(E, dtype=np.float32) * np.float32(BIAS_SIGMA))
        m["shared_gate_vec"] = normal((H,))
        m["shared_gate"] = synth.quantize_q8_0(normal((SF, H))).reshape(-1)
        m["shared_up"] = synth.quantize_q8_0(normal((SF, H))).reshape(-1)
        m["shared_down"] = synth.quantize_q8_0(normal((H, SF))).reshape(-1)
        x = rng.standard_normal(H, dtype=np.float32)
        xq = orc.quantize_q8_0(x)
        rb = H // 32 * 34
        logits = np.array([orc.row(ol.TYPE_Q8_0, m["router"][e * rb:(e + 1) * rb], xq, H) for e in range(E)], np.float32)
        _, ids, _ = orc.router(logits + m["router_bias"], K)
        gate, up, down = np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8)
        for e in map(int, ids):       # only the experts this input selects are ever read
            gate[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((F, H))).reshape(-1)
            up[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((F, H))).reshape(-1)
            down[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((H, F))).reshape(-1)
        m.update(gate=gate, up=up, down=down)
        layers.append((m, x))
    run = (lambda m, x: ref.moe_block(m, x, threads)) if use_ref else (lambda m, x: orc.moe_block(m, x))
    for _ in range(max(min(warmup, 2), 1)):
        for m, x in layers:
            run(m, x)
    per_step = []
    t_begin = time.perf_counter()
    for s in range(max(steps, 1)):
        t0 = time.perf_counter()
        for m, x in layers:
            run(m, x)
        per_step.append((time.perf_counter() - t0) / n_blocks)
        if time.perf_counter() - t_begin > budget_s:
            break
    layer_s = float(np.median(per_step))
    tok_s = 1.0 / (layer_s * CFG["n_layers"])
    desc = (f"{len(per_step)} timed passes over {n_blocks} distinct full MoE blocks (router + 10 experts + shared "
            f"expert, config shapes); tok/s = 1 / (48 x median block time {layer_s * 1e3:.3f} ms)")
    return tok_s, {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "reference" if use_ref else "port",
                   "sample": desc}


def token_hash(tokens):
    """FNV-1a over the little-endian token ids (the reference's token_hash, src/qwen38_forward.cuh:3866-3876)."""
    h = 0xcbf29ce484222325
    for t in tokens:
        for b in int(t).to_bytes(4, "little", signed=True):
            h = ((h ^ b) * 0x100000001b3) & 0xffffffffffffffff
    return f"{h:016x}"


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import warpdecode_b200 as wd

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    wd.lib()
    H = CFG["hidden"]
    capped = args.cache_mib > 0
    eng = wd.Engine(H, CFG["expert_ffn"], CFG["n_experts"], CFG["top_k"], CFG["shared_ffn"], args.layers,
                    ep_rank=rank, ep_size=world, device=local_rank, cache_mib=args.cache_mib, max_tokens=4)
    t0 = time.perf_counter()
    # cfg4 (capped expert cache) is the unbiased model from seed 5, unless --cache-bias asks for cfg3's skewed router
    seed, bias_sigma = (5, args.cache_bias) if capped else (SEED, BIAS_SIGMA)
    eng.synth_model(seed, SIGMA, bias_sigma)
    torch.cuda.synchronize()
    gen_s = time.perf_counter() - t0

    def barrier():
        # The layer kernel is a cooperative launch that takes every SM and waits for its peers: no NCCL kernel may
        # be in flight beside queued layer kernels. So the launch stream is drained first, then the ranks meet.
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if world > 1:
        wd.ep_connect_all(eng, dist, rank, world)
    barrier()
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    g = torch.Generator(device="cpu").manual_seed(SEED)
    res0 = torch.randn(H, generator=g, dtype=torch.float32)
    residual = res0.cuda()

    def steps(n):
        with torch.cuda.stream(stream):
            for _ in range(n):
                eng.stack_step_device(residual.data_ptr(), sp)

    def check_status(where):
        status = eng.device_status()
        if status != 0:
            raise RuntimeError(f"device status {status} after {where} (1 wait timeout, 2 copy timeout, "
                               "4 expert without slot, 8 geometry, 16 exchange overrun)")

    # ---- validation pass: 8 steps from the seeded start, hash of the residual bits ---------------------------------
    steps(8)
    barrier()
    check_status("the validation pass")
    final = residual.cpu().numpy()
    if not np.all(np.isfinite(final)):
        raise RuntimeError("the validation pass left a non-finite residual")
    sha = hashlib.sha256(final.tobytes()).hexdigest()[:16]
    ids_sha = hashlib.sha256(eng.tap("ids").tobytes()).hexdigest()[:16]
    identical = True
    if world > 1:
        every = [None] * world
        dist.all_gather_object(every, (sha, ids_sha))
        identical = all(v == every[0] for v in every)
        barrier()
        if not identical:
            raise RuntimeError(f"ranks disagree on the residual after 8 steps: {every}")

    # ---- device-resident timing: R repeats of K steps ----------------------------------------------------------------
    steps(max(args.warmup, 3))
    barrier()
    stop, samples = threading.Event(), []
    th = threading.Thread(target=sample_clocks, args=(stop, samples), daemon=True)
    th.start()
    rep_ms = []
    n_rep = args.repeats
    while len(rep_ms) < n_rep:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(args.steps):
                eng.stack_step_device(residual.data_ptr(), sp)
            ev1.record(stream)
        barrier()
        rep_ms.append(ev0.elapsed_time(ev1))
        if len(rep_ms) == 1:
            # enough repeats for about three seconds under load, so that the clock sampler sees the timed region;
            # rank 0 decides for everyone
            want = [min(300, max(args.repeats, int(3000.0 / max(rep_ms[0], 1e-3)) + 1))]
            if world > 1:
                dist.broadcast_object_list(want, src=0)
                barrier()
            n_rep = want[0]
    stop.set()
    th.join(timeout=2)
    check_status("the timed steps")
    # ---- end to end through host buffers -------------------------------------------------------------------------------
    host = res0.numpy().copy()
    for _ in range(3):
        host = eng.stack_step_host(host)
    barrier()
    e2e_steps = max(10, args.steps)
    e2e_rep = []
    for _ in range(min(args.repeats, 5)):
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host = eng.stack_step_host(host)
        e2e_rep.append((time.perf_counter() - t0) * 1e3)
        barrier()
    check_status("the end-to-end steps")
    if not np.all(np.isfinite(host)):
        raise RuntimeError("the end-to-end steps left a non-finite residual")

    # ---- greedy decode loop on the device: embedding row -> 48 blocks -> head -> arg-max -----------------------
    decode = None
    if not args.no_decode and not capped:
        nb = H // 32
        table = torch.empty(VOCAB * nb * 34, dtype=torch.uint8, device="cuda")
        wd.synth_tensor_device(wd.TYPE_Q8_0, VOCAB, H, 1.0, SEED, 1000, table.data_ptr())
        head_w = torch.empty(VOCAB * nb * 34, dtype=torch.uint8, device="cuda")
        wd.synth_tensor_device(wd.TYPE_Q8_0, VOCAB, H, SIGMA, SEED, 1001, head_w.data_ptr())
        torch.cuda.synchronize()
        head = wd.HeadQ8_0(VOCAB, H, ggml_dev_ptr=head_w.data_ptr())
        torch.cuda.synchronize()
        del head_w
        n_prompt, n_gen = 8, 64
        prompt = np.random.Generator(np.random.PCG64(SEED)).integers(0, VOCAB, n_prompt).astype(np.int32)
        token = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = torch.zeros(n_gen, dtype=torch.int32, device="cuda")
        res = torch.zeros(H, dtype=torch.float32, device="cuda")

        def one(tok_src):
            wd.embed_q8_0(table.data_ptr(), VOCAB, H, tok_src.data_ptr(), res.data_ptr(), sp)
            eng.stack_step_device(res.data_ptr(), sp)
            head.argmax(res.data_ptr(), token.data_ptr(), None, None, sp)

        best, toks = None, None
        ptoks = [torch.tensor([int(t)], dtype=torch.int32, device="cuda") for t in prompt]
        for rep in range(3):                    # fastest of three, as the reference's --bench-repeat protocol
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                for pt in ptoks:                # the prompt: each token through the stack (no batching at batch 1)
                    one(pt)
                ev0.record(stream)
                for t in range(n_gen):
                    one(token)
                    got[t:t + 1].copy_(token, non_blocking=True)
                ev1.record(stream)
            barrier()
            ms_d = ev0.elapsed_time(ev1)
            cur = got.cpu().numpy().tolist()
            if toks is not None and cur != toks:
                raise RuntimeError("greedy decode is not repeatable between runs")
            toks = cur
            best = ms_d if best is None else min(best, ms_d)
        check_status("the greedy decode loop")
        th_ = token_hash(toks)
        same_tokens = True
        if world > 1:
            every = [None] * world
            dist.all_gather_object(every, th_)
            same_tokens = all(v == every[0] for v in every)
            barrier()
            if not same_tokens:
                raise RuntimeError(f"ranks disagree on the greedy tokens: {every}")
        per_tok_bytes = args.layers * (10 * EXPERT_BYTES + world * REPLICATED_BYTES) + world * HEAD_BYTES
        decode = {"value": n_gen / (best * 1e-3), "unit": "tok/s", "tokens": n_gen, "prompt_tokens": n_prompt,
                  "ms_per_token": best / n_gen, "token_hash": th_, "distinct_tokens": len(set(toks)),
                  "launches_per_token": 5, "bytes_per_token": per_tok_bytes,
                  "hbm_frac": per_tok_bytes / (best * 1e-3 / n_gen) / 1e9,
                  "what": "embedding row -> 48 MoE blocks -> Q8_0 head [151936 x 2048] -> arg-max, on one stream, "
                          "no host synchronisation inside; fastest of 3 runs of 64 tokens after an 8-token prompt"}
        head.close()
        del table

    # ---- speculative verify: batches of 4 tokens through the per-layer forward (one launch per layer and batch) --------
    verify = None
    if not args.no_verify:
        gx = torch.Generator(device="cpu").manual_seed(SEED + 1)
        xb = torch.randn(4, H, generator=gx, dtype=torch.float32).cuda()
        ob = torch.zeros(4, H, dtype=torch.float32, device="cuda")

        def passes(n_tok, count):
            with torch.cuda.stream(stream):
                for _ in range(count):
                    for l in range(args.layers):
                        eng.forward_device(l, xb.data_ptr(), ob.data_ptr(), sp, n_tok)

        rates = {}
        for n_tok in (1, 4):
            passes(n_tok, 2)
            barrier()
            best = None
            for _ in range(3):
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    ev0.record(stream)
                passes(n_tok, 10)
                with torch.cuda.stream(stream):
                    ev1.record(stream)
                barrier()
                ms_v = ev0.elapsed_time(ev1)
                best = ms_v if best is None else min(best, ms_v)
            rates[n_tok] = n_tok * 10 / (best * 1e-3)
        check_status("the verify batches")
        if not bool(torch.isfinite(ob).all()):
            raise RuntimeError("the verify batches left non-finite outputs")
        verify = {"value": rates[4], "unit": "tok/s", "tokens_per_call": 4, "single_token_calls": rates[1],
                  "ratio": rates[4] / rates[1], "kernel": eng.batch_kernel_name(),
                  "us_per_call": 4e6 / rates[4] / args.layers,
                  "what": "4 tokens per wd_moe_forward call, 48 calls (one launch each) per batch, against the same "
                          "calls with one token; fastest of 3 runs of 10 batches. The stack value above is the rate "
                          "to compare a verify step with: it is what decoding the same tokens one by one costs"}

    # ---- config 1: the plain Q4_0 decoder (rank 0 of a 1-GPU run only; the MoE engine's memory stays allocated) ------------
    dense = None
    if not args.no_dense and world == 1 and not capped:
        dec = wd.DenseDecoder(2048, 32, 8, 64, 8192, 128256, 16, 128, 1e-5, 500000.0, device=local_rank)
        dec.synth(2, 0.02)
        prompt = np.random.Generator(np.random.PCG64(2)).integers(0, 128256, 8)
        best_ms, toks = None, None
        for _ in range(3):
            toks, ms_d = dec.decode(prompt, 64)
            best_ms = ms_d if best_ms is None else min(best_ms, ms_d)
        q4 = lambda r, c: r * (c // 32) * 18
        tok_bytes = 16 * (q4(3072, 2048) + q4(2048, 2048) + q4(16384, 2048) + q4(2048, 8192)) + q4(128256, 2048)
        us_tok = best_ms * 1e3 / 71
        dense = {"value": 1e6 / us_tok, "unit": "tok/s", "us_per_token": us_tok, "bytes_per_token": tok_bytes,
                 "hbm_gbs": tok_bytes / us_tok / 1e3, "token_hash": token_hash(toks.tolist()),
                 "distinct_tokens": len(set(toks[8:].tolist())), "launches_per_token": 131,
                 "what": "config 1: Llama-style dense decoder (16 layers, hidden 2048, 32 query / 8 KV heads of 64, SwiGLU 8192, "
                         "vocab 128256, RoPE theta 5e5, every 2-D tensor Q4_0 from N(0, 0.02), norms 1), greedy decode of 64 tokens "
                         "after an 8-token prompt, one CUDA-graph replay per token; fastest of 3 runs"}
        dec.close()

    # ---- the block shape of the reference's own model on the plain-layout path (1-GPU run only) -----------------------------
    plain = None
    if not args.no_plain and world == 1 and not capped:
        from warpdecode_b200 import synth
        PH, PF, PE, PK, PSF, PL = 2560, 640, 512, 10, 640, 2
        peng = wd.Engine(PH, PF, PE, PK, PSF, PL, expert_type=synth.TYPE_IQ2_S, down_type=synth.TYPE_IQ4_NL, w_scale=1.25,
                         router_f32=True, max_tokens=4, device=local_rank)
        prng = np.random.Generator(np.random.PCG64(4))
        small = synth.make_moe_block(5, PH, PF, 8, 8, PSF, synth.TYPE_IQ2_S, synth.TYPE_IQ4_NL, sigma=0.02, router_f32=True)
        for l in range(PL):
            m = dict(small)
            m.update(n_experts=PE, top_k=PK, w_scale=1.25)
            m["router_f32"] = (prng.standard_normal(PE * PH) * 0.02).astype(np.float32)
            m["router_bias"] = (prng.standard_normal(PE) * 0.5).astype(np.float32)
            m["gate"] = synth.random_blocks(prng, synth.TYPE_IQ2_S, PE * PF * PH // 256)
            m["up"] = synth.random_blocks(prng, synth.TYPE_IQ2_S, PE * PF * PH // 256)
            m["down"] = synth.random_blocks(prng, synth.TYPE_IQ4_NL, PE * PH * PF // 32)
            peng.load_block(l, m)
        px = torch.randn(4, PH, generator=torch.Generator().manual_seed(2), dtype=torch.float32).cuda()
        po = torch.zeros_like(px)
        us_call = {}
        for n_tok in (1, 4):
            best = None
            for rep in range(4):
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    ev0.record(stream)
                    for _ in range(20):
                        for l in range(PL):
                            peng.forward_device(l, px.data_ptr(), po.data_ptr(), sp, n_tok)
                    ev1.record(stream)
                torch.cuda.synchronize()
                if rep:         # the first round warms up
                    v = ev0.elapsed_time(ev1) * 1e3 / (20 * PL)
                    best = v if best is None else min(best, v)
            us_call[n_tok] = best
        if peng.device_status() != 0 or not bool(torch.isfinite(po).all()):
            raise RuntimeError("the plain-layout calls left a status or non-finite outputs")
        # the reference's own host code on the same block (the last layer's bytes), all its threads: beside, not instead
        cpu_us, cpu_threads = None, None
        try:
            import oracle_lib as ol
            ol.build_oracle()
            if ol.Reference.available():
                pref = ol.Reference()
                cpu_threads = pref.threads()
                xs_host = px.cpu().numpy()
                got = peng.forward_host(PL - 1, xs_host[0])
                want = pref.moe_block(m, xs_host[0], cpu_threads)["out"]
                if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
                    raise RuntimeError("the plain-layout block differs from the reference's host code on the bench input")
                times = []
                for rep in range(6):
                    t0 = time.perf_counter()
                    pref.moe_block(m, xs_host[rep % 4], cpu_threads)
                    times.append(time.perf_counter() - t0)
                cpu_us = float(np.median(times[1:])) * 1e6
        except (ImportError, OSError):
            pass
        p_bytes = PK * (2 * PF * (PH // 256) * 82 + PH * (PF // 32) * 18) + PE * PH * 4 + 3 * PSF * (PH // 32) * 34
        plain = {"us_per_call": us_call[1], "us_per_call_4_tokens": us_call[4], "bytes_per_token_layer": p_bytes,
                 "hbm_gbs": p_bytes / us_call[1] / 1e3, "kernel": peng.kernel_name(), "launches_per_call": 4,
                 "cpu_reference_us_per_call": cpu_us, "cpu_threads": cpu_threads, "equals_cpu_reference": cpu_us is not None,
                 "what": "one MoE block call (wd_moe_forward) at the block shape of the reference's own model: hidden 2560, "
                         "expert_ffn 640, 512 experts, top 10, shared expert 640, IQ2_S gate/up, IQ4_NL down, F32 router with "
                         "bias; two layers of random block bytes, device-resident input, fastest of 3 rounds of 40 calls"}
        peng.close()

    t = torch.tensor([float(np.median(rep_ms)), min(rep_ms), max(rep_ms), float(np.median(e2e_rep))],
                     dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        torch.cuda.synchronize()
    ms, ms_min, ms_max, e2e_ms = (float(v) for v in t)
    cache_stats = eng.cache_stats() + eng.cache_stream_stats() if capped else None
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    launches = args.steps * n_rep               # one launch of the layer kernel per token (on every rank)
    launch_s = ms * 1e-3 / args.steps
    # algorithmic bytes of one token over all ranks: the selected experts once, router + shared expert per rank
    token_bytes = args.layers * (10 * EXPERT_BYTES + world * REPLICATED_BYTES)
    achieved = token_bytes / launch_s / 1e9
    if decode is not None:
        decode["hbm_frac"] = decode["hbm_frac"] / (peak * world)
    peak *= world
    tok_s = args.steps / (ms * 1e-3)            # one token stream, whatever the number of ranks
    cpu_tok_s, cpu = cpu_reference_run(20, 1, budget_s=15.0)
    cfg = config_dict(args, world, "B200, CUDA events on the launch stream")
    if capped:
        cfg["cache_mib"] = args.cache_mib
        cfg["workload"] = ("cfg4 MoE stack: the 48-layer model from seed 5 (router bias sigma %g) with the expert cache capped at %d MiB, "
                           "misses streamed from page-locked host memory" % (args.cache_bias, args.cache_mib))
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": cfg,
        "repeats": {"n": n_rep, "ms_per_step_median": ms / args.steps, "ms_per_step_min": ms_min / args.steps,
                    "ms_per_step_max": ms_max / args.steps},
        "residual_sha": sha, "ids_sha": ids_sha, "ranks_identical": identical,
        "e2e": {"value": e2e_steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": H * 4,
                "d2h_bytes_per_step": H * 4},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": eng.kernel_name(), "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": TRAFFIC_PER_LAYER * args.layers if world == 1 else None,
                     "peak_source": "measured" if peaks else "fallback",
                     "bytes_per_launch": token_bytes, "us_per_launch": launch_s * 1e6,
                     "us_per_layer": launch_s * 1e6 / args.layers,
                     "expert_gemv_frac": args.layers * 10 * EXPERT_BYTES / launch_s / 1e9 / peak},
        "cpu_baseline": cpu,
        "clocks": clocks_summary(samples),
        "model_gen_s": round(gen_s, 2),
    }
    if decode is not None:
        line["decode"] = decode
    if verify is not None:
        line["verify_m4"] = verify
    if dense is not None:
        dense["hbm_frac"] = dense["hbm_gbs"] / peak
        line["dense_cfg1"] = dense
    if plain is not None:
        plain["hbm_frac"] = plain["hbm_gbs"] / peak
        line["plain_ref_shape"] = plain
    if cache_stats is not None:
        hits, misses, evictions, h2d_bytes, host_ns, placed = cache_stats
        line["cache"] = {"cache_mib": args.cache_mib, "slots": eng.slot_count(), "hits": hits, "misses": misses,
                         "evictions": evictions, "hit_rate": hits / max(hits + misses, 1),
                         "h2d_gb_per_token": h2d_bytes / max(placed, 1) * args.layers / 1e9,
                         "host_placement_us_per_layer": host_ns / max(placed, 1) / 1e3,
                         "what": "cfg4: expert cache capped, misses streamed from page-locked host tensors (the whole run, "
                                 "warm-up included); a token is one launch while every selected expert is resident, a layer that misses stops "
                                 "the launch, the host places its experts and the stack resumes there"}
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=CFG["n_layers"], help="debug only; the bench line needs 48")
    ap.add_argument("--cache-mib", type=int, default=0, help="cap the expert cache (cfg4: 8192); 0 = all resident")
    ap.add_argument("--cache-bias", type=float, default=0.0, help="router bias sigma of the capped-cache model (cfg4: 0)")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-dense", action="store_true")
    ap.add_argument("--no-plain", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        tok_s, cpu = cpu_reference_run(args.steps, args.warmup, budget_s=120.0)
        emit({"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
              "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tok_s, "higher_is_better": True,
              "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": DTYPE,
              "data": "synthetic", "config": config_dict(args, args.gpus, "host CPU cores (the reference's CPU MoE path)"),
              "cpu_baseline": cpu,
              "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return
    try:
        run_ours(args, rank, world, local_rank)
    except BaseException as ex:      # the reason must survive torchrun's traceback: one JSON line, then a non-zero exit
        if isinstance(ex, SystemExit) and ex.code in (0, None):
            raise
        emit({"error": f"{type(ex).__name__}: {ex}", "rank": rank, "n_gpus": world, "metric": METRIC})
        os._exit(1)


if __name__ == "__main__":
    main()
