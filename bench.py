"""Bench of the batch-1 MoE decode hot path (48-layer, 512-expert IQ3_S MoE stack).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one decode token through the 48 MoE blocks of the synthetic model (hidden 2048, 512
routed experts of ffn 512 in IQ3_S, top-10, one Q8_0 shared expert per layer, every expert resident
in HBM; weights N(0, 0.02) generated on the device from seed 3). Each layer reads different weights
(863 MB per token, far beyond the 126 MB L2), so no cache flush is needed between steps.
With N > 1 (one process per GPU under torchrun) the same single token stream runs expert-parallel:
rank r holds experts [r*512/N, (r+1)*512/N) of every layer, router and shared expert are replicated,
the router gets a per-expert N(0, 1) bias (skewed load), and the ranks' kernels exchange expert output
rows over NVLink inside the layer kernel. The job still decodes ONE stream, so scaling is "strong".
Prints ONE JSON line (rank 0).
"""
import argparse
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
SEED, SIGMA = 3, 0.02
EXPERT_BYTES = 3 * 450560
LAYER_BYTES = 10 * EXPERT_BYTES + 3 * 1114112 + 8192 + 1114112     # routed + shared + gate vec + router
# dram__bytes_read + dram__bytes_write of moe_layer_kernel per layer, from an ncu capture of a two-layer
# launch of the same shape (36.18 MB + 0.09 MB for two layers); every layer reads its own weights once,
# so a launch of n layers moves n times this.
TRAFFIC_PER_LAYER = 18_137_000
METRIC = "batch-1 decode tok/s (48L 512-expert IQ3_S MoE)"
WORKLOAD = ("cfg2 MoE stack: 48 layers x (router top-10 of 512 IQ3_S experts + Q8_0 shared expert), "
            "hidden 2048, all experts resident; per token x=RMSNorm(residual), residual+=moe(x); "
            "attention/GDN mixers, embedding and head are not part of the path")


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
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
    sm = sorted(float(s[1]) for s in samples if s[1].replace(".", "").isdigit())
    reasons = set()
    for s in samples:
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
            if v.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": float(samples[0][2]) if samples[0][2].replace(".", "").isdigit() else None,
            "reasons": sorted(reasons)}


def cpu_reference_run(steps, warmup, budget_s=20.0):
    """Times the reference's own host MoE code (oracle/_ref) on the box's host cores: whole blocks of
    the same shape, weights from the same encoders, all threads. Returns (tok/s, description)."""
    import oracle_lib as ol
    from warpdecode_b200 import synth
    ol.build_oracle()
    use_ref = ol.Reference.available()
    ref = ol.Reference() if use_ref else None
    orc = ol.Oracle()
    threads = ref.threads() if use_ref else 1
    H, F, E, K, SF = CFG["hidden"], CFG["expert_ffn"], CFG["n_experts"], CFG["top_k"], CFG["shared_ffn"]
    n_sample_layers = 2
    rng = np.random.Generator(np.random.PCG64(SEED))
    layers = []
    gb = F * (H // 256) * 110
    for l in range(n_sample_layers):
        normal = lambda shape: (rng.standard_normal(shape, dtype=np.float32) * np.float32(SIGMA))
        m = dict(hidden=H, expert_ffn=F, shared_ffn=SF, n_experts=E, top_k=K, gate_type=21, up_type=21,
                 down_type=21, w_scale=1.0)
        m["router"] = synth.quantize_q8_0(normal((E, H))).reshape(-1)
        m["shared_gate_vec"] = normal((H,))
        m["shared_gate"] = synth.quantize_q8_0(normal((SF, H))).reshape(-1)
        m["shared_up"] = synth.quantize_q8_0(normal((SF, H))).reshape(-1)
        m["shared_down"] = synth.quantize_q8_0(normal((H, SF))).reshape(-1)
        x = rng.standard_normal(H, dtype=np.float32)
        xq = orc.quantize_q8_0(x)
        rb = H // 32 * 34
        logits = np.array([orc.row(ol.TYPE_Q8_0, m["router"][e * rb:(e + 1) * rb], xq, H) for e in range(E)], np.float32)
        _, ids, _ = orc.router(logits, K)
        gate, up, down = np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8), np.zeros(E * gb, np.uint8)
        for e in map(int, ids):       # only the experts this input selects are ever read
            gate[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((F, H))).reshape(-1)
            up[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((F, H))).reshape(-1)
            down[e * gb:(e + 1) * gb] = synth.quantize_iq3_s(normal((H, F))).reshape(-1)
        m.update(gate=gate, up=up, down=down)
        layers.append((m, x))
    run = (lambda m, x: ref.moe_block(m, x, threads)) if use_ref else (lambda m, x: orc.moe_block(m, x))
    for _ in range(max(warmup, 1)):
        for m, x in layers:
            run(m, x)
    per_step = []
    t_begin = time.perf_counter()
    for s in range(max(steps, 1)):
        t0 = time.perf_counter()
        for m, x in layers:
            run(m, x)
        per_step.append((time.perf_counter() - t0) / n_sample_layers)
        if time.perf_counter() - t_begin > budget_s:
            break
    layer_s = float(np.mean(per_step))
    tok_s = 1.0 / (layer_s * CFG["n_layers"])
    desc = (f"{len(per_step)} timed passes over {n_sample_layers} full MoE blocks (router + 10 experts + shared "
            f"expert, config shapes); tok/s = 1 / (48 x mean block time {layer_s * 1e3:.3f} ms)")
    return tok_s, {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "reference" if use_ref else "port",
                   "sample": desc}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=CFG["n_layers"], help="debug only; the bench line needs 48")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        tok_s, cpu = cpu_reference_run(args.steps, args.warmup, budget_s=120.0)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tok_s, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x IQ3_S/Q8_0 blocks, f32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOAD, "timed_on": "host CPU cores"},
            "cpu_baseline": cpu,
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    import torch.distributed as dist
    import warpdecode_b200 as wd

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    wd.lib()
    H = CFG["hidden"]
    eng = wd.Engine(H, CFG["expert_ffn"], CFG["n_experts"], CFG["top_k"], CFG["shared_ffn"], args.layers,
                    ep_rank=rank, ep_size=world, device=local_rank)
    t0 = time.perf_counter()
    eng.synth_model(SEED, SIGMA, 1.0 if world > 1 else 0.0)
    torch.cuda.synchronize()
    gen_s = time.perf_counter() - t0
    if world > 1:
        wd.ep_connect_all(eng, dist, rank, world)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    g = torch.Generator(device="cpu").manual_seed(SEED)
    res0 = torch.randn(H, generator=g, dtype=torch.float32)
    residual = res0.cuda()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------------
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            eng.stack_step_device(residual.data_ptr(), sp)
    barrier()
    stop, samples = threading.Event(), []
    th = threading.Thread(target=sample_clocks, args=(stop, samples), daemon=True)
    th.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            eng.stack_step_device(residual.data_ptr(), sp)
        ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    # ---- end to end through host buffers ---------------------------------------------------------
    host = res0.numpy().copy()
    for _ in range(3):
        host = eng.stack_step_host(host)
    barrier()
    e2e_steps = max(10, args.steps // 4)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host = eng.stack_step_host(host)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    stop.set()
    th.join(timeout=2)
    status = eng.device_status()
    if not np.all(np.isfinite(host)) or status != 0:
        raise SystemExit(f"bench: invalid run (device status {status}, finite={bool(np.all(np.isfinite(host)))})")
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    launches = args.steps                    # one launch of the layer kernel per token (on every rank)
    launch_s = ms * 1e-3 / launches
    # algorithmic bytes of one token over all ranks: the selected experts once, router + shared expert per rank
    replicated = 3 * 1114112 + 8192 + 1114112
    token_bytes = args.layers * (10 * EXPERT_BYTES + world * replicated)
    achieved = token_bytes / launch_s / 1e9
    peak *= world
    tok_s = args.steps / (ms * 1e-3)         # one token stream, whatever the number of ranks
    cpu_tok_s, cpu = cpu_reference_run(20, 1, budget_s=15.0)
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "int8 x IQ3_S/Q8_0 blocks, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": args.layers, "parallelism": f"ep{world} (experts sharded, router bias N(0,1))" if world > 1 else "1 GPU",
                   "l2": "863 MB of distinct weights per step, no flush needed", "model_gen_s": round(gen_s, 2)},
        "e2e": {"value": e2e_steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": H * 4,
                "d2h_bytes_per_step": H * 4},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "moe_layer_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": TRAFFIC_PER_LAYER * args.layers if world == 1 else None,
                     "peak_source": "measured" if peaks else "fallback",
                     "bytes_per_launch": token_bytes, "us_per_launch": launch_s * 1e6,
                     "us_per_layer": launch_s * 1e6 / args.layers},
        "cpu_baseline": cpu,
        "clocks": clocks_summary(samples),
    }
    if world > 1:
        dist.destroy_process_group()
    # the JSON line must be the LAST line on stdout: native libraries (NCCL's version banner) write through C stdio,
    # which is block-buffered on a pipe, so that buffer is emptied first
    import ctypes
    try:
        ctypes.CDLL(None).fflush(None)
    except Exception:
        pass
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
