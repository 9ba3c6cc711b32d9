"""A small, self-ending workload for profilers (ncu): a few forward calls of the MoE layer kernel
at the headline block shape, with direct launches (no CUDA graph) so every launch is one kernel.

    python -m warpdecode_b200.profile_case [--layers 2] [--iters 4] [--stamps] [--stack]

Holds about 0.7 GB per layer on the device. With --stamps it prints the kernel's own per-phase
timestamps (mean over CTAs) instead, which needs no profiler.
"""
import argparse
import time

import numpy as np

import warpdecode_b200 as wd

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--stamps", action="store_true")
    ap.add_argument("--stack", action="store_true", help="run every layer in one launch (wd_stack_step)")
    a = ap.parse_args()
    eng = wd.Engine(2048, 512, 512, 10, 512, a.layers)
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


if __name__ == "__main__":
    main()
