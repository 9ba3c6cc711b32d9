"""A small, self-ending workload for profilers (ncu): a few forward calls of the MoE layer kernel
at the headline block shape, with direct launches (no CUDA graph) so every launch is one kernel.

    python -m warpdecode_b200.profile_case [--layers 2] [--iters 4] [--stamps]

Holds about 0.7 GB per layer on the device. With --stamps it prints the kernel's own per-phase
timestamps (mean over CTAs) instead, which needs no profiler.
"""
import argparse

import numpy as np

import warpdecode_b200 as wd

PHASES = ["table", "x_quant", "q8_rows", "barrier1", "select", "issue", "gate_up", "barrier2", "act_quant", "down"]


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
            res = eng.stack_step_host(res)
            if a.stamps:
                st = eng.stamps().astype(np.int64)
                extra = [(st[:, 12] - st[:, 4]).mean(), (st[:, 13] - st[:, 12]).mean(), (st[:, 5] - st[:, 13]).mean(),
                         (st[:, 11] - st[:, 6]).mean()]
                rows.append(np.concatenate([np.diff(st[:, :11], axis=1).mean(0), [st[:, 10].max() - st[:, 0].min()],
                                            extra]))
        a.layers = 1
    else:
        eng.set_profiling(a.stamps)
    for it in range(0 if a.stack else a.iters):
        for layer in range(a.layers):
            eng.forward_host(layer, rng.standard_normal(2048).astype(np.float32))
            if a.stamps:
                st = eng.stamps().astype(np.int64)
                extra = [(st[:, 12] - st[:, 4]).mean(), (st[:, 13] - st[:, 12]).mean(), (st[:, 5] - st[:, 13]).mean(),
                         (st[:, 11] - st[:, 6]).mean()]
                rows.append(np.concatenate([np.diff(st[:, :11], axis=1).mean(0), [st[:, 10].max() - st[:, 0].min()],
                                            extra]))
    assert eng.device_status() == 0
    if a.stamps:
        m = np.array(rows[a.layers:]).mean(0)          # skip the first pass (cold)
        names = PHASES + ["kernel", "select.load", "select.router", "select.rest", "gate_up.first_copy_wait"]
        print("mean ns per phase:", {n: int(v) for n, v in zip(names, m)})
    print("done")


if __name__ == "__main__":
    main()
