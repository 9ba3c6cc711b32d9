"""Times model load from a GGUF file: wd_gguf_open + wd_engine_create + wd_engine_load_gguf for a few layers of
the headline shape (692 MB of expert tensors per layer), all experts resident.

    python -m warpdecode_b200.load_case [--layers 2] [--dir /tmp]

The file holds random block bytes (a load does not look at the values); it is written once, read back once to
warm the page cache, loaded, and deleted. Prints GB/s of expert bytes from file to repacked HBM slots.
"""
import argparse
import json
import os
import time

import numpy as np

import warpdecode_b200 as wd
from warpdecode_b200 import synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--dir", default="/tmp")
    a = ap.parse_args()
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


if __name__ == "__main__":
    main()
