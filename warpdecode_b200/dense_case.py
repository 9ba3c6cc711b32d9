"""Streams Q4_0 matrices of the plain decoder's output-head size through the dense matvec kernel and
prints the achieved HBM bandwidth (algorithmic bytes = 18 bytes per 32 weights, read once).

    python -m warpdecode_b200.dense_case [--rows 128256] [--cols 2048] [--mats 2] [--iters 20]

Two matrices of 148 MB alternate, so the 126 MB L2 cannot serve the reads. Random block bytes with
small f16 scales, generated on the device; about 0.6 GB held.
"""
import argparse
import json
import os

import torch

import warpdecode_b200 as wd


def head_case(a):
    """Q8_0 matrix [rows][cols] (default: the 48-layer decoder's head, 151936 x 2048 = 331 MB) + arg-max."""
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
    peak = 6650.0
    try:
        peak = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                 "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    gbs = nbytes / us / 1e3
    print(json.dumps({"kernel": "q8_0_head_kernel (+ memset, finish)", "rows": a.rows, "cols": a.cols,
                      "bytes_per_call": nbytes, "us_per_call": us, "achieved_gbs": gbs, "peak_gbs": peak,
                      "frac": gbs / peak, "token": int(tok[0])}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=128256)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--mats", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--head", action="store_true", help="Q8_0 output head with fused arg-max instead of the Q4_0 matvec")
    a = ap.parse_args()
    if a.head:
        return head_case(a)
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
    peak = 6650.0
    try:
        peak = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                 "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    gbs = nbytes / us / 1e3
    print(json.dumps({"kernel": "q4_0_gemv_kernel", "rows": a.rows, "cols": a.cols, "bytes_per_launch": nbytes,
                      "us_per_launch": us, "achieved_gbs": gbs, "peak_gbs": peak, "frac": gbs / peak,
                      "finite": bool(torch.isfinite(y).all())}))


if __name__ == "__main__":
    main()
