"""The allocation-free matvec entry point (wd_matvec_iq3s_noalloc), called through the C ABI.

It exists for callers that cannot call cudaMalloc while decoding: when the expert pool already owns
nearly all of HBM an allocation can fail, and even a successful one synchronises the device in the
middle of a token. Its scratch is a fixed array inside the library, shared by every call, so the
test makes two calls in a row with different matrices and checks each result, bit for bit, against
the ordinary entry point (wd_matvec_host), which allocates its own buffers, and against the CPU oracle's
row dot on the same block bytes: stale contents of the shared array must never leak into a later
result. The file name keeps it last in collection order.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def test_no_alloc_matvec_matches_allocating_entry_point_twice(oracle):
    import torch
    import warpdecode_b200 as wd
    lib = wd.lib()
    lib.wd_matvec_iq3s_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    rng = np.random.Generator(np.random.PCG64(2024))
    torch.cuda.set_device(0)
    for rows, cols in ((512, 2048), (64, 512)):          # second call: smaller matrix over the first one's tiles
        w = ol.random_blocks(rng, ol.TYPE_IQ3_S, rows * cols // 256)
        x = rng.standard_normal(cols).astype(np.float32)
        want = wd.matvec(ol.TYPE_IQ3_S, w, rows, cols, x)
        w_d = torch.from_numpy(w.copy()).cuda()
        x_d = torch.from_numpy(x).cuda()
        y_d = torch.full((rows,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        rc = lib.wd_matvec_iq3s_noalloc(w_d.data_ptr(), rows, cols, x_d.data_ptr(), y_d.data_ptr(), None)
        assert rc == 0, lib.wd_last_error().decode()
        torch.cuda.synchronize()
        got = y_d.cpu().numpy()
        assert np.array_equal(ol.fbits(got), ol.fbits(want)), (rows, cols)
        # and the oracle itself, row by row, on the same bytes (not only the sibling entry point)
        xk = oracle.quantize_q8_K(x)
        rb = cols // 256 * 110
        ref = np.array([oracle.row(ol.TYPE_IQ3_S, w[r * rb:(r + 1) * rb], xk, cols) for r in range(rows)], np.float32)
        assert np.array_equal(ol.fbits(got), ol.fbits(ref)), (rows, cols)


def test_no_alloc_matvec_refuses_more_than_its_fixed_scratch():
    import torch
    import warpdecode_b200 as wd
    lib = wd.lib()
    lib.wd_matvec_iq3s_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    dummy = torch.zeros(16, device="cuda")
    rows, cols = 16384, 2048                              # 14 MiB of blocks > 8 MiB - 1 KiB
    rc = lib.wd_matvec_iq3s_noalloc(dummy.data_ptr(), rows, cols, dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc != 0
    assert b"exceeds the fixed scratch" in lib.wd_last_error()
