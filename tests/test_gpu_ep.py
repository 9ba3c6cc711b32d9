"""Expert parallelism on two GPUs of one process: every rank must produce the single-GPU bits.

Needs two CUDA devices with peer access; skipped otherwise. The ranks' kernels wait for one another's
rows, so each step launches on both devices before anything synchronises.
"""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


@pytest.fixture(scope="module")
def torch2():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    return torch


H, F, E, K, SF, L = 512, 256, 64, 6, 256, 3


def _blocks_and_norms():
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(77))
    ms = [synth.make_moe_block(300 + l, H, F, E, K, SF, bias_sigma=1.0) for l in range(L)]
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    return ms, norms, rng


def _engine(wd, ms, norms, rank, size, device, compiled=False):
    """compiled: run the kernel compiled for this geometry instead of the generic one (WD_COMPILED_KERNEL is read
    when an engine is created)."""
    import os
    old = os.environ.get("WD_COMPILED_KERNEL")
    os.environ["WD_COMPILED_KERNEL"] = "1" if compiled else "0"
    try:
        eng = wd.Engine(H, F, E, K, SF, L, ep_rank=rank, ep_size=size, device=device)
    finally:
        if old is None:
            os.environ.pop("WD_COMPILED_KERNEL", None)
        else:
            os.environ["WD_COMPILED_KERNEL"] = old
    assert eng.kernel_name() == ("moe_fast_kernel" if compiled else "moe_layer_kernel")
    for l in range(L):
        eng.load_block(l, ms[l])
        eng.set_norm(l, norms[l])
    return eng


@pytest.mark.parametrize("compiled", [False, True])
def test_two_ranks_reproduce_one_gpu_bit_for_bit(wd, oracle, torch2, compiled):
    torch = torch2
    ms, norms, rng = _blocks_and_norms()
    single = _engine(wd, ms, norms, 0, 1, 0)
    ranks = [_engine(wd, ms, norms, r, 2, r, compiled) for r in range(2)]
    ranks[0].ep_connect_local([ranks[1]])
    ranks[1].ep_connect_local([ranks[0]])
    res = rng.standard_normal(H).astype(np.float32)
    dev = [torch.zeros(H, dtype=torch.float32, device=f"cuda:{r}") for r in range(2)]
    for step in range(4):
        want = single.stack_step_host(res)
        ref = res.copy()
        for l in range(L):
            x = oracle.rmsnorm(ref, norms[l], 1e-6)
            ref = (ref + oracle.moe_block(ms[l], x)["out"]).astype(np.float32)
        assert np.array_equal(bits(want), bits(ref))
        for r in range(2):
            dev[r].copy_(torch.from_numpy(res))
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        for r in range(2):
            ranks[r].stack_step_device(dev[r].data_ptr())
        torch.cuda.synchronize(0), torch.cuda.synchronize(1)
        for r in range(2):
            assert ranks[r].device_status() == 0
            assert np.array_equal(bits(dev[r].cpu().numpy()), bits(want)), (step, r)
            assert np.array_equal(ranks[r].tap("ids"), single.tap("ids"))
            assert np.array_equal(bits(ranks[r].tap("expert_out")), bits(single.tap("expert_out")))
        res = want
    # the ranks really split the work: each holds half of the experts
    assert ranks[0].slot_count() == L * E // 2
    for e in ranks + [single]:
        e.ep_disconnect()
        e.close()


@pytest.mark.parametrize("compiled", [False, True])
def test_a_rank_that_owns_nothing_and_launches_late_is_waited_for(wd, oracle, torch2, compiled):
    """Every selected expert belongs to rank 0 (router bias), so nothing rank 0 computes depends on rank 1: without
    flow control it would run layers and whole launches ahead and overwrite rows in rank 1's buffer that rank 1 has
    not combined yet. Rank 1 starts each step late (a host-side sleep, well under the one-second wait limit); both
    ranks must still produce the single-GPU bits, with no status raised."""
    import time
    torch = torch2
    ms, norms, rng = _blocks_and_norms()
    for m in ms:
        b = np.zeros(E, np.float32)
        b[:E // 2] = 100.0                                  # the top-k all come from rank 0's half
        m["router_bias"] = b
    single = _engine(wd, ms, norms, 0, 1, 0)
    ranks = [_engine(wd, ms, norms, r, 2, r, compiled) for r in range(2)]
    ranks[0].ep_connect_local([ranks[1]])
    ranks[1].ep_connect_local([ranks[0]])
    res = rng.standard_normal(H).astype(np.float32)
    n_steps = 3
    want = []
    cur = res
    for step in range(n_steps):
        cur = single.stack_step_host(cur)
        assert max(single.tap("ids")) < E // 2
        want.append(cur)
    dev = [torch.from_numpy(res).to(f"cuda:{r}") for r in range(2)]
    torch.cuda.synchronize(0), torch.cuda.synchronize(1)
    # rank 0 is given all its launches at once; rank 1 follows late, launch by launch
    for step in range(n_steps):
        ranks[0].stack_step_device(dev[0].data_ptr())
    for step in range(n_steps):
        time.sleep(0.15)
        ranks[1].stack_step_device(dev[1].data_ptr())
    torch.cuda.synchronize(0), torch.cuda.synchronize(1)
    for r in range(2):
        assert ranks[r].device_status() == 0
        assert np.array_equal(bits(dev[r].cpu().numpy()), bits(want[-1])), r
    for e in ranks + [single]:
        e.ep_disconnect()
        e.close()


def test_unconnected_ranks_return_partial_sums(wd, oracle, torch2):
    ms, norms, rng = _blocks_and_norms()
    single = _engine(wd, ms, norms, 0, 1, 0)
    ranks = [_engine(wd, ms, norms, r, 2, r) for r in range(2)]
    x = rng.standard_normal(H).astype(np.float32)
    want = single.forward_host(0, x)
    shared = single.tap("shared") * single.tap("shared_gate")[0]
    parts = [ranks[r].forward_host(0, x) - shared for r in range(2)]      # routed partial of each rank
    got = parts[0] + parts[1] + shared
    assert np.allclose(got, want, rtol=1e-3, atol=1e-5)       # a different float order: the 1e-3 contract
    for e in ranks + [single]:
        e.close()


def test_silent_peer_ends_in_a_status_not_a_hang(wd, torch2):
    # rank 1 never launches: rank 0 waits about a second for its rows, then reports and returns
    torch = torch2
    ms, norms, rng = _blocks_and_norms()
    ranks = [_engine(wd, ms, norms, r, 2, r) for r in range(2)]
    ranks[0].ep_connect_local([ranks[1]])
    ranks[1].ep_connect_local([ranks[0]])
    x = torch.from_numpy(rng.standard_normal(H).astype(np.float32)).to("cuda:0")
    ranks[0].stack_step_device(x.data_ptr())
    torch.cuda.synchronize(0)
    assert ranks[0].device_status() & 1
    for e in ranks:
        e.reset_exchange()
    # and the group works again afterwards
    dev = [torch.zeros(H, dtype=torch.float32, device=f"cuda:{r}") for r in range(2)]
    for r in range(2):
        ranks[r].stack_step_device(dev[r].data_ptr())
    torch.cuda.synchronize(0), torch.cuda.synchronize(1)
    assert ranks[0].device_status() == 0 and ranks[1].device_status() == 0
    for e in ranks:
        e.ep_disconnect()
        e.close()
