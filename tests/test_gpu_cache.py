"""Capped expert cache on the forward path: same bits as the all-resident engine, and the slot
bookkeeping follows the reference's rule (hit -> most recent; miss -> least recently used slot;
src/expert_cache.cuh:2252-2330, :2467)."""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
H, F, E, K, SF, L = 512, 256, 32, 4, 256, 3


def bits(a):
    return ol.fbits(a)


@pytest.fixture(scope="module")
def wd():
    import warpdecode_b200 as w
    w.lib()
    return w


def _model():
    from warpdecode_b200 import synth
    rng = np.random.Generator(np.random.PCG64(55))
    ms = [synth.make_moe_block(500 + l, H, F, E, K, SF) for l in range(L)]
    norms = [(1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32) for _ in range(L)]
    return ms, norms, rng


def _engine(wd, ms, norms, cache_mib):
    eng = wd.Engine(H, F, E, K, SF, L, cache_mib=cache_mib)
    for l in range(L):
        eng.load_block(l, ms[l])
        eng.set_norm(l, norms[l])
    return eng


class LruModel:
    """The slot rule, restated: a list of keys, most recent first."""

    def __init__(self, n_slots):
        self.n, self.keys = n_slots, []
        self.hits = self.misses = self.evictions = 0

    def layer(self, layer, ids):
        want = []
        for x in ids:
            if (layer, int(x)) not in want:
                want.append((layer, int(x)))
        missing = []
        for k in want:
            if k in self.keys:
                self.hits += 1
                self.keys.remove(k)
                self.keys.insert(0, k)
            else:
                missing.append(k)
        for k in missing:
            self.misses += 1
            if len(self.keys) == self.n:
                self.keys.pop()
                self.evictions += 1
            self.keys.insert(0, k)


def test_capped_cache_matches_resident_engine_and_lru_model(wd, oracle):
    ms, norms, rng = _model()
    full = _engine(wd, ms, norms, 0)
    capped = _engine(wd, ms, norms, 3)          # 3 MiB: 18 slots of 168,960 bytes for 96 experts
    assert capped.slot_count() == (3 << 20) // capped.slot_bytes() == 18
    assert full.slot_count() == L * E
    model = LruModel(18)
    for rep in range(6):
        for l in range(L):
            x = rng.standard_normal(H).astype(np.float32)
            want = full.forward_host(l, x)
            got = capped.forward_host(l, x)
            assert np.array_equal(bits(got), bits(want)), (rep, l)
            assert np.array_equal(bits(got), bits(oracle.moe_block(ms[l], x)["out"]))
            model.layer(l, capped.tap("ids"))
            assert capped.cache_stats() == (model.hits, model.misses, model.evictions)
            if rep % 2:     # the same input again: every expert is still in its slot
                before = capped.cache_stats()
                assert np.array_equal(bits(capped.forward_host(l, x)), bits(want))
                model.layer(l, capped.tap("ids"))
                assert capped.cache_stats() == (before[0] + len(set(capped.tap("ids").tolist())), before[1], before[2])
    assert model.evictions > 0 and model.hits > 0
    res = rng.standard_normal(H).astype(np.float32)
    for step in range(3):
        want = full.stack_step_host(res)
        got = capped.stack_step_host(res)
        assert np.array_equal(bits(got), bits(want)), step
        res = want
    assert capped.device_status() == 0
    full.close(), capped.close()


def test_capped_cache_reads_pinned_host_tensors_without_a_bounce_copy(wd):
    import torch
    ms, norms, rng = _model()
    keep = []
    for m in ms:
        for name in ("gate", "up", "down"):
            t = torch.from_numpy(np.ascontiguousarray(m[name])).pin_memory()
            keep.append(t)
            m[name] = t.numpy()
    full = _engine(wd, ms, norms, 0)
    capped = _engine(wd, ms, norms, 1)
    for l in range(L):
        x = rng.standard_normal(H).astype(np.float32)
        assert np.array_equal(bits(capped.forward_host(l, x)), bits(full.forward_host(l, x)))
    assert capped.cache_stats()[1] >= K
    full.close(), capped.close()


def test_cache_smaller_than_one_selection_is_refused(wd):
    with pytest.raises(wd.WdError, match="smaller than one layer"):
        wd.Engine(2048, 512, 512, 10, 512, 2, cache_mib=8)     # 8 MiB < 10 slots of 1.35 MB


def test_capped_cache_at_the_model_shape_streams_misses_and_matches_resident(wd):
    """Hidden 2048, 512 experts, top-10, three layers generated on the device, the cache capped at 64 MiB (49 slots
    for 1,536 experts): a stack launch runs on while the selected experts are resident and stops at the first layer
    that misses; the host streams that layer's experts in from page-locked memory and the stack resumes there.
    Different inputs keep the routing moving, so the cache misses and evicts all the time; every token's residual must
    equal, bit for bit, what an engine with every expert resident computes."""
    Hh, Fh, Eh, Kh, SFh, Lh = 2048, 512, 512, 10, 512, 3
    full = wd.Engine(Hh, Fh, Eh, Kh, SFh, Lh)
    capped = wd.Engine(Hh, Fh, Eh, Kh, SFh, Lh, cache_mib=64)
    assert capped.slot_count() == 64 * 2 ** 20 // capped.slot_bytes() and capped.slot_count() < Lh * Eh
    rng = np.random.Generator(np.random.PCG64(77))
    for eng in (full, capped):
        eng.synth_model(41, 0.02, 0.0)
    norms = [(1.0 + 0.1 * rng.standard_normal(Hh)).astype(np.float32) for _ in range(Lh)]
    for eng in (full, capped):
        for l in range(Lh):
            eng.set_norm(l, norms[l])
    for t in range(12):
        res = (rng.standard_normal(Hh) * (1.0 + t % 3)).astype(np.float32)
        a, b = full.stack_step_host(res), capped.stack_step_host(res)
        assert np.array_equal(bits(a), bits(b)), t
        # the same token again: now every expert is resident and the token is a single launch
        before = capped.cache_stats()
        assert np.array_equal(bits(capped.stack_step_host(res)), bits(a)), t
        after = capped.cache_stats()
        assert after[1] == before[1] and after[0] == before[0] + Lh * Kh
    hits, misses, evictions = capped.cache_stats()
    sent, host_ns, placed = capped.cache_stream_stats()
    assert misses > 100 and evictions > 50 and hits > 0
    assert sent == misses * 3 * 450560 and placed > 0
    assert capped.device_status() == 0 and full.device_status() == 0
    full.close()
    capped.close()
