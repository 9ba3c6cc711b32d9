"""Expert parallelism, host side, on CPU: two gloo ranks.

What runs here without a GPU: the expert partition, the handle exchange, and the claim the GPU path
rests on: if every rank computes the rows of the selected experts it owns and all ranks gather the
rows and combine them in router rank order, the result has the bits of the single-rank block.
The rows come from the CPU oracle (test infrastructure), the exchange is a real all_gather.
"""
import os
import socket

import numpy as np
import pytest

import oracle_lib as ol

H, F, E, K, SF = 512, 256, 32, 6, 256


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class FakeEngine:
    def __init__(self, rank):
        self.rank, self.connected = rank, None

    def ep_export(self):
        return bytes([self.rank]) * 64

    def ep_connect(self, handles):
        self.connected = handles


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import warpdecode_b200 as wd
    from warpdecode_b200 import synth
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # handle exchange: every rank ends up with the others' handles, in rank order, not its own
        fake = FakeEngine(rank)
        wd.ep_connect_all(fake, dist, rank, world)
        assert fake.connected == [bytes([r]) * 64 for r in range(world) if r != rank]
        # partition
        first, count = wd.ep_range(E, rank, world)
        assert (first, count) == (rank * E // world, E // world)
        # deterministic combine over gathered rows
        import torch
        oracle = ol.Oracle()
        m = synth.make_moe_block(900, H, F, E, K, SF, bias_sigma=1.0)
        rng = np.random.Generator(np.random.PCG64(901))
        for rep in range(3):
            x = rng.standard_normal(H).astype(np.float32)
            whole = oracle.moe_block(m, x)
            mine = oracle.moe_block(m, x, first, count)
            assert np.array_equal(mine["ids"], whole["ids"])            # replicated router: same selection
            owned = np.array([first <= e < first + count for e in whole["ids"]])
            rows = torch.from_numpy(np.where(owned[:, None], mine["expert_out"], 0).astype(np.float32))
            mask = torch.from_numpy(owned.astype(np.int32))
            all_rows = [torch.zeros_like(rows) for _ in range(world)]
            all_mask = [torch.zeros_like(mask) for _ in range(world)]
            dist.all_gather(all_rows, rows)
            dist.all_gather(all_mask, mask)
            full = np.zeros((K, H), np.float32)
            seen = np.zeros(K, np.int32)
            for r in range(world):
                mk = all_mask[r].numpy().astype(bool)
                full[mk] = all_rows[r].numpy()[mk]
                seen += mk
            assert np.all(seen == 1)                                    # every selected expert has one owner
            acc = np.zeros(H, np.float32)
            for j in range(K):                                          # add_rn(acc, mul_rn(row, w)) in rank order
                acc = (acc + (full[j] * whole["weights"][j]).astype(np.float32)).astype(np.float32)
            out = (acc + (whole["shared"] * whole["shared_gate"][0]).astype(np.float32)).astype(np.float32)
            assert np.array_equal(ol.fbits(acc), ol.fbits(whole["routed"]))
            assert np.array_equal(ol.fbits(out), ol.fbits(whole["out"]))
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_partition_exchange_and_ordered_combine(tmp_path):
    import torch.multiprocessing as mp
    ol.build_oracle()
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_partition_refuses_uneven_shares():
    import warpdecode_b200 as wd
    assert wd.ep_range(512, 3, 8) == (192, 64)
    with pytest.raises(ValueError):
        wd.ep_range(512, 0, 3)
    with pytest.raises(ValueError):
        wd.ep_range(512, 8, 8)
