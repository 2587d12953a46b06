"""Host logic of the multi-GPU modes, and the N > 1 exchange on CPU ranks (gloo, world size 2)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import b200kv
from b200kv import dist as kvdist
import kvo
import scenarios


def test_lpt_partition_balances_ragged_lengths():
    lens = scenarios.ragged_lengths(256, 512, 32768)
    ranks, loads = kvdist.partition_sequences(lens, 8)
    assert ranks.min() == 0 and ranks.max() == 7
    assert int(loads.sum()) == int(lens.astype(np.int64).sum())
    for r in range(8):
        assert int(lens[ranks == r].astype(np.int64).sum()) == int(loads[r])
    # LPT is within 4/3 of optimal; on 256 ragged sequences it is much tighter than that
    assert loads.max() / loads.mean() < 1.01
    # deterministic: ties broken by index, then by rank
    ranks2, _ = kvdist.partition_sequences(lens, 8)
    assert (ranks == ranks2).all()
    r1, l1 = kvdist.partition_sequences([5, 5, 5], 2)
    assert list(r1) == [0, 1, 0] and list(l1) == [10, 5]


def test_kv_range_split_covers_the_sequence_on_block_boundaries():
    for kv_len, bs, n in [(262144, 64, 8), (262144, 64, 1), (1000, 64, 4), (63, 64, 4), (0, 64, 2), (129, 128, 3)]:
        at = 0
        for r in range(n):
            begin, length = kvdist.split_kv_range(kv_len, bs, n, r)
            assert begin % bs == 0 or length == 0
            assert begin == min(at, kv_len) or length == 0
            at = begin + length if length else at
        assert at == kv_len
    assert kvdist.split_kv_range(262144, 64, 8, 3) == (3 * 32768, 32768)
    with pytest.raises(b200kv.B200KVError):
        kvdist.split_kv_range(100, 64, 2, 2)


def _shard_worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bs, n, blocks = 64, 1000, 20
        kv_len = np.array([n], dtype=np.int32)
        table = scenarios.build_tables(kv_len, bs, blocks)
        pool = kvo.make_pool(blocks * bs)
        q = kvo.make_q(1, scale=8.0 / 24.0)
        begin, length = kvdist.split_kv_range(n, bs, world, rank)
        # each rank's shard partial comes from the oracle here: the exchange and the bookkeeping are under test
        po, pm, pl = kvo.mla_decode(q, pool, table, np.array([length], np.int32), bs, 1.0 / 24.0,
                                    kv_begin=np.array([begin], np.int32), partial=True)
        o, m, l = kvdist.all_gather_partials(torch.from_numpy(po.reshape(64, 512)), torch.from_numpy(pm.reshape(64)),
                                             torch.from_numpy(pl.reshape(64)))
        assert o.shape == (world, 64, 512) and m.shape == (world, 64)
        assert torch.equal(o[rank], torch.from_numpy(po.reshape(64, 512)))
        merged, merged_lse = kvo.lse_merge(o.numpy(), m.numpy(), l.numpy())
        want, want_lse = kvo.mla_decode(q, pool, table, kv_len, bs, 1.0 / 24.0)
        err = np.abs(kvo.bf16_to_f32(merged) - kvo.bf16_to_f32(want[0])).max()
        assert err <= 2e-3 * max(1.0, float(np.abs(kvo.bf16_to_f32(want)).max())), err
        assert np.abs(merged_lse - want_lse[0]).max() <= 1e-4
        # sequence-partitioned mode: ranks agree on who owns what without talking
        lens = scenarios.ragged_lengths(16, 512, 4096)
        ranks, loads = kvdist.partition_sequences(lens, world)
        mine = torch.tensor([int(loads[rank])])
        every = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(every, mine)
        assert sum(int(t) for t in every) == int(lens.astype(np.int64).sum())
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_kv_range_shards_exchange_over_gloo_world_size_2(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_shard_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
