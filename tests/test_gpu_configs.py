"""The benchmark configurations beyond the single-GPU batched one, at sizes that fit one GPU and finish in
seconds: the bookkeeping stress with device-side arena checks after every step, the ragged fragmented
batch of one rank of the 8-GPU partition, and the 262,144-token sequence split by KV range."""
import numpy as np
import pytest
import torch

import b200kv
from b200kv import dist as kvdist
import kvo
import scenarios
from gpu_util import from_dev_bf16, run_decode, status_ok, to_dev_bf16, to_dev_i32
from test_block_pool import churn_steps

pytestmark = pytest.mark.gpu


def test_churn_stress_arena_bit_exact_after_every_step():
    """64 live sequences appended in 256-token chunks to 2048 tokens, 25% finishing each step: block
    tables, free list and the whole pool are compared with the oracle after every step."""
    n_live, bs, target = 64, 64, 2048
    blocks_per_seq = target // bs
    num_blocks = n_live * blocks_per_seq
    order = kvo.permutation(num_blocks)
    pool_host = b200kv.BlockPool(num_blocks, bs, n_live, blocks_per_seq, free_order=order)
    book = kvo.Book(num_blocks, bs, n_live, blocks_per_seq, free_order=order)
    want = np.zeros((num_blocks * bs, kvo.ROW), dtype=np.uint16)      # the arena starts zero-filled
    pool = to_dev_bf16(want)
    view = b200kv.pool_view(pool)
    status = b200kv.new_status()
    for s in range(n_live):
        pool_host.admit(s)
        book.admit(s)
    counter = 0
    for step, finished, grows in churn_steps(n_live=n_live, steps=12):
        slots_all, want_slots = [], []
        for s, n in grows:
            slots_all.append(pool_host.grow(s, n))
            rc, ws = book.grow(s, n)
            assert rc == 0
            want_slots.append(ws)
        slots = np.concatenate(slots_all)
        assert (slots == np.concatenate(want_slots)).all()
        rows = kvo.normal_bf16(len(slots) * kvo.ROW, kvo.STREAM_NEW, first=counter).reshape(len(slots), kvo.ROW)
        counter += rows.size
        rows_d = to_dev_bf16(rows)
        b200kv.append(view, rows_d[:, :512], rows_d[:, 512:], to_dev_i32(slots), status=status)
        assert kvo.append(want, rows[:, :512], rows[:, 512:], slots) == 0
        for s in finished:
            pool_host.release(s)
            book.release(s)
            pool_host.admit(s)
            book.admit(s)
        status_ok(status)
        table, lens, free = book.export()
        assert (pool_host.table() == table).all() and (pool_host.lens() == lens).all()
        assert (pool_host.free_list() == free).all()
        pool_host.validate()
        assert torch.equal(pool.view(torch.int16).cpu(), torch.from_numpy(want.view(np.int16))), f"step {step}"
    # attention over the live sequences reads exactly what the bookkeeping says is theirs
    table, lens, _ = book.export()
    live = np.nonzero(lens)[0][:6]
    q = kvo.make_q(len(live))
    out, lse = run_decode(q, want, table[live], lens[live], bs, 1.0 / 24.0, b200kv.DECODE_TCGEN05)
    ref, ref_lse = kvo.mla_decode(q, want, table[live], lens[live], bs, 1.0 / 24.0, use_double=True)
    scenarios.check_attention(out, lse, kvo.bf16_to_f32(ref).astype(np.float64), ref_lse.astype(np.float64),
                              what="after churn", strict_abs=True)


def test_ragged_batch_of_one_rank_of_the_eight_gpu_partition():
    """256 sequences with lengths in [512, 32768] are partitioned over 8 ranks by length; rank 0's share
    (fragmented tables from a shared shuffled free list) is attended on this GPU and sampled against the
    oracle. Lengths are scaled down by 8 to keep the pool small; the partition is computed at full size."""
    lens_full = scenarios.ragged_lengths(256, 512, 32768)
    ranks, loads = kvdist.partition_sequences(lens_full, 8)
    assert loads.max() / loads.mean() < 1.01
    mine = np.nonzero(ranks == 0)[0]
    kv_len = np.maximum(lens_full[mine] // 8, 1).astype(np.int32)
    bs = 64
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 11
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(len(kv_len))
    out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, b200kv.DECODE_TCGEN05)
    pick = np.array([0, len(kv_len) // 2, len(kv_len) - 1])
    ref, ref_lse = kvo.mla_decode(q[pick], pool, table[pick], kv_len[pick], bs, 1.0 / 24.0, use_double=True)
    scenarios.check_attention(out[pick], lse[pick], kvo.bf16_to_f32(ref).astype(np.float64),
                              ref_lse.astype(np.float64), what="ragged rank share", strict_abs=True)
    # the two kernels agree on every sequence
    out2, lse2 = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, b200kv.DECODE_SIMT)
    assert np.abs(kvo.bf16_to_f32(out) - kvo.bf16_to_f32(out2)).max() <= 2e-3
    assert np.abs(lse - lse2).max() <= 1e-3


@pytest.mark.parametrize("n_shards", [1, 2, 8])
def test_long_context_split_by_kv_range(n_shards):
    """One sequence of 262,144 tokens (one layer: 302 MB): each shard's partial comes from the device, the
    shards are merged by the LSE merge kernel, and the result is held against the oracle on 8 heads."""
    bs, n = 64, 262144
    blocks = n // bs
    table = kvo.permutation(blocks).reshape(1, blocks)
    pool_t = torch.empty((blocks * bs, kvo.ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(pool_t, kvo.BASE_SEED, kvo.STREAM_KV)
    view = b200kv.pool_view(pool_t)
    q_np = kvo.make_q(1, scale=3.0 / 24.0)
    q = to_dev_bf16(q_np)
    tbl = to_dev_i32(table)
    ws = torch.empty(b200kv.decode_workspace_bytes(1), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    po = torch.empty((n_shards, 64, 512), dtype=torch.float32, device="cuda")
    pm = torch.empty((n_shards, 64), dtype=torch.float32, device="cuda")
    pl = torch.empty((n_shards, 64), dtype=torch.float32, device="cuda")
    for r in range(n_shards):
        begin, length = kvdist.split_kv_range(n, bs, n_shards, r)
        b200kv.mla_decode(q, view, tbl, to_dev_i32([length]), bs, 1.0 / 24.0, kv_begin=to_dev_i32([begin]),
                          partial=(po[r:r + 1], pm[r:r + 1], pl[r:r + 1]), workspace=ws, status=status)
    out = torch.empty((64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(64, dtype=torch.float32, device="cuda")
    b200kv.lse_merge(po, pm, pl, out, lse)
    status_ok(status)
    heads = np.arange(0, 64, 8)
    pool_np = from_dev_bf16(pool_t)
    ref, ref_lse = kvo.mla_decode(q_np[:, heads], pool_np, table, np.array([n], np.int32), bs, 1.0 / 24.0)
    scenarios.check_attention(from_dev_bf16(out)[heads][None], lse.cpu().numpy()[heads][None],
                              kvo.bf16_to_f32(ref).astype(np.float64), ref_lse.astype(np.float64),
                              what=f"{n_shards} shards", strict_abs=True)
