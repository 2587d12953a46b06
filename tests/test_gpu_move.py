"""Append and gather on the device against the oracle, bit for bit, through the C ABI."""
import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32, to_dev_i64

pytestmark = pytest.mark.gpu

POISON = 0x7FC1  # a bf16 NaN pattern: any stray write or unwritten read shows


def _slots_for(table, kv_len, bs):
    out = []
    for b, n in enumerate(kv_len):
        j = np.arange(int(n))
        out.append(table[b, j // bs].astype(np.int64) * bs + j % bs)
    return np.concatenate(out).astype(np.int32) if out else np.zeros(0, np.int32)


@pytest.mark.parametrize("bs,kv_len", [
    (64, [129]),                       # one sequence at token 129
    (128, [129]),                      # the reference's default block size
    (64, [1, 63, 64, 65, 200, 7]),     # ragged, block-edge lengths
    (64, [2048] * 8),                  # prefill-sized chunk rows
])
def test_append_whole_pool_bit_exact(bs, kv_len):
    kv_len = np.asarray(kv_len, dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 3
    table = scenarios.build_tables(kv_len, bs, blocks)
    slots = _slots_for(table, kv_len, bs)
    rows = len(slots)
    src = kvo.normal_bf16(rows * kvo.ROW, kvo.STREAM_NEW).reshape(rows, kvo.ROW)
    want = np.full((blocks * bs, kvo.ROW), POISON, dtype=np.uint16)
    assert kvo.append(want, src[:, :512], src[:, 512:], slots) == 0

    pool = to_dev_bf16(np.full((blocks * bs, kvo.ROW), POISON, dtype=np.uint16))
    src_d = to_dev_bf16(src)
    status = b200kv.new_status()
    b200kv.append(b200kv.pool_view(pool), src_d[:, :512], src_d[:, 512:], to_dev_i32(slots), status=status)
    status_ok(status)
    assert (from_dev_bf16(pool) == want).all()


def test_append_split_caches_padding_and_bad_slot_status():
    rows = 512
    lat = to_dev_bf16(np.zeros((rows, 512), dtype=np.uint16))
    rope = to_dev_bf16(np.zeros((rows, 64), dtype=np.uint16))
    src = kvo.normal_bf16(5 * kvo.ROW, kvo.STREAM_NEW).reshape(5, kvo.ROW)
    slots = np.array([5, -1, 511, 512, 77], dtype=np.int32)
    want_l = np.zeros((rows, 512), dtype=np.uint16)
    want_r = np.zeros((rows, 64), dtype=np.uint16)
    bad = kvo.append(want_l, np.ascontiguousarray(src[:, :512]), np.ascontiguousarray(src[:, 512:]), slots,
                     rope_pool=want_r)
    assert bad == 1
    src_l = to_dev_bf16(np.ascontiguousarray(src[:, :512]))
    src_r = to_dev_bf16(np.ascontiguousarray(src[:, 512:]))
    status = b200kv.new_status()
    b200kv.append(b200kv.pool_view(lat, rope), src_l, src_r, to_dev_i32(slots), status=status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == b200kv.DEV_BAD_SLOT and st[1] == 3 and st[2] == 512
    assert (from_dev_bf16(lat) == want_l).all() and (from_dev_bf16(rope) == want_r).all()


@pytest.mark.parametrize("case", ["chunks", "mixed", "scattered"])
def test_append_through_shared_memory_on_back_to_back_rows(case):
    """The reference's layout (latent [rows][512] and rope [rows][64] as two arrays, sources of the same shape):
    runs of consecutive slots move as groups of 16 rows through shared memory with bulk copies, everything else
    row by row in the same launch. chunks: the churn configuration's prefill chunk (sequences x 256 tokens into
    64-row blocks). mixed: runs broken by padding, by a slot outside the pool, by block ends at odd offsets and
    by a ragged tail. scattered: no runs at all."""
    bs, blocks = 64, 300
    rows = blocks * bs
    order = kvo.permutation(blocks)
    if case == "chunks":
        slots = np.concatenate([order[4 * s + c].astype(np.int64) * bs + np.arange(bs) for s in range(64) for c in range(4)])
    elif case == "mixed":
        pieces, at = [], 0
        for n in (64, 1, 17, 16, 64, 15, 33, 128, 5, 250):
            pieces.append(order[at].astype(np.int64) * bs + (7 if n < 50 else 0) + np.arange(min(n, bs)))
            if n > bs:
                pieces.append(order[at + 1].astype(np.int64) * bs + np.arange(min(n - bs, bs)))
            at += 3
        slots = np.concatenate(pieces)
        slots[40] = -1           # padding inside a run
        slots[200] = rows + 5    # outside the pool: recorded, skipped
        slots = slots[:-3]       # a ragged last group
    else:
        slots = kvo.permutation(rows)[:5000].astype(np.int64)
    slots = slots.astype(np.int32)
    n = len(slots)
    src = kvo.normal_bf16(n * kvo.ROW, kvo.STREAM_NEW).reshape(n, kvo.ROW)
    src_l, src_r = np.ascontiguousarray(src[:, :512]), np.ascontiguousarray(src[:, 512:])
    want_l = np.full((rows, 512), POISON, dtype=np.uint16)
    want_r = np.full((rows, 64), POISON, dtype=np.uint16)
    bad = kvo.append(want_l, src_l, src_r, slots, rope_pool=want_r)
    assert bad == (1 if case == "mixed" else 0)
    lat = to_dev_bf16(np.full((rows, 512), POISON, dtype=np.uint16))
    rope = to_dev_bf16(np.full((rows, 64), POISON, dtype=np.uint16))
    status = b200kv.new_status()
    for _ in range(2):   # idempotent
        b200kv.append(b200kv.pool_view(lat, rope), to_dev_bf16(src_l), to_dev_bf16(src_r), to_dev_i32(slots), status=status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    if case == "mixed":
        assert st[0] == b200kv.DEV_BAD_SLOT and st[1] == 200 and st[2] == rows + 5, st
    else:
        assert st[0] == 0, st
    assert (from_dev_bf16(lat) == want_l).all() and (from_dev_bf16(rope) == want_r).all()


def test_append_zero_tokens_is_a_no_op():
    pool = to_dev_bf16(np.full((64, kvo.ROW), POISON, dtype=np.uint16))
    empty = torch.empty((0, kvo.ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.append(b200kv.pool_view(pool), empty[:, :512], empty[:, 512:], torch.empty(0, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert (from_dev_bf16(pool) == POISON).all()


@pytest.mark.parametrize("bs,kv_len,fragmented", [
    (64, [129], False),
    (128, [129, 1], False),
    (64, [1, 63, 64, 65, 200, 0, 7], True),
    (64, [4097] * 4, True),
    (64, [1], False),                       # outputs smaller than a tile
    (64, [0, 3], True),
    (192, [500, 191, 193], True),           # blocks of three tiles
    (16, [100, 5], True),                   # blocks smaller than a tile: the register kernel
    (64, [(37 * i) % 150 for i in range(300)], True),   # many short sequences
])
def test_gather_bit_exact(bs, kv_len, fragmented):
    kv_len = np.asarray(kv_len, dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 5
    table = (scenarios.fragmented_tables if fragmented else scenarios.build_tables)(kv_len, bs, blocks)
    pool_np = kvo.make_pool(blocks * bs)
    want_l, want_r, offsets = kvo.gather(pool_np, table, kv_len, bs)
    total = int(kv_len.sum())
    pool = to_dev_bf16(pool_np)
    out_l = to_dev_bf16(np.full((total, 512), POISON, dtype=np.uint16))
    out_r = to_dev_bf16(np.full((total, 64), POISON, dtype=np.uint16))
    status = b200kv.new_status()
    b200kv.gather(b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, out_l, out_r,
                  to_dev_i64(offsets), total, status=status)
    status_ok(status)
    assert (from_dev_bf16(out_l) == want_l).all() and (from_dev_bf16(out_r) == want_r).all()


def test_gather_reports_out_of_range_block():
    bs = 64
    pool = to_dev_bf16(kvo.make_pool(4 * bs))
    table = np.array([[1, 9]], dtype=np.int32)  # block 9 does not exist
    out_l = to_dev_bf16(np.zeros((100, 512), dtype=np.uint16))
    out_r = to_dev_bf16(np.zeros((100, 64), dtype=np.uint16))
    status = b200kv.new_status()
    b200kv.gather(b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32([100]), bs, out_l, out_r, to_dev_i64([0]),
                  100, status=status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == b200kv.DEV_BAD_BLOCK and st[1] == 0 and st[2] == 1 and st[3] == 9
    # rows of the valid block were still gathered
    assert (from_dev_bf16(out_l)[:64] == kvo.make_pool(4 * bs)[64:128, :512]).all()


def test_gather_length_beyond_the_table_row_is_reported_not_read():
    """A device-side length that runs past the sequence's row of the block table: the rows the table covers are
    gathered, the rest is recorded as a bad block; the next sequence's entries are not used in its place."""
    bs = 64
    pool_np = kvo.make_pool(8 * bs)
    pool = to_dev_bf16(pool_np)
    table = np.array([[1, 2], [3, 4]], dtype=np.int32)
    kv_len = np.array([3 * bs, 10], dtype=np.int32)  # sequence 0 claims a third block its row does not have
    total = int(kv_len.sum())
    out_l = to_dev_bf16(np.full((total, 512), POISON, dtype=np.uint16))
    out_r = to_dev_bf16(np.full((total, 64), POISON, dtype=np.uint16))
    status = b200kv.new_status()
    b200kv.gather(b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, out_l, out_r,
                  to_dev_i64([0, 3 * bs]), total, status=status)
    torch.cuda.synchronize()
    st = status.cpu().tolist()
    assert st[0] == b200kv.DEV_BAD_BLOCK and st[1] == 0 and st[2] == 2 and st[3] == -1, st
    got = from_dev_bf16(out_l)
    assert (got[: 2 * bs] == pool_np[bs: 3 * bs, :512]).all()
    assert (got[2 * bs: 3 * bs] == POISON).all(), "rows beyond the table were written from somewhere"
    assert (got[3 * bs:] == pool_np[3 * bs: 3 * bs + 10, :512]).all()


def test_generator_on_device_matches_oracle_bits():
    n = 3_000_001
    dst = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for stream, first, scale in [(kvo.STREAM_KV, 0, 1.0), (kvo.STREAM_Q, 12345, 1.0 / 24.0)]:
        b200kv.fill_normal_bf16(dst, kvo.BASE_SEED, stream, first, scale)
        torch.cuda.synchronize()
        want = kvo.normal_bf16(n, stream, first, scale)
        got = from_dev_bf16(dst)
        mismatches = int((got != want).sum())
        assert mismatches == 0, f"{mismatches} of {n} generator values differ between device and oracle"


def test_append_gather_round_trip_at_full_layer_size():
    """One layer of the B=32 x 4K configuration (2048 blocks of 64 rows = 151 MB): write one new row per
    sequence at position 4096, gather all 4097 rows of every sequence, compare with the pool and sources
    through the block table (size-independent property: gather(append(x)) returns x at the appended rows)."""
    bs, B, ctx = 64, 32, 4096
    blocks = B * (ctx // bs + 1)
    kv_len = np.full(B, ctx + 1, dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = torch.empty((blocks * bs, kvo.ROW), dtype=torch.bfloat16, device="cuda")
    b200kv.fill_normal_bf16(pool, kvo.BASE_SEED, kvo.STREAM_KV)
    new_rows = to_dev_bf16(kvo.normal_bf16(B * kvo.ROW, kvo.STREAM_NEW).reshape(B, kvo.ROW))
    slots = (table[:, ctx // bs].astype(np.int64) * bs + ctx % bs).astype(np.int32)
    view = b200kv.pool_view(pool)
    status = b200kv.new_status()
    b200kv.append(view, new_rows[:, :512], new_rows[:, 512:], to_dev_i32(slots), status=status)
    total = int(kv_len.sum())
    offsets = np.arange(B, dtype=np.int64) * (ctx + 1)
    out_l = torch.empty((total, 512), dtype=torch.bfloat16, device="cuda")
    out_r = torch.empty((total, 64), dtype=torch.bfloat16, device="cuda")
    b200kv.gather(view, to_dev_i32(table), to_dev_i32(kv_len), bs, out_l, out_r, to_dev_i64(offsets), total,
                  status=status)
    status_ok(status)
    # expected rows straight from the pool through the table, with torch indexing
    tok = torch.arange(ctx + 1, device="cuda")
    tbl = to_dev_i32(table).long()
    rows = tbl[:, tok // bs] * bs + (tok % bs)[None, :]
    want = pool[rows.reshape(-1)]
    assert torch.equal(out_l.view(torch.int16), want[:, :512].contiguous().view(torch.int16))
    assert torch.equal(out_r.view(torch.int16), want[:, 512:].contiguous().view(torch.int16))
    last = out_l.view(B, ctx + 1, 512)[:, ctx]
    assert torch.equal(last.contiguous().view(torch.int16), new_rows[:, :512].contiguous().view(torch.int16))
