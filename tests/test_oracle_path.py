"""The oracle against the committed golden vectors and an independent numpy restatement (CPU)."""
import os
import sys

import numpy as np
import pytest

import kvo
import scenarios

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_attention_matches_golden(name):
    q, pool, table, kv_len, bs, scale = make_golden.case_inputs(name)
    ref_out = GOLDEN[name + "/out"].astype(np.float64)
    ref_lse = GOLDEN[name + "/lse"].astype(np.float64)
    for use_double in (False, True):
        out, lse = kvo.mla_decode(q, pool, table, kv_len, bs, scale, use_double=use_double)
        scenarios.check_attention(out, lse, ref_out, ref_lse, what=f"{name} double={use_double}",
                                  strict_abs=not name.startswith("sharp"))


def test_golden_is_what_the_numpy_restatement_computes():
    q, pool, table, kv_len, bs, scale = make_golden.case_inputs("ragged_bs64")
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, scale)
    assert np.allclose(GOLDEN["ragged_bs64/out"], ref_out.astype(np.float32))
    assert np.allclose(GOLDEN["ragged_bs64/lse"], ref_lse.astype(np.float32))


def test_append_then_gather_round_trip_bit_exact():
    bs, blocks = 64, 12
    kv_len = np.array([129, 1, 64, 200], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = np.full((blocks * bs, kvo.ROW), 0x7FC1, dtype=np.uint16)  # poison
    rows_total = int(kv_len.sum())
    src = kvo.normal_bf16(rows_total * kvo.ROW, kvo.STREAM_NEW).reshape(rows_total, kvo.ROW)
    slots, at = [], 0
    for b, n in enumerate(kv_len):
        j = np.arange(n)
        slots.append(table[b, j // bs].astype(np.int64) * bs + j % bs)
    slots = np.concatenate(slots).astype(np.int32)
    assert kvo.append(pool, src[:, :512], src[:, 512:], slots) == 0
    # every written row equals its source, every other row is still poison
    assert (pool[slots] == src).all()
    untouched = np.ones(blocks * bs, dtype=bool)
    untouched[slots] = False
    assert (pool[untouched] == 0x7FC1).all()
    out_l, out_r, offsets = kvo.gather(pool, table, kv_len, bs)
    assert (out_l == src[:, :512]).all() and (out_r == src[:, 512:]).all()
    assert list(offsets) == [0, 129, 130, 194]


def test_append_split_caches_and_padding_and_bad_slot():
    rows = 256
    lat = np.zeros((rows, 512), dtype=np.uint16)
    rope = np.zeros((rows, 64), dtype=np.uint16)
    src = kvo.normal_bf16(4 * kvo.ROW, kvo.STREAM_NEW).reshape(4, kvo.ROW)
    slots = np.array([5, -1, 255, 256], dtype=np.int32)  # padding row and an out-of-range slot
    bad = kvo.append(lat, np.ascontiguousarray(src[:, :512]), np.ascontiguousarray(src[:, 512:]), slots, rope_pool=rope)
    assert bad == 1
    assert (lat[5] == src[0, :512]).all() and (rope[5] == src[0, 512:]).all()
    assert (lat[255] == src[2, :512]).all() and (rope[255] == src[2, 512:]).all()
    assert int(np.count_nonzero(lat.any(axis=1))) == 2


def test_partials_merge_to_the_direct_result():
    bs, blocks = 64, 40
    kv_len = np.array([1000, 517], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(2, scale=8.0 / 24.0)
    scale = 1.0 / 24.0
    direct, direct_lse = kvo.mla_decode(q, pool, table, kv_len, bs, scale)
    # three KV-range shards on block boundaries; the last shard of sequence 1 is empty
    begins = np.array([[0, 0], [384, 256], [768, 576]], dtype=np.int32)
    lens = np.array([[384, 256], [384, 261], [232, 0]], dtype=np.int32)
    parts = [kvo.mla_decode(q, pool, table, lens[r], bs, scale, kv_begin=begins[r], partial=True) for r in range(3)]
    po = np.stack([p[0].reshape(-1, 512) for p in parts])
    pm = np.stack([p[1].reshape(-1) for p in parts])
    pl = np.stack([p[2].reshape(-1) for p in parts])
    merged, merged_lse = kvo.lse_merge(po, pm, pl)
    a = kvo.bf16_to_f32(merged).reshape(2, 64, 512)
    b = kvo.bf16_to_f32(direct)
    assert np.abs(a - b).max() <= 2e-3 * max(1.0, float(np.abs(b).max()))
    assert np.abs(merged_lse.reshape(2, 64) - direct_lse).max() <= 1e-4


def test_empty_sequence_and_single_token():
    bs, blocks = 64, 4
    kv_len = np.array([0, 1], dtype=np.int32)
    table = np.array([[0], [2]], dtype=np.int32)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(2)
    out, lse = kvo.mla_decode(q, pool, table, kv_len, bs, 1.0 / 24.0)
    assert (out[0] == 0).all() and np.isneginf(lse[0]).all()
    # one token: softmax is 1, the output is that token's latent (already bf16) for every head
    assert (out[1] == pool[2 * bs, :512][None, :]).all()
    po, pm, pl = kvo.mla_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, partial=True)
    assert (pl[0] == 0).all() and np.isneginf(pm[0]).all() and (po[0] == 0).all()


def test_attention_is_invariant_to_where_blocks_live():
    """Moving a sequence's blocks elsewhere in the pool (and updating its table) changes nothing."""
    bs, blocks = 64, 16
    kv_len = np.array([300], dtype=np.int32)
    pool_a = kvo.make_pool(blocks * bs)
    table_a = np.array([[0, 1, 2, 3, 4]], dtype=np.int32)
    perm = np.array([11, 3, 7, 0, 9], dtype=np.int32)
    pool_b = np.full_like(pool_a, 0x7FC1)
    for i, dst in enumerate(perm):
        pool_b[dst * bs:(dst + 1) * bs] = pool_a[i * bs:(i + 1) * bs]
    q = kvo.make_q(1)
    out_a, lse_a = kvo.mla_decode(q, pool_a, table_a, kv_len, bs, 1.0 / 24.0)
    out_b, lse_b = kvo.mla_decode(q, pool_b, perm[None, :], kv_len, bs, 1.0 / 24.0)
    assert (out_a == out_b).all() and (lse_a == lse_b).all()
