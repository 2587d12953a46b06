"""Host bookkeeping of the product (C++ block pool behind the C ABI) against the oracle's model,
bit for bit: tables, lengths, free-list order, returned slots (CPU)."""
import numpy as np
import pytest

import b200kv
import kvo


def _same(pool: b200kv.BlockPool, book: kvo.Book):
    table, lens, free = book.export()
    assert (pool.table() == table).all()
    assert (pool.lens() == lens).all()
    assert (pool.free_list() == free).all()
    assert pool.free_count == book.free_count
    pool.validate()


def test_grow_release_match_model_with_shuffled_free_list():
    order = kvo.permutation(32)
    pool = b200kv.BlockPool(32, 64, 4, 8, free_order=order)
    book = kvo.Book(32, 64, 4, 8, free_order=order)
    for s in range(4):
        pool.admit(s)
        assert book.admit(s) == 0
    for s, n in [(0, 1), (1, 64), (2, 65), (0, 63), (0, 1), (3, 500), (1, 130)]:
        rc, want = book.grow(s, n)
        assert rc == 0
        assert (pool.grow(s, n) == want).all()
        _same(pool, book)
    pool.release(2)
    assert book.release(2) == 0
    _same(pool, book)
    pool.admit(2)
    book.admit(2)
    rc, want = book.grow(2, 200)
    assert rc == 0 and (pool.grow(2, 200) == want).all()
    _same(pool, book)


def test_failed_calls_change_nothing():
    pool = b200kv.BlockPool(4, 64, 2, 3)
    book = kvo.Book(4, 64, 2, 3)
    pool.admit(0)
    book.admit(0)
    pool.grow(0, 100)
    book.grow(0, 100)
    before = (pool.table(), pool.lens(), pool.free_list())
    with pytest.raises(b200kv.B200KVError) as err:
        pool.grow(0, 100)  # would need 4 blocks, the row holds 3
    assert err.value.code == b200kv.ERR_INVALID and "table row holds 3" in str(err.value)
    assert book.grow(0, 100)[0] == -1
    pool.admit(1)
    book.admit(1)
    with pytest.raises(b200kv.B200KVError) as err:
        pool.grow(1, 64 * 3)  # 3 blocks wanted, 2 free
    assert "2 free of 4" in str(err.value)
    assert book.grow(1, 64 * 3)[0] == -1
    with pytest.raises(b200kv.B200KVError):
        pool.admit(1)  # already live
    with pytest.raises(b200kv.B200KVError):
        pool.release(5)  # out of range
    after = (pool.table(), pool.lens(), pool.free_list())
    for a, b in zip(before, after):
        assert (a == b).all()
    _same(pool, book)


def test_create_refuses_bad_free_order():
    with pytest.raises(b200kv.B200KVError):
        b200kv.BlockPool(4, 64, 1, 4, free_order=[0, 1, 1, 3])
    with pytest.raises(b200kv.B200KVError):
        b200kv.BlockPool(0, 64, 1, 4)


def churn_steps(n_live=64, chunk=256, target=2048, steps=24):
    """The bookkeeping stress: every sequence is appended in `chunk`-token pieces up to `target`; each
    step a seeded 25% of the live sequences finish and are re-admitted empty. Yields
    (step, finished ids, [(seq, n_tokens)])."""
    progress = [0] * n_live
    for step in range(steps):
        grows = []
        for s in range(n_live):
            if progress[s] < target:
                grows.append((s, chunk))
                progress[s] += chunk
        x = kvo.draws(n_live, kvo.STREAM_CHURN, first=step * n_live)
        order = np.argsort(x, kind="stable")
        finished = sorted(int(s) for s in order[: n_live // 4])
        yield step, finished, grows
        for s in finished:
            progress[s] = 0


def test_churn_bit_exact_against_model():
    n_live, bs = 64, 64
    blocks_per_seq = 2048 // bs
    num_blocks = n_live * blocks_per_seq
    order = kvo.permutation(num_blocks)
    pool = b200kv.BlockPool(num_blocks, bs, n_live, blocks_per_seq, free_order=order)
    book = kvo.Book(num_blocks, bs, n_live, blocks_per_seq, free_order=order)
    for s in range(n_live):
        pool.admit(s)
        book.admit(s)
    for step, finished, grows in churn_steps():
        for s, n in grows:
            rc, want = book.grow(s, n)
            assert rc == 0
            assert (pool.grow(s, n) == want).all()
        for s in finished:
            pool.release(s)
            book.release(s)
            pool.admit(s)
            book.admit(s)
        _same(pool, book)
    # the free list has been through many laps of the ring by now
    assert pool.free_count + int((pool.lens() + bs - 1).__floordiv__(bs).sum()) == num_blocks
