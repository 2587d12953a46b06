"""The batched engine driver's bookkeeping without a GPU (host-simulated arena): Build latches the arena, a step is
planned before it is committed (a step that does not fit changes nothing), tables, lengths and slots of a step are
what the block pool says, and the per-step zero-allocation assertion holds."""
import numpy as np
import pytest

import b200kv


def make(max_step_tokens=8, num_blocks=12, max_blocks_per_seq=4):
    return b200kv.Engine(layers=3, max_seqs=4, num_blocks=num_blocks, block_size=64, max_blocks_per_seq=max_blocks_per_seq,
                         max_step_tokens=max_step_tokens, scale=1.0 / 24.0, backend=b200kv.ARENA_HOST_SIM)


def read_i32(address, count):
    import ctypes

    return np.ctypeslib.as_array(ctypes.cast(address, ctypes.POINTER(ctypes.c_int32)), shape=(count,)).copy()


def test_build_seals_the_arena_and_makes_two_allocations():
    e = make()
    assert e.sealed and e.allocations == 2   # the spans, and the workspace
    c = e.cache
    assert c.geometry.blocks_per_layer == 12 and c.layers == 3 and c.max_blocks_per_seq == 4 and c.seq_lens_handle >= 0
    with pytest.raises(b200kv.B200KVError):
        b200kv.Engine(layers=0, max_seqs=4, num_blocks=12, block_size=64, max_blocks_per_seq=4, max_step_tokens=8,
                      scale=1.0, backend=b200kv.ARENA_HOST_SIM)
    with pytest.raises(b200kv.B200KVError):   # a block of 48 rows is not a multiple of the attention tile
        b200kv.Engine(layers=1, max_seqs=1, num_blocks=2, block_size=48, max_blocks_per_seq=2, max_step_tokens=1,
                      scale=1.0, backend=b200kv.ARENA_HOST_SIM)


def test_steps_upload_what_the_block_pool_says():
    e = make(max_step_tokens=200)
    for s in (0, 2, 3):
        e.admit(s)
    c = e.cache
    # a prefill chunk: 130 tokens of sequence 2, 65 of sequence 0
    e.begin_step([2, 0], [130, 65])
    table = read_i32(e.span_address(c.block_table_handle), 4 * 4).reshape(4, 4)
    lens = read_i32(e.span_address(c.seq_lens_handle), 4)
    slots = read_i32(e.span_address(c.slot_mapping_handle), 200)
    host = e.table()
    assert np.array_equal(table[0], host[2]) and np.array_equal(table[1], host[0])   # rows in step order
    assert lens[0] == 130 and lens[1] == 65
    want = [int(host[2][t // 64]) * 64 + t % 64 for t in range(130)] + [int(host[0][t // 64]) * 64 + t % 64 for t in range(65)]
    assert slots[:195].tolist() == want and (slots[195:] == -1).all()
    with pytest.raises(b200kv.B200KVError):
        e.begin_step([3])            # the previous step has not ended
    with pytest.raises(b200kv.B200KVError):
        e.admit(1)                   # nor can a sequence enter in mid-step
    e.end_step()
    # a decode step: one token each; slots continue where the sequences stand
    e.begin_step([0, 2, 3])
    lens = read_i32(e.span_address(c.seq_lens_handle), 4)
    slots = read_i32(e.span_address(c.slot_mapping_handle), 200)
    host = e.table()
    assert lens[:3].tolist() == [66, 131, 1]
    assert slots[:3].tolist() == [int(host[0][1]) * 64 + 1, int(host[2][2]) * 64 + 2, int(host[3][0]) * 64]
    e.end_step()
    assert '"active_context_tokens": 198' in e.stats_json() and '"total_blocks_allocated": 36' in e.stats_json()
    e.release(2)
    assert '"active_context_tokens": 67' in e.stats_json()


def test_a_step_that_does_not_fit_changes_nothing():
    e = make(max_step_tokens=100, num_blocks=5, max_blocks_per_seq=3)
    e.admit(0)
    e.admit(1)
    e.begin_step([0, 1], [64, 36])
    e.end_step()
    before = (e.seq_len(0), e.seq_len(1), e.table().copy())
    for seqs, grow in (([0, 1], [60, 41]),      # 101 tokens: more than a step holds
                       ([0], [129]),            # 193 tokens need 4 blocks, a table row holds 3
                       ([0, 1], [65, 64]),      # 2 + 1 more blocks, one too many for the 3 that are free ... (5 - 2)
                       ([2], [1]),              # not admitted
                       ([1, 1], [1, 1])):       # twice in one step
        if seqs == [0, 1] and grow == [65, 64]:
            grow = [65, 93]                     # sequence 0 -> 3 blocks (+2), sequence 1 -> 3 blocks (+2): 4 > 3 free
            with pytest.raises(b200kv.B200KVError):
                e.begin_step(seqs, grow)
            continue
        with pytest.raises(b200kv.B200KVError):
            e.begin_step(seqs, grow)
    assert (e.seq_len(0), e.seq_len(1)) == before[:2] and np.array_equal(e.table(), before[2])
    e.begin_step([0, 1])          # and the engine still steps
    e.end_step()
    assert (e.seq_len(0), e.seq_len(1)) == (65, 37)
    with pytest.raises(b200kv.B200KVError):
        e.end_step()              # no step in flight


def snapshot(e):
    return {s: e.seq_len(s) for s in range(4)}, e.table().copy(), e.free_list()


def same(a, b):
    return a[0] == b[0] and np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])


def test_an_abandoned_step_leaves_no_trace():
    """abort_step takes the step's growth back newest first: lengths, table rows and the ORDER of the free list
    are those of before begin_step, however many blocks the step had taken."""
    e = make(max_step_tokens=200)
    for s in (0, 1, 3):
        e.admit(s)
    e.begin_step([1, 0], [70, 10])
    e.end_step()
    before = snapshot(e)
    e.begin_step([3, 0, 1], [130, 60, 1])      # three new blocks for 3, one for 0, none for 1
    assert not same(snapshot(e), before)
    e.abort_step()
    assert same(snapshot(e), before)
    with pytest.raises(b200kv.B200KVError):
        e.abort_step()                          # nothing in flight any more
    e.begin_step([3, 0, 1], [130, 60, 1])      # the same step again takes the same blocks in the same order
    after = snapshot(e)
    e.end_step()
    assert after[0] == {0: 70, 1: 71, 2: -1, 3: 130}


def test_an_injected_upload_failure_is_a_refused_step():
    """The host-side fault hook fails the n-th call of a named entry point before it reaches the device, as the
    reference's FailRuntimeCall does for its stand-in runtime. A step whose upload fails changed nothing."""
    e = make(max_step_tokens=200)
    e.admit(0)
    e.admit(1)
    e.begin_step([0, 1], [65, 3])
    e.end_step()
    before = snapshot(e)
    b200kv.fault_inject("b200kv_engine_step_upload", after_calls=1)
    e.begin_step([0, 1])                        # the first call goes through
    e.end_step()
    mid = snapshot(e)
    with pytest.raises(b200kv.B200KVError) as err:
        e.begin_step([1, 0], [64, 64])          # the second is the injected failure
    assert err.value.code == b200kv.ERR_RUNTIME and "injected failure: b200kv_engine_step_upload" in str(err.value)
    assert same(snapshot(e), mid) and not same(mid, before)
    assert b200kv.fault_clear() == 1            # one failure fired, and the hook disarmed itself
    e.begin_step([1, 0], [64, 64])              # the same step goes through now
    e.end_step()
    with pytest.raises(b200kv.B200KVError):
        b200kv.fault_inject("b200kv_append", -1)
