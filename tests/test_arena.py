"""The KV arena against the reference's own StaticMemoryArena, run through oracle/_ref/arena_probe (the
reference's sources compiled where they lie), and against the reference's arena test script
(tests/mock_contract_smoke.cpp:533-584 of the reference). CPU only: the arena's host-simulated backend."""
import ctypes
import os
import subprocess

import pytest

import b200kv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROBE = os.path.join(ROOT, "oracle", "_ref", "arena_probe")


def drive_reference(script):
    """Runs the command script through the reference arena; returns the per-line answers."""
    res = subprocess.run([PROBE], input="\n".join(script) + "\n", capture_output=True, text=True, check=True)
    return [line.split() for line in res.stdout.strip().splitlines()]


def drive_product(script):
    arena = b200kv.Arena(b200kv.ARENA_HOST_SIM)
    out = []
    for line in script:
        cmd, *args = line.split()
        try:
            if cmd == "reserve":
                handle = arena.reserve(args[0], int(args[1]), int(args[2]))
                out.append(["ok", str(handle), str(arena.offset(handle)), str(arena.reserved_bytes)])
            elif cmd == "commit":
                arena.commit()
                base = arena.address(0)
                raw = (ctypes.c_ubyte * arena.nbytes).from_address(base)
                zero = not any(raw)
                out.append(["ok", str(arena.nbytes), str(arena.allocations), "1" if zero else "0"])
            elif cmd == "address":
                out.append(["ok", str(arena.address(int(args[0])) - arena.address(0))])
            elif cmd == "note":
                arena.note_workspace(int(args[0]))
                out.append(["ok"])
            elif cmd == "commit_workspace":
                arena.commit_workspace()
                out.append(["ok", str(arena.workspace_bytes), str(arena.allocations)])
            elif cmd == "fits":
                arena.workspace_fits(int(args[0]))
                out.append(["ok"])
            elif cmd == "seal":
                arena.seal()
                out.append(["ok", "1" if arena.sealed else "0"])
            elif cmd == "validate":
                arena.validate()
                out.append(["ok"])
            else:
                out.append(["unknown"])
        except b200kv.B200KVError:
            out.append(["refused"])
    return out


# The reference's own arena test, as a script (tests/mock_contract_smoke.cpp:548-583).
REFERENCE_TEST_SCRIPT = [
    "reserve a.small 100 512", "reserve b.aligned 4096 4096", "reserve c.tail 7 512",
    "address 0",                    # refused: no address before Commit
    "reserve d.zero 0 512",         # refused: empty
    "reserve e.odd-align 64 3",     # refused: alignment not a power of two
    "commit", "address 1", "address 2", "validate",
    "reserve f.late 8 512",         # refused: after Commit
    "note 1024", "note 4096", "note 2048", "commit_workspace",
    "fits 4096",
    "fits 4097",                    # refused: would grow
    "seal",
    "reserve g.sealed 8 512", "commit_workspace",   # refused: sealed
]

EXPECTED_FROM_REFERENCE_TEST = {
    6: ["ok", "8704", "1", "1"],    # ONE allocation, zero-filled
    7: ["ok", "4096"],              # the 4096-aligned reservation got its alignment
    14: ["ok", "4096", "2"],        # workspace = high-water mark; second and last allocation
}


def test_product_passes_the_reference_arena_test():
    got = drive_product(REFERENCE_TEST_SCRIPT)
    refused = {3, 4, 5, 10, 16, 18, 19}
    for i, ans in enumerate(got):
        assert (ans[0] == "refused") == (i in refused), (i, REFERENCE_TEST_SCRIPT[i], ans)
    for i, want in EXPECTED_FROM_REFERENCE_TEST.items():
        assert got[i] == want, (i, got[i], want)


@pytest.mark.skipif(not os.path.exists(PROBE), reason="oracle/_ref/arena_probe not built (needs the reference tree)")
def test_product_matches_reference_arena_line_by_line():
    assert drive_product(REFERENCE_TEST_SCRIPT) == drive_reference(REFERENCE_TEST_SCRIPT)
    # the KV reservation of the reference defaults and of the B=32 x 4K configuration, span by span
    for ctx, bs, seqs in [(8192, 128, 1), (256, 128, 1), (4096, 64, 32)]:
        r = b200kv.plan_reservation(ctx, bs, 43, seqs, seqs)
        script = [
            "reserve act.some_activation 12345 512",
            f"reserve kv.block_table {r.block_table_bytes} 512",
            f"reserve kv.slot_mapping {r.slot_mapping_bytes} 512",
            "reserve w.rope_sin 1048576 512",
            f"reserve kv.latent_cache {r.latent_bytes} 512",
            f"reserve kv.rope_cache {r.rope_bytes} 512",
            "reserve w.tail 3 512",
        ]
        # offsets only: committing would really allocate the pool
        assert drive_product(script) == drive_reference(script)


def test_kv_cache_reservation_and_layer_views():
    arena = b200kv.Arena(b200kv.ARENA_HOST_SIM)
    cache = arena.reserve_kv_cache(max_context=256, block_size=128, layers=43, max_seqs=1)
    assert cache.geometry.total_blocks == 86          # tests/mock_pipeline_e2e.cpp:615-618 of the reference
    assert cache.geometry.latent_bytes == 43 * 256 * 512 * 2 and cache.geometry.rope_bytes == 43 * 256 * 64 * 2
    with pytest.raises(b200kv.B200KVError):
        arena.layer_view(cache, 0)                    # no address before Commit
    arena.commit()
    assert arena.allocations == 1
    arena.seal()
    with pytest.raises(b200kv.B200KVError):
        arena.reserve("late", 8)
    lat0, rope0 = arena.address(cache.latent_handle), arena.address(cache.rope_handle)
    for layer in (0, 1, 42):
        view = arena.layer_view(cache, layer)
        # per-layer base = span + layer * blocks * block_size * width * 2 (src/pipeline/pipeline.cpp:391-395)
        assert view.latent == lat0 + layer * 2 * 128 * 512 * 2
        assert view.rope == rope0 + layer * 2 * 128 * 64 * 2
        assert (view.latent_row_stride, view.rope_row_stride, view.pool_rows) == (512, 64, 256)
        assert view.latent % 512 == 0 and view.rope % 512 == 0
    with pytest.raises(b200kv.B200KVError):
        arena.layer_view(cache, 43)
    with pytest.raises(b200kv.B200KVError):
        b200kv.Arena(b200kv.ARENA_HOST_SIM).reserve_kv_cache(max_context=64, block_size=128)  # below one block


def test_batched_kv_cache_reservation_host_sim():
    """The batched form: a pool shared by many sequences, a table per sequence, the step's slots and the lengths,
    under the reference's span names and in its order, all in one allocation."""
    arena = b200kv.Arena(b200kv.ARENA_HOST_SIM)
    cache = arena.reserve_kv_cache_batched(num_blocks=40, block_size=64, layers=3, max_seqs=5, max_blocks_per_seq=12,
                                           tokens_per_step=256)
    g = cache.geometry
    assert (g.blocks_per_layer, g.total_blocks) == (40, 120)
    assert g.latent_bytes == 3 * 40 * 64 * 512 * 2 and g.rope_bytes == 3 * 40 * 64 * 64 * 2
    assert g.block_table_bytes == 5 * 12 * 4 and g.slot_mapping_bytes == 256 * 4
    assert cache.max_blocks_per_seq == 12 and cache.seq_lens_handle >= 0
    handles = [cache.block_table_handle, cache.slot_mapping_handle, cache.seq_lens_handle, cache.latent_handle,
               cache.rope_handle]
    offsets = [arena.offset(h) for h in handles]
    assert offsets == sorted(offsets) and all(o % 512 == 0 for o in offsets)
    arena.commit()
    assert arena.allocations == 1
    view = arena.layer_view(cache, 2)
    assert view.pool_rows == 40 * 64 and view.latent == arena.address(cache.latent_handle) + 2 * 40 * 64 * 512 * 2
    with pytest.raises(b200kv.B200KVError):
        b200kv.Arena(b200kv.ARENA_HOST_SIM).reserve_kv_cache_batched(0, 64, 1, 1, 1, 1)
