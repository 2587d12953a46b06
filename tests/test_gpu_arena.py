"""The path on the pool the engine would give it: ONE device allocation made by the static arena's Commit, the KV
spans carved from it under the reference's names (src/memory/static_arena.cpp:108-118,
src/memory/static_arena_manager.cpp:298-300, 315-318), a per-layer view by base + layer * bytes
(src/pipeline/pipeline.cpp:390-400), the workspace from NoteWorkspace / CommitWorkspace, and the latch. Append,
gather and attention run on those addresses and are held against the oracle."""
import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, status_ok, to_dev_bf16

pytestmark = pytest.mark.gpu


def _fill_from(tensor, values_u16):
    tensor.view(torch.int16).copy_(torch.from_numpy(np.ascontiguousarray(values_u16).view(np.int16)).cuda())


@pytest.mark.parametrize("fused", [False, True])
def test_append_and_attention_on_the_arena_carved_cache(fused):
    bs, B, ctx, layers = 64, 32, 4096, 3   # configs[1]'s geometry, three of its 43 layers
    blocks_per_seq = ctx // bs
    num_blocks = B * blocks_per_seq
    arena = b200kv.Arena(b200kv.ARENA_DEVICE)
    cache = arena.reserve_kv_cache_batched(num_blocks, bs, layers, max_seqs=B, max_blocks_per_seq=blocks_per_seq,
                                           tokens_per_step=B)
    h_q = arena.reserve("attn.q", layers * B * 64 * kvo.ROW * 2)
    h_new = arena.reserve("attn.new_rows", layers * B * kvo.ROW * 2)
    h_out = arena.reserve("attn.out", layers * B * 64 * 512 * 2)
    h_status = arena.reserve("attn.status", 16)
    arena.note_workspace(b200kv.decode_workspace_bytes(B))
    with pytest.raises(b200kv.B200KVError):
        arena.layer_view(cache, 0)   # no address before Commit
    before = torch.cuda.memory_allocated()
    arena.commit()
    assert arena.allocations == 1
    arena.commit_workspace()
    assert arena.allocations == 2 and arena.workspace_bytes >= b200kv.decode_workspace_bytes(B)
    arena.workspace_fits(b200kv.decode_workspace_bytes(B))
    arena.seal()
    assert torch.cuda.memory_allocated() == before   # the arena is the library's own allocation, not torch's
    with pytest.raises(b200kv.B200KVError):
        arena.reserve("late", 8)
    with pytest.raises(b200kv.B200KVError):
        arena.reserve_kv_cache_batched(1, bs, 1, 1, 1, 1)
    arena.validate()

    table_d = arena.tensor(cache.block_table_handle, (B, blocks_per_seq), torch.int32)
    slots_d = arena.tensor(cache.slot_mapping_handle, (B,), torch.int32)
    lens_d = arena.tensor(cache.seq_lens_handle, (B,), torch.int32)
    latent_d = arena.tensor(cache.latent_handle, (layers, num_blocks * bs, 512), torch.bfloat16)
    rope_d = arena.tensor(cache.rope_handle, (layers, num_blocks * bs, 64), torch.bfloat16)
    q_d = arena.tensor(h_q, (layers, B, 64, kvo.ROW), torch.bfloat16)
    new_d = arena.tensor(h_new, (layers, B, kvo.ROW), torch.bfloat16)
    out_d = arena.tensor(h_out, (layers, B, 64, 512), torch.bfloat16)
    status = arena.tensor(h_status, (4,), torch.int32)
    ws = b200kv.device_tensor(arena.workspace, (arena.workspace_bytes,), torch.uint8)
    # Commit zero-fills: an unwritten block must read as zeros, not as stale memory
    assert int(latent_d[layers - 1, -bs:].view(torch.int16).abs().max()) == 0 and int(table_d.abs().max()) == 0
    assert int(ws[:4096].max()) == 0

    table = kvo.permutation(num_blocks).reshape(B, blocks_per_seq)
    kv_len = np.full(B, ctx, dtype=np.int32)
    slots = (table[:, -1].astype(np.int64) * bs + (ctx - 1) % bs).astype(np.int32)
    table_d.copy_(torch.from_numpy(table).cuda())
    lens_d.copy_(torch.from_numpy(kv_len).cuda())
    slots_d.copy_(torch.from_numpy(slots).cuda())
    pools, qs, news = [], [], []
    for layer in range(layers):
        pool = kvo.make_pool(num_blocks * bs, seed=kvo.BASE_SEED + layer)
        q = kvo.make_q(B, seed=kvo.BASE_SEED + 50 + layer)
        new = kvo.normal_bf16(B * kvo.ROW, kvo.STREAM_NEW, first=layer * B * kvo.ROW).reshape(B, kvo.ROW)
        _fill_from(latent_d[layer], pool[:, :512])
        _fill_from(rope_d[layer], pool[:, 512:])
        _fill_from(q_d[layer], q)
        _fill_from(new_d[layer], new)
        pools.append(pool), qs.append(q), news.append(new)

    for layer in range(layers):
        view = arena.layer_view(cache, layer)
        assert view.latent == latent_d[layer].data_ptr() and view.rope == rope_d[layer].data_ptr()
        new_lat, new_rope = new_d[layer][:, :512], new_d[layer][:, 512:]
        if not fused:
            b200kv.append(view, new_lat, new_rope, slots_d, status=status)
        b200kv.mla_decode(q_d[layer], view, table_d, lens_d, bs, 1.0 / 24.0, out=out_d[layer], workspace=ws,
                          status=status, stable_tables=True, new_rows=(new_lat, new_rope) if fused else None)
    status_ok(status)

    for layer in (0, layers - 1):
        want_pool = pools[layer].copy()
        assert kvo.append(want_pool, np.ascontiguousarray(news[layer][:, :512]),
                          np.ascontiguousarray(news[layer][:, 512:]), slots) == 0
        got = np.concatenate([from_dev_bf16(latent_d[layer]), from_dev_bf16(rope_d[layer])], axis=1)
        assert np.array_equal(got, want_pool), f"layer {layer}: arena pool differs from the oracle's append"
        want, _ = kvo.mla_decode(qs[layer], want_pool, table, kv_len, bs, 1.0 / 24.0, use_double=True)
        scenarios.check_attention(from_dev_bf16(out_d[layer]), None, kvo.bf16_to_f32(want).astype(np.float64), None,
                                  what=f"arena-carved cache, layer {layer}, fused={fused}", strict_abs=True,
                                  elementwise=True)
    # gather reads the same spans through the same table
    total = int(kv_len[:2].sum())
    out_l = torch.empty((total, 512), dtype=torch.bfloat16, device="cuda")
    out_r = torch.empty((total, 64), dtype=torch.bfloat16, device="cuda")
    offsets = torch.tensor([0, ctx], dtype=torch.int64, device="cuda")
    b200kv.gather(arena.layer_view(cache, 1), table_d[:2], lens_d[:2], bs, out_l, out_r, offsets, total, status=status)
    status_ok(status)
    want_pool = pools[1].copy()
    kvo.append(want_pool, np.ascontiguousarray(news[1][:, :512]), np.ascontiguousarray(news[1][:, 512:]), slots)
    want_l, want_r, _ = kvo.gather(want_pool, table[:2], kv_len[:2], bs)
    assert np.array_equal(from_dev_bf16(out_l), want_l) and np.array_equal(from_dev_bf16(out_r), want_r)
    del table_d, slots_d, lens_d, latent_d, rope_d, q_d, new_d, out_d, status, ws
    torch.cuda.synchronize()
    arena.close()
