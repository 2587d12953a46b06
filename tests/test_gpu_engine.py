"""The batched engine driver on the GPU (b200kv_engine_*): eight sequences enter, their prompts are appended in
chunks (chunked prefill-append instead of one single-token step per prompt token, apps/moe_runner.cpp:434-439),
then sixteen decode steps run the reference's stage order per layer (src/pipeline/pipeline.cpp:212-258): producer
(RMSNorm + rotary + paged write), attention, MX quantisation. After every step the pools are compared with the
oracle's bit for bit; attention outputs within the path's tolerance on the oracle's pool; the quantised output bit
for bit with the oracle's quantiser applied to the device's own attention output. A sequence leaves and another
enters half way. No allocation happens after Build."""
import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu


def rope_rows(positions):
    inv = 1.0 / (10000.0 ** (np.arange(32) / 32.0))
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1).astype(np.float32)
    return kvo.f32_to_bf16(cos), kvo.f32_to_bf16(sin)


def test_sixteen_decode_steps_of_eight_sequences_after_chunked_prefill():
    layers, bs, max_seqs, chunk = 3, 64, 9, 256
    num_blocks, max_blocks = 80, 12
    eng = b200kv.Engine(layers=layers, max_seqs=max_seqs, num_blocks=num_blocks, block_size=bs, max_blocks_per_seq=max_blocks,
                        max_step_tokens=2 * chunk, scale=1.0 / 24.0)
    assert eng.sealed and eng.allocations == 2
    allocations = eng.allocations
    torch_bytes = torch.cuda.memory_allocated()
    c = eng.cache
    rows = num_blocks * bs
    latent = b200kv.device_tensor(eng.span_address(c.latent_handle), (layers, rows, 512), torch.bfloat16)
    rope = b200kv.device_tensor(eng.span_address(c.rope_handle), (layers, rows, 64), torch.bfloat16)
    status = eng.status()
    gamma = [kvo.f32_to_bf16(1.0 + 0.1 * kvo.bf16_to_f32(kvo.normal_bf16(512, 7, first=512 * l))) for l in range(layers)]
    d_gamma = [to_dev_bf16(g) for g in gamma]
    oracle_pool = [np.zeros((rows, 576), dtype=np.uint16) for _ in range(layers)]   # the arena starts zero-filled
    counter = [0]

    def fresh(count, stream):
        counter[0] += count
        return kvo.normal_bf16(count, stream, first=counter[0])

    def pools_equal(what):
        torch.cuda.synchronize()
        assert status.cpu().tolist()[0] == 0, status.cpu().tolist()
        for l in range(layers):
            got = np.concatenate([from_dev_bf16(latent[l]), from_dev_bf16(rope[l])], axis=1)
            assert np.array_equal(got, oracle_pool[l]), f"{what}: layer {l} pool differs from the oracle's"

    def slots_of(seqs, grow, lens_before):
        table = eng.table()
        out = []
        for s, n in zip(seqs, grow):
            t = lens_before[s] + np.arange(n)
            out.append(table[s][t // bs].astype(np.int64) * bs + t % bs)
        return np.concatenate(out).astype(np.int32)

    # ---- prompts of different lengths, appended in chunks of at most `chunk` tokens per sequence ----
    prompts = {0: 300, 1: 64, 2: 517, 3: 1, 4: 255, 5: 129, 6: 63, 7: 400}
    for s in prompts:
        eng.admit(s)
    done = {s: 0 for s in prompts}
    while any(done[s] < prompts[s] for s in prompts):
        seqs, grow = [], []
        for s in prompts:   # at most two sequences per prefill step: 2 x chunk tokens
            if done[s] < prompts[s] and len(seqs) < 2:
                seqs.append(s)
                grow.append(min(chunk, prompts[s] - done[s]))
        lens_before = dict(done)
        eng.begin_step(seqs, grow)
        slots = slots_of(seqs, grow, lens_before)
        positions = np.concatenate([lens_before[s] + np.arange(n) for s, n in zip(seqs, grow)])
        cos, sin = rope_rows(positions)
        d_cos, d_sin = to_dev_bf16(cos), to_dev_bf16(sin)
        for l in range(layers):
            kv_a = fresh(len(slots) * 576, 3).reshape(-1, 576)
            eng.layer_append(l, to_dev_bf16(kv_a), d_gamma[l], d_cos, d_sin)
            assert kvo.append_fused(oracle_pool[l], kv_a, gamma[l], cos, sin, slots) == 0
        eng.end_step()
        for s, n in zip(seqs, grow):
            done[s] += n
        with pytest.raises(b200kv.B200KVError):
            eng.layer_attend(0, d_cos, d_cos)   # no step in flight
    pools_equal("after prefill")
    lens = dict(prompts)

    # ---- sixteen decode steps ----
    live = list(prompts)
    for step in range(16):
        if step == 8:   # churn: sequence 2 finishes, sequence 8 enters with a short prompt in one chunk
            eng.release(2)
            live.remove(2)
            lens.pop(2)
            eng.admit(8)
            eng.begin_step([8], [70])
            slots = slots_of([8], [70], {8: 0})
            cos, sin = rope_rows(np.arange(70))
            for l in range(layers):
                kv_a = fresh(70 * 576, 3).reshape(-1, 576)
                eng.layer_append(l, to_dev_bf16(kv_a), d_gamma[l], to_dev_bf16(cos), to_dev_bf16(sin))
                kvo.append_fused(oracle_pool[l], kv_a, gamma[l], cos, sin, slots)
            eng.end_step()
            live.append(8)
            lens[8] = 70
        n = len(live)
        eng.begin_step(live)
        slots = slots_of(live, [1] * n, lens)
        cos, sin = rope_rows([lens[s] for s in live])
        d_cos, d_sin = to_dev_bf16(cos), to_dev_bf16(sin)
        table = eng.table()[live]
        kv_len = np.array([lens[s] + 1 for s in live], dtype=np.int32)
        for l in range(layers):
            kv_a = fresh(n * 576, 3).reshape(n, 576)
            q = kvo.f32_to_bf16(kvo.bf16_to_f32(fresh(n * 64 * 576, 2)) / 24.0).reshape(n, 64, 576)
            d_q = to_dev_bf16(q)
            out = torch.full((n, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
            out8 = torch.zeros((n, 64 * 512), dtype=torch.uint8, device="cuda")
            scales = torch.zeros((n, 64 * 512 // 32), dtype=torch.uint8, device="cuda")
            # the reference's rope stage rotates q's rope slices with k's: the producer does it in place
            eng.layer_append(l, to_dev_bf16(kv_a), d_gamma[l], d_cos, d_sin, q_rope=d_q[:, :, 512:])
            eng.layer_attend(l, d_q, out, out8, scales)
            kvo.append_fused(oracle_pool[l], kv_a, gamma[l], cos, sin, slots)
            q_rot = q.copy()
            q_rot[:, :, 512:] = kvo.rope_half64(q[:, :, 512:], cos, sin)
            torch.cuda.synchronize()
            assert np.array_equal(from_dev_bf16(d_q), q_rot), "q rope slices differ from the oracle's rotation"
            want, _ = kvo.mla_decode(q_rot, oracle_pool[l], table, kv_len, bs, 1.0 / 24.0, use_double=True)
            got = from_dev_bf16(out)
            scenarios.check_attention(got, None, kvo.bf16_to_f32(want).astype(np.float64), None,
                                      what=f"engine step {step} layer {l}")  # short sequences: outputs of magnitude 2
            want8, want_scales = kvo.mx_quant_e4m3(got.reshape(n, -1))
            assert np.array_equal(out8.cpu().numpy(), want8) and np.array_equal(scales.cpu().numpy(), want_scales)
        eng.end_step()
        for s in live:
            lens[s] += 1
        pools_equal(f"decode step {step}")
    assert eng.allocations == allocations and torch.cuda.memory_allocated() >= torch_bytes
    assert f'"active_context_tokens": {sum(lens.values())}' in eng.stats_json()
    del latent, rope, status
    eng.close()


def test_a_failed_launch_in_mid_step_leaves_pool_and_arena_consistent():
    """The attention launch of the second layer of a step fails on the host (injected, before it reaches the
    device: no GPU fault is made). The error comes back as a status, the step is abandoned as a whole
    (lengths, tables and the free list as before it, no allocation made), the GPU context is unharmed, and the
    same step then runs to the oracle's result."""
    layers, bs = 3, 64
    eng = b200kv.Engine(layers=layers, max_seqs=4, num_blocks=24, block_size=bs, max_blocks_per_seq=6, max_step_tokens=192,
                        scale=1.0 / 24.0)
    c = eng.cache
    rows = 24 * bs
    latent = b200kv.device_tensor(eng.span_address(c.latent_handle), (layers, rows, 512), torch.bfloat16)
    rope = b200kv.device_tensor(eng.span_address(c.rope_handle), (layers, rows, 64), torch.bfloat16)
    gamma = kvo.f32_to_bf16(np.ones(512, dtype=np.float32))
    d_gamma = to_dev_bf16(gamma)
    oracle_pool = [np.zeros((rows, 576), dtype=np.uint16) for _ in range(layers)]
    seqs, prompt = [0, 1, 2], [100, 64, 1]
    for s in seqs:
        eng.admit(s)
    eng.begin_step(seqs, prompt)
    table = eng.table()
    slots = np.concatenate([table[s][np.arange(n) // bs].astype(np.int64) * bs + np.arange(n) % bs
                            for s, n in zip(seqs, prompt)]).astype(np.int32)
    cos, sin = rope_rows(np.concatenate([np.arange(n) for n in prompt]))
    for l in range(layers):
        kv_a = kvo.normal_bf16(len(slots) * 576, 3, first=l * 99991).reshape(-1, 576)
        eng.layer_append(l, to_dev_bf16(kv_a), d_gamma, to_dev_bf16(cos), to_dev_bf16(sin))
        kvo.append_fused(oracle_pool[l], kv_a, gamma, cos, sin, slots)
    eng.end_step()
    lens = dict(zip(seqs, prompt))

    def decode_step(fail_layer=None):
        eng.begin_step(seqs)
        table = eng.table()[seqs]
        slots = np.array([int(table[i][lens[s] // bs]) * bs + lens[s] % bs for i, s in enumerate(seqs)], dtype=np.int32)
        cos, sin = rope_rows([lens[s] for s in seqs])
        kv_len = np.array([lens[s] + 1 for s in seqs], dtype=np.int32)
        for l in range(layers):
            kv_a = kvo.normal_bf16(3 * 576, 3, first=7777 + l).reshape(3, 576)
            q = kvo.make_q(3, seed=kvo.BASE_SEED + l)
            out = torch.full((3, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
            eng.layer_append(l, to_dev_bf16(kv_a), d_gamma, to_dev_bf16(cos), to_dev_bf16(sin))
            if fail_layer is None:
                kvo.append_fused(oracle_pool[l], kv_a, gamma, cos, sin, slots)
            eng.layer_attend(l, to_dev_bf16(q), out)      # raises on the injected failure
            if fail_layer is not None:
                continue                                   # (the oracle's pool does not follow an abandoned step)
            want, _ = kvo.mla_decode(q, oracle_pool[l], table, kv_len, bs, 1.0 / 24.0, use_double=True)
            scenarios.check_attention(from_dev_bf16(out), None, kvo.bf16_to_f32(want).astype(np.float64), None,
                                      what=f"after the failed step, layer {l}")
        eng.end_step()

    before = ({s: eng.seq_len(s) for s in seqs}, eng.table().copy(), eng.free_list(), eng.allocations)
    b200kv.fault_inject("b200kv_mla_decode", after_calls=1)   # layer 0 attends, layer 1's launch fails
    with pytest.raises(b200kv.B200KVError) as err:
        decode_step(fail_layer=1)
    assert err.value.code == b200kv.ERR_RUNTIME and "injected failure: b200kv_mla_decode" in str(err.value)
    with pytest.raises(b200kv.B200KVError):
        eng.begin_step(seqs)                                   # the failed step is still in flight
    eng.abort_step()
    torch.cuda.synchronize()
    assert eng.status().cpu().tolist()[0] == 0
    after = ({s: eng.seq_len(s) for s in seqs}, eng.table().copy(), eng.free_list(), eng.allocations)
    assert before[0] == after[0] and np.array_equal(before[1], after[1]) and np.array_equal(before[2], after[2])
    assert before[3] == after[3] and b200kv.fault_clear() == 1
    decode_step()                                              # the same step, now to the end
    for s in seqs:
        lens[s] += 1
    for l in range(layers):
        got = np.concatenate([from_dev_bf16(latent[l]), from_dev_bf16(rope[l])], axis=1)
        live = np.zeros(rows, dtype=bool)
        for s in seqs:
            t = np.arange(lens[s])
            live[eng.table()[s][t // bs].astype(np.int64) * bs + t % bs] = True
        assert np.array_equal(got[live], oracle_pool[l][live]), f"layer {l}: live rows differ from the oracle's"
    del latent, rope
    eng.close()
