"""Pins the oracle (and the product's reservation arithmetic) to the structural known-answers the
reference holds for this path. The reference has no numeric vector for append / gather / attention
(its operator launches are no-ops), so these are the only pins it offers; they are stored with their
citations in tests/golden/reference_structural.json."""
import json
import os

import numpy as np

import kvo

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_structural.json")


def _facts():
    with open(GOLDEN) as f:
        return json.load(f)


def test_block_counts_match_reference():
    for case in _facts()["block_counts"]:
        got = kvo.lib().kvo_total_blocks(case["max_context"], case["block_size"], case["layers"])
        assert got == case["total_blocks"], case


def test_utilisation_matches_reference():
    for case in _facts()["utilisation"]:
        got = kvo.lib().kvo_utilisation(case["position"], case["max_context"], case["block_size"])
        assert got == case["value"], case


def test_pool_bytes_match_reference_ledger():
    for case in _facts()["pool_bytes"]:
        lat = np.zeros(1, dtype=np.int64)
        rope = np.zeros(1, dtype=np.int64)
        kvo.lib().kvo_pool_bytes(case["max_context"], case["block_size"], case["layers"], 512, 64, lat.ctypes.data,
                                 rope.ctypes.data)
        assert int(lat[0]) == case["latent_bytes"] and int(rope[0]) == case["rope_bytes"], case


def test_product_reservation_agrees_with_oracle_and_reference():
    import b200kv

    facts = _facts()
    for case in facts["block_counts"]:
        r = b200kv.plan_reservation(case["max_context"], case["block_size"], case["layers"])
        assert r.total_blocks == case["total_blocks"]
        assert r.blocks_per_layer == kvo.lib().kvo_blocks_per_layer(case["max_context"], case["block_size"])
    for case in facts["pool_bytes"]:
        r = b200kv.plan_reservation(case["max_context"], case["block_size"], case["layers"])
        assert (r.latent_bytes, r.rope_bytes) == (case["latent_bytes"], case["rope_bytes"])
        # block table [1][blocks] int32 and one int32 slot per step, as the reference reserves them
        assert r.block_table_bytes == 4 * r.blocks_per_layer and r.slot_mapping_bytes == 4
    for case in facts["utilisation"]:
        blocks = kvo.lib().kvo_blocks_per_layer(case["max_context"], case["block_size"])
        assert b200kv.utilisation(case["position"] + 1, blocks, case["block_size"]) == case["value"]


def test_generator_is_counter_based_and_stable():
    a = kvo.normal_bf16(1000, kvo.STREAM_KV)
    b = kvo.normal_bf16(500, kvo.STREAM_KV, first=500)
    assert (a[500:] == b).all()
    c = kvo.normal_bf16(7, kvo.STREAM_KV, first=3)
    assert (a[3:10] == c).all()
    # known-answer: the first values of the KV stream at the base seed never change
    with open(os.path.join(os.path.dirname(__file__), "golden", "generator_kat.json")) as f:
        kat = json.load(f)
    assert [int(v) for v in a[:16]] == kat["kv_stream_first16_bf16_bits"]
    assert [int(v) for v in kvo.permutation(16)] == kat["perm16"]
    x = kvo.bf16_to_f32(kvo.normal_bf16(1 << 20, kvo.STREAM_Q))
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 1.0) < 5e-3


def test_bf16_round_to_nearest_even():
    vals = np.array([1.0, 1.00390625, 1.005859375, 1.001953125, -2.5, 3.3895313892515355e38, 0.0], dtype=np.float32)
    bits = kvo.f32_to_bf16(vals)
    # 1.00390625 = 1 + 2^-8 is a tie between 0x3F80 and 0x3F81 -> even (0x3F80); 1.005859375 = 1 + 1.5*2^-8 -> 0x3F81
    assert [int(b) for b in bits[:5]] == [0x3F80, 0x3F80, 0x3F81, 0x3F80, 0xC020]
    assert int(bits[5]) == 0x7F7F and int(bits[6]) == 0
    assert np.isnan(kvo.bf16_to_f32(kvo.f32_to_bf16(np.array([np.nan], dtype=np.float32)))).all()


def test_paged_attention_stats_json_has_the_reference_shape():
    """The diagnostics object the reference writes (src/diagnostics/inference_stats.cpp:42-47): same keys, same
    number formatting, and the two structural known answers of its tests and examples (2,752 blocks at context
    8192 / block 128, docs/examples/inference_diagnostics_dry_run.json:20-24; utilisation (128 + 1) / 8192 after
    a 128-token prompt and one decoded token, tests/mock_pipeline_e2e.cpp:663-666)."""
    import ctypes
    import json

    import b200kv

    fn = b200kv.lib.b200kv_paged_attention_stats_json
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_char_p, ctypes.c_int64]
    buf = ctypes.create_string_buffer(512)
    n = fn(64, 43, 0, 128, buf, 512)
    text = buf.value.decode()
    assert n == len(text)
    assert text == ('"paged_attention": {\n    "total_blocks_allocated": 2752,\n    "active_context_tokens": 0,\n'
                    '    "block_size": 128,\n    "kv_cache_utilization": 0\n  }')
    fn(64, 43, 129, 128, buf, 512)
    obj = json.loads("{" + buf.value.decode() + "}")["paged_attention"]
    assert obj == {"total_blocks_allocated": 2752, "active_context_tokens": 129, "block_size": 128,
                   "kv_cache_utilization": 0.0157470703125}
    assert fn(64, 43, 129, 128, None, 0) == len(buf.value)   # sizing call
    small = ctypes.create_string_buffer(16)
    assert fn(64, 43, 129, 128, small, 16) == len(buf.value) and len(small.value) == 15
