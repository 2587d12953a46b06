"""Regenerates the golden fixtures in this folder.

    python tests/golden/make_golden.py

generator_kat.json    first values of the seeded generator (pins the input streams).
attention_small.npz   float64-accurate attention outputs (stored fp32) for small seeded cases, computed by
                      the independent numpy restatement in tests/scenarios.py, NOT by the oracle; the oracle
                      and the CUDA kernels are both checked against it.
The reference tree holds no numeric vectors for this path (its operator launches are no-ops), so these
fixtures pin this repository's own definitions; reference_structural.json holds what the reference does pin.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import kvo  # noqa: E402
import scenarios  # noqa: E402

CASES = {
    # name: (kv_len list, block_size, scale, q_scale, num_blocks)
    "cfg1_bs64": ([129], 64, 1.0 / 24.0, 1.0 / 24.0, 8),
    "cfg1_ref_defaults_bs128": ([129], 128, 1.0 / np.sqrt(192.0), 1.0 / 24.0, 4),
    "ragged_bs64": ([1, 63, 64, 65, 200], 64, 1.0 / 24.0, 1.0 / 24.0, 16),
    "sharp_softmax_bs64": ([300], 64, 1.0 / 24.0, 64.0 / 24.0, 8),
}


def case_inputs(name):
    kv_len, bs, scale, q_scale, num_blocks = CASES[name]
    pool = kvo.make_pool(num_blocks * bs)
    q = kvo.make_q(len(kv_len), scale=q_scale)
    table = scenarios.build_tables(kv_len, bs, num_blocks)
    return q, pool, table, np.asarray(kv_len, dtype=np.int32), bs, float(scale)


def main():
    a = kvo.normal_bf16(16, kvo.STREAM_KV)
    with open(os.path.join(HERE, "generator_kat.json"), "w") as f:
        json.dump({"_about": "Known answers of the seeded generator (base seed 20251008): regenerate with "
                             "tests/golden/make_golden.py",
                   "kv_stream_first16_bf16_bits": [int(v) for v in a],
                   "perm16": [int(v) for v in kvo.permutation(16)]}, f, indent=1)
    out = {}
    for name in CASES:
        q, pool, table, kv_len, bs, scale = case_inputs(name)
        ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, scale)
        out[name + "/out"] = ref_out.astype(np.float32)
        out[name + "/lse"] = ref_lse.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **out)
    print("wrote", sorted(out))


if __name__ == "__main__":
    main()
