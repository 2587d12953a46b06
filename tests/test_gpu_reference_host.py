"""The reference engine's own host code for the KV path (OpTable, PlanAclnnOp, StaticOpSlot, AclDeviceOps:
src/core/op_table.cpp, src/core/device_ops.cpp), compiled from the reference tree into oracle/_ref/op_slot_probe
and linked against this repository's library, runs one decode step over three layers: plan once, repoint the
caches per layer, launch the cache write and the attention. Its outputs are held against the oracle: the
appended rows bit for bit, the attention within the path's tolerance. Skipped where the probe was not built
(it needs the reference tree at build time; the built binary travels with the repository)."""
import os
import struct
import subprocess

import numpy as np
import pytest

import kvo
import scenarios

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROBE = os.path.join(ROOT, "oracle", "_ref", "op_slot_probe")
OPERATORS = 27  # operators the reference's table resolves by name, the KV path's two included


@pytest.mark.skipif(not os.path.exists(PROBE), reason="oracle/_ref/op_slot_probe not built (needs the reference tree)")
@pytest.mark.parametrize("block_size,context,scale", [(128, 385, 1.0 / np.sqrt(192.0)), (64, 129, 1.0 / 24.0)])
def test_reference_op_slots_drive_the_library(tmp_path, block_size, context, scale):
    layers, heads = 3, 64
    blocks = scenarios.blocks_for(context, block_size) + 1
    rows = blocks * block_size
    table = np.arange(blocks, dtype=np.int32)[::-1].copy()  # reversed, so the table is really consulted
    slot_row = int(table[(context - 1) // block_size]) * block_size + (context - 1) % block_size
    f_in, f_out = tmp_path / "in.bin", tmp_path / "out.bin"
    per_layer = []
    with open(f_in, "wb") as f:
        scale_bits = struct.unpack("<I", struct.pack("<f", float(scale)))[0]
        f.write(np.array([layers, blocks, block_size, context, heads, scale_bits, slot_row], dtype=np.int64).tobytes())
        for layer in range(layers):
            pool = kvo.make_pool(rows, seed=kvo.BASE_SEED + layer)          # uint16 [rows, 576]
            new = kvo.normal_bf16(576, 3, first=layer * 576)                # the row the step appends
            q = kvo.make_q(1, heads, scale=1.0, seed=kvo.BASE_SEED + 100 + layer)[0]  # [heads, 576]
            per_layer.append((pool, new, q))
            f.write(np.ascontiguousarray(pool[:, :512]).tobytes())
            f.write(np.ascontiguousarray(pool[:, 512:]).tobytes())
            f.write(new[:512].tobytes())
            f.write(new[512:].tobytes())
            f.write(np.ascontiguousarray(q[:, :512]).tobytes())
            f.write(np.ascontiguousarray(q[:, 512:]).tobytes())
        f.write(table.tobytes())

    # The engine's batch-1 loop uses slot = position (src/pipeline/pipeline.cpp:515-519), right for an identity
    # table; here the slot is the row the reversed table maps that position to.
    done = subprocess.run([PROBE, str(f_in), str(f_out)], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    raw = open(f_out, "rb").read()
    n_out, n_row = heads * 512 * 2, 576 * 2
    outs = [np.frombuffer(raw, dtype=np.uint16, count=heads * 512, offset=l * n_out).reshape(heads, 512) for l in range(layers)]
    rows_back = [np.frombuffer(raw, dtype=np.uint16, count=576, offset=layers * n_out + l * n_row) for l in range(layers)]
    inventory = raw[layers * (n_out + n_row):].decode()
    assert inventory.count(" found ") >= OPERATORS and "MISSING" not in inventory, inventory

    for layer, (pool, new, q) in enumerate(per_layer):
        # bit-exact append at the engine's slot
        assert np.array_equal(rows_back[layer], new), f"layer {layer}: appended row differs"
        expect_pool = pool.copy()
        expect_pool[slot_row] = new
        ref_out, ref_lse = scenarios.ref_attention_f64(q[None], expect_pool, table[None], np.array([context], dtype=np.int32),
                                                       block_size, float(scale))
        scenarios.check_attention(outs[layer][None], None, ref_out, ref_lse, what=f"reference host, layer {layer}")
