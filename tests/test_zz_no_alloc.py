"""b200kv_mla_decode_static, the decode entry point for hosts that may not allocate device memory (a
serving loop whose arena is sealed, a plugin living inside another runtime's memory budget): it must
give what b200kv_mla_decode gives, call after call, using only the scratch array built into the
library. Collected last on purpose, so a run that stops at the first failure has seen every other test."""
import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

pytestmark = pytest.mark.gpu


def _case(shift):
    bs = 64
    kv_len = np.array([4097, 1000, 0, 65, 2300, 64, 1, 700], dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 5
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = kvo.normal_bf16(blocks * bs * kvo.ROW, kvo.STREAM_KV, first=shift).reshape(blocks * bs, kvo.ROW)
    q = kvo.normal_bf16(len(kv_len) * 64 * kvo.ROW, kvo.STREAM_Q, first=shift, scale=2.0 / 24.0)
    return bs, kv_len, table, pool, q.reshape(len(kv_len), 64, kvo.ROW)


def test_static_scratch_entry_matches_workspace_entry_on_two_calls_in_a_row():
    assert b200kv.lib.b200kv_mla_decode_static_scratch_bytes is not None
    for call in range(2):  # the second call reuses the scratch the first one left behind
        bs, kv_len, table, pool_np, q_np = _case(shift=call * 7919)
        B = len(kv_len)
        pool, q = to_dev_bf16(pool_np), to_dev_bf16(q_np)
        view = b200kv.pool_view(pool)
        tbl, lens = to_dev_i32(table), to_dev_i32(kv_len)
        status = b200kv.new_status()

        want = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        want_lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
        ws = torch.empty(b200kv.decode_workspace_bytes(B), dtype=torch.uint8, device="cuda")
        b200kv.mla_decode(q, view, tbl, lens, bs, 1.0 / 24.0, out=want, lse=want_lse, workspace=ws,
                          variant=b200kv.DECODE_TCGEN05, status=status)

        got = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        got_lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
        b200kv.mla_decode_static(q, view, tbl, lens, bs, 1.0 / 24.0, out=got, lse=got_lse, status=status)
        status_ok(status)

        ref = kvo.bf16_to_f32(from_dev_bf16(want)).astype(np.float64)
        scenarios.check_attention(from_dev_bf16(got), got_lse.cpu().numpy(), ref,
                                  want_lse.cpu().numpy().astype(np.float64), what=f"static scratch, call {call}")
        # and both agree with the oracle, so the comparison above is not two wrongs
        o_out, o_lse = kvo.mla_decode(q_np, pool_np, table, kv_len, bs, 1.0 / 24.0, use_double=True)
        scenarios.check_attention(from_dev_bf16(got), got_lse.cpu().numpy(),
                                  kvo.bf16_to_f32(o_out).astype(np.float64), o_lse.astype(np.float64),
                                  what=f"static scratch vs oracle, call {call}")


def test_static_scratch_entry_refuses_grids_beyond_its_array():
    bs, kv_len, table, pool_np, q_np = _case(shift=0)
    pool, q = to_dev_bf16(pool_np), to_dev_bf16(q_np)
    out = torch.zeros((len(kv_len), 64, 512), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(b200kv.B200KVError) as err:
        b200kv.mla_decode_static(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0,
                                 out=out, max_ctas=33)
    assert err.value.code == b200kv.ERR_INVALID and "at most 32" in str(err.value)
    assert b200kv.lib.b200kv_mla_decode_static_scratch_bytes() == 32 * 2 * 64 * 514 * 4



def test_static_scratch_entry_refuses_what_the_workspace_entry_refuses():
    """Both entry points share their argument checks: a query whose head stride is shorter than a row (8
    elements: a multiple of 8, so the tensor-core kernel's own alignment rule alone would let it through) is
    refused as invalid before anything is launched."""
    bs, kv_len, table, pool_np, q_np = _case(shift=0)
    pool, q = to_dev_bf16(pool_np), to_dev_bf16(q_np)
    out = torch.zeros((len(kv_len), 64, 512), dtype=torch.bfloat16, device="cuda")
    narrow = q.as_strided((len(kv_len), 64, kvo.ROW), (64 * kvo.ROW, 8, 1))
    for call in (b200kv.mla_decode_static,
                 lambda *a, **k: b200kv.mla_decode(*a, workspace=torch.empty(
                     b200kv.decode_workspace_bytes(len(kv_len)), dtype=torch.uint8, device="cuda"), **k)):
        with pytest.raises(b200kv.B200KVError) as err:
            call(narrow, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out)
        assert err.value.code == b200kv.ERR_INVALID
