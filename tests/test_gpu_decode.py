"""Decode attention on the device (both kernels) against the oracle and the golden vectors, within the
path's tolerance as scenarios.check_attention states it: on benchmark-distributed inputs every element within
2e-3 absolute (which implies |err| <= 2e-3 + 1e-2*|ref|); on the adversarial inputs (large logits, rows that
hold big values beside cancelling ones) |err| <= 2e-3 + 1e-2*max_row|ref|, with the per-element form measured
and reported for each comparison; lse within 1e-3. All calls go through the C ABI."""
import os
import sys

import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import run_decode

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))
VARIANTS = [pytest.param(b200kv.DECODE_SIMT, id="simt"), pytest.param(b200kv.DECODE_TCGEN05, id="tcgen05")]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_decode_matches_golden(name, variant):
    q, pool, table, kv_len, bs, scale = make_golden.case_inputs(name)
    out, lse = run_decode(q, pool, table, kv_len, bs, scale, variant)
    scenarios.check_attention(out, lse, GOLDEN[name + "/out"].astype(np.float64),
                              GOLDEN[name + "/lse"].astype(np.float64), what=name,
                              strict_abs=not name.startswith("sharp"))


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_matches_oracle_batched_permuted(variant):
    """Four sequences of the B=32 x 4K configuration (context 4097 after the append), permuted tables."""
    bs, B, n = 64, 4, 4097
    blocks = B * scenarios.blocks_for(n, bs) + 7
    kv_len = np.full(B, n, dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(B)
    want, want_lse = kvo.mla_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, use_double=True)
    out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, variant)
    scenarios.check_attention(out, lse, kvo.bf16_to_f32(want).astype(np.float64), want_lse.astype(np.float64),
                              abs_tol=2e-3, what="batched", strict_abs=True)


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_ragged_fragmented_with_empty_and_tiny_sequences(variant):
    bs = 64
    kv_len = np.array([0, 1, 31, 32, 33, 64, 65, 127, 128, 129, 1000, 2, 0, 517], dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 9
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    # unowned blocks and the tails of last blocks hold NaN: they must never reach a result
    owned = np.zeros(blocks * bs, dtype=bool)
    for b, n in enumerate(kv_len):
        j = np.arange(int(n))
        owned[table[b, j // bs].astype(np.int64) * bs + j % bs] = True
    pool[~owned] = 0x7FC1
    q = kvo.make_q(len(kv_len), scale=4.0 / 24.0)
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, 1.0 / 24.0)
    for max_ctas in (0, 3, 1):
        out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, variant, max_ctas=max_ctas)
        scenarios.check_attention(out, lse, ref_out, ref_lse, what=f"ragged max_ctas={max_ctas}")
        assert (out[kv_len == 0] == 0).all()


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_online_softmax_stress(variant):
    """A late dominant key (forces the running maximum to jump), large logits, and a one-token tail tile."""
    bs, n = 64, 961  # 15 blocks + 1 token
    blocks = 20
    kv_len = np.array([n], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(1, scale=16.0 / 24.0)
    # make the last token nearly parallel to head 0's query, scaled up: its logit dwarfs the rest
    qf = kvo.bf16_to_f32(q)[0, 0]
    row = int(table[0, (n - 1) // bs]) * bs + (n - 1) % bs
    pool[row] = kvo.f32_to_bf16((qf * 3.0).astype(np.float32))
    mid = int(table[0, 5]) * bs + 17
    pool[mid] = kvo.f32_to_bf16((kvo.bf16_to_f32(q)[0, 1] * 2.0).astype(np.float32))
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, 1.0 / 24.0)
    out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, variant)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what="stress")


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_reference_layout_two_caches_bs128(variant):
    """The reference's own geometry: separate latent [rows,512] and rope [rows,64] caches, block 128,
    scale 1/sqrt(192)."""
    bs, n, blocks = 128, 700, 8
    kv_len = np.array([n, 129], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    fused = kvo.make_pool(blocks * bs)
    lat = np.ascontiguousarray(fused[:, :512])
    rope = np.ascontiguousarray(fused[:, 512:])
    q = kvo.make_q(2)
    scale = float(1.0 / np.sqrt(192.0))
    want, want_lse = kvo.mla_decode(q, lat, table, kv_len, bs, scale, use_double=True, rope_pool=rope)
    out, lse = run_decode(q, lat, table, kv_len, bs, scale, variant, rope_pool_u16=rope)
    scenarios.check_attention(out, lse, kvo.bf16_to_f32(want).astype(np.float64), want_lse.astype(np.float64),
                              what="two caches", strict_abs=True)


@pytest.mark.parametrize("variant", VARIANTS)
def test_kv_range_shards_merge_to_whole(variant):
    """KV-range split: each shard's un-normalised partial, merged by b200kv_lse_merge, equals the
    single-device result (the multi-GPU long-context path run on one device)."""
    bs, n, blocks = 64, 8192, 140
    kv_len = np.array([n], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(1, scale=6.0 / 24.0)
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, 1.0 / 24.0)
    shards = 4
    per = n // shards
    parts = []
    for r in range(shards):
        po, pm, pl = run_decode(q, pool, table, np.array([per], np.int32), bs, 1.0 / 24.0, variant,
                                kv_begin=np.array([r * per], np.int32), partial=True)
        want_o, want_m, want_l = kvo.mla_decode(q, pool, table, np.array([per], np.int32), bs, 1.0 / 24.0,
                                                kv_begin=np.array([r * per], np.int32), partial=True)
        # partials may use different reference maxima: compare after normalising each
        got_n = po / pl[..., None]
        want_n = want_o / want_l[..., None]
        assert np.abs(got_n - want_n).max() <= 2e-3 + 1e-2 * np.abs(want_n).max()
        assert np.abs((pm + np.log(pl)) - (want_m + np.log(want_l))).max() <= 1e-3
        parts.append((po, pm, pl))
    po = torch.from_numpy(np.stack([p[0].reshape(-1, 512) for p in parts])).cuda()
    pm = torch.from_numpy(np.stack([p[1].reshape(-1) for p in parts])).cuda()
    pl = torch.from_numpy(np.stack([p[2].reshape(-1) for p in parts])).cuda()
    out = torch.empty((64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(64, dtype=torch.float32, device="cuda")
    b200kv.lse_merge(po, pm, pl, out, lse)
    torch.cuda.synchronize()
    from gpu_util import from_dev_bf16
    scenarios.check_attention(from_dev_bf16(out).reshape(1, 64, 512), lse.cpu().numpy().reshape(1, 64), ref_out,
                              ref_lse, what="merged shards")
    # and the device merge equals the oracle's merge of the same partials
    want_out, want_lse = kvo.lse_merge(po.cpu().numpy(), pm.cpu().numpy(), pl.cpu().numpy())
    assert np.abs(kvo.bf16_to_f32(from_dev_bf16(out)) - kvo.bf16_to_f32(want_out)).max() <= 1e-3
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 1e-4


def test_simt_handles_other_head_counts():
    bs, blocks = 64, 8
    kv_len = np.array([150, 64], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    for heads in (8, 128):
        q = kvo.make_q(2, heads=heads)
        want, want_lse = kvo.mla_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, use_double=True)
        out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, b200kv.DECODE_AUTO)
        scenarios.check_attention(out, lse, kvo.bf16_to_f32(want).astype(np.float64), want_lse.astype(np.float64),
                                  what=f"heads={heads}", strict_abs=True)


def test_decode_reports_bad_block_without_faulting():
    bs = 64
    pool = kvo.make_pool(4 * bs)
    table = np.array([[1, 99]], dtype=np.int32)
    q = kvo.make_q(1)
    from gpu_util import to_dev_bf16, to_dev_i32
    for variant in (b200kv.DECODE_SIMT, b200kv.DECODE_TCGEN05):
        qd, pd = to_dev_bf16(q), to_dev_bf16(pool)
        out = torch.zeros((1, 64, 512), dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(b200kv.decode_workspace_bytes(1), dtype=torch.uint8, device="cuda")
        status = b200kv.new_status()
        b200kv.mla_decode(qd, b200kv.pool_view(pd), to_dev_i32(table), to_dev_i32([100]), bs, 1.0 / 24.0, out=out,
                          workspace=ws, variant=variant, status=status)
        torch.cuda.synchronize()
        st = status.cpu().tolist()
        assert st[0] == b200kv.DEV_BAD_BLOCK and st[1] == 0 and st[2] == 1 and st[3] == 99


def test_attention_over_a_selected_subset_of_tokens():
    """A top-k style selection (512 of a few thousand tokens per sequence, in arbitrary order) resolved to pool
    rows and attended over as a table of single-row blocks; the oracle gets the same rows as its table."""
    import torch

    from gpu_util import to_dev_i32

    bs, sel = 64, 512
    kv_len = np.array([3000, 640, 4096, 17], dtype=np.int32)
    B = len(kv_len)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 3
    table = scenarios.build_tables(kv_len, bs, blocks, order=kvo.permutation(blocks))
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(B)
    index = np.full((B, sel), -7, dtype=np.int32)
    n_sel = np.minimum(kv_len, sel).astype(np.int32)
    for b in range(B):
        picks = kvo.permutation(int(kv_len[b]), seed=kvo.BASE_SEED + b)[: n_sel[b]]   # distinct, unordered
        index[b, : n_sel[b]] = picks
    d_table, d_index, d_n = to_dev_i32(table), to_dev_i32(index), to_dev_i32(n_sel)
    st = b200kv.new_status()
    rows = b200kv.resolve_rows(d_table, bs, d_index, d_n, blocks * bs, status=st)
    torch.cuda.synchronize()
    rows_np = rows.cpu().numpy()
    expect = np.full((B, sel), -1, dtype=np.int32)
    for b in range(B):
        t = index[b, : n_sel[b]].astype(np.int64)
        expect[b, : n_sel[b]] = table[b, t // bs].astype(np.int64) * bs + t % bs
    assert np.array_equal(rows_np, expect) and st.cpu().tolist()[0] == 0
    out, lse = run_decode(q, pool, rows_np, n_sel, 1, 1.0 / 24.0, b200kv.DECODE_AUTO)
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, rows_np, n_sel, 1, 1.0 / 24.0)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what="selected subset")
    o_out, o_lse = kvo.mla_decode(q, pool, rows_np, n_sel, 1, 1.0 / 24.0)[:2]
    scenarios.check_attention(o_out, o_lse, ref_out, ref_lse, what="oracle on the same rows")
    # a token outside the sequence's table is recorded, not dereferenced
    index[1, 0] = 64 * 4096
    st2 = b200kv.new_status()
    b200kv.resolve_rows(d_table, bs, to_dev_i32(index), d_n, blocks * bs, status=st2)
    torch.cuda.synchronize()
    assert st2.cpu().tolist()[0] == b200kv.DEV_BAD_BLOCK


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("max_ctas", [0, 3], ids=["all-sms", "3-ctas"])
def test_attention_over_gathered_rows(variant, max_ctas):
    """The row list itself as the call's argument (row_index): the tensor-core kernel copies the listed rows
    into its swizzled stages with 16-byte asynchronous copies; the CUDA-core kernel reads the list as single-row blocks. Selections of
    512 tokens in arbitrary order out of long, fragmented histories, a short one (17 rows: one partial tile), an
    empty one, one of exactly a tile, and one whose list is longer than the others (stride larger than any count).
    Against the float64 statement on the same rows, and the two kernels agree on what the rows are: a repeated
    row counts twice."""
    from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

    bs, stride = 64, 520
    kv_len = np.array([3000, 640, 4096, 17, 0, 64, 2049], dtype=np.int32)
    n_sel = np.array([512, 512, 512, 17, 0, 64, 515], dtype=np.int32)
    B = len(kv_len)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 3
    table = scenarios.build_tables(kv_len, bs, blocks, order=kvo.permutation(blocks))
    pool_np = kvo.make_pool(blocks * bs)
    q_np = kvo.make_q(B, scale=2.0 / 24.0)
    rows = np.full((B, stride), -1, dtype=np.int32)
    for b in range(B):
        if n_sel[b] == 0:
            continue
        picks = kvo.permutation(int(kv_len[b]), seed=kvo.BASE_SEED + 31 * b)[: n_sel[b]].astype(np.int64)
        rows[b, : n_sel[b]] = table[b, picks // bs].astype(np.int64) * bs + picks % bs
    rows[3, 5] = rows[3, 4]  # the same row twice
    q, pool = to_dev_bf16(q_np), to_dev_bf16(pool_np)
    status = b200kv.new_status()
    out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(B, 64, max_ctas), dtype=torch.uint8, device="cuda")
    b200kv.mla_decode(q, b200kv.pool_view(pool), None, to_dev_i32(n_sel), bs, 1.0 / 24.0, out=out, lse=lse, workspace=ws,
                      variant=variant, max_ctas=max_ctas, status=status, row_index=to_dev_i32(rows))
    status_ok(status)
    ref_out, ref_lse = scenarios.ref_attention_f64(q_np, pool_np, rows, n_sel, 1, 1.0 / 24.0)
    scenarios.check_attention(from_dev_bf16(out), lse.cpu().numpy(), ref_out, ref_lse, what="gathered rows")


def test_gathered_rows_outside_the_pool_are_recorded_not_read():
    from gpu_util import to_dev_bf16, to_dev_i32

    pool_rows = 256
    pool = to_dev_bf16(kvo.make_pool(pool_rows))
    q = to_dev_bf16(kvo.make_q(2))
    rows = np.arange(2 * 64, dtype=np.int32).reshape(2, 64)
    rows[1, 7] = pool_rows  # one past the end
    out = torch.zeros((2, 64, 512), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(2, 64, 0), dtype=torch.uint8, device="cuda")
    for variant in (b200kv.DECODE_TCGEN05, b200kv.DECODE_SIMT):
        status = b200kv.new_status()
        b200kv.mla_decode(q, b200kv.pool_view(pool), None, to_dev_i32(np.array([64, 64], dtype=np.int32)), 64, 1.0 / 24.0,
                          out=out, workspace=ws, variant=variant, status=status, row_index=to_dev_i32(rows))
        torch.cuda.synchronize()
        assert status.cpu().tolist()[0] == b200kv.DEV_BAD_BLOCK
    with pytest.raises(b200kv.B200KVError) as err:  # a row list and a KV range exclude each other
        b200kv.mla_decode(q, b200kv.pool_view(pool), None, to_dev_i32(np.array([64, 64], dtype=np.int32)), 64, 1.0 / 24.0,
                          out=out, workspace=ws, row_index=to_dev_i32(rows), kv_begin=to_dev_i32(np.zeros(2, dtype=np.int32)))
    assert err.value.code == b200kv.ERR_INVALID


@pytest.mark.parametrize("case", ["batch-split", "few-long", "many-short", "simt"])
def test_output_quantised_by_the_launch_that_writes_it(case):
    """out_fp8 / out_scale: the MX quantisation of the attention output as the epilogue of the merge kernel (and,
    for sequences a single CTA covers, of the read-back of what the decode kernel wrote). Bit for bit the
    stand-alone quantiser on `out`, which is bit for bit the oracle's. Sequences cut over several CTAs (the
    32-CTAs-per-sequence merge), a few long ones (the 256-CTAs-per-sequence merge), many short ones with empty
    ones among them (whole sequences per CTA), and the CUDA-core path (quantiser behind the attention)."""
    from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

    bs = 64
    kv_len = {"batch-split": np.array([2000 + 37 * i for i in range(20)], dtype=np.int32),
              "few-long": np.array([9000, 4097], dtype=np.int32),
              "many-short": np.array([(i * 37) % 130 for i in range(200)], dtype=np.int32),
              "simt": np.array([300, 0, 65, 1000], dtype=np.int32)}[case]
    variant = b200kv.DECODE_SIMT if case == "simt" else b200kv.DECODE_TCGEN05
    B = len(kv_len)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 3
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = to_dev_bf16(kvo.make_pool(blocks * bs))
    q = to_dev_bf16(kvo.make_q(B, scale=2.0 / 24.0))
    out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    q8 = torch.full((B, 64, 512), 0x55, dtype=torch.uint8, device="cuda")
    sc = torch.full((B, 64, 16), 0x55, dtype=torch.uint8, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(B, 64, 0), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out,
                      workspace=ws, variant=variant, status=status, quantised=(q8, sc))
    status_ok(status)
    want8 = torch.empty((B, 64 * 512), dtype=torch.uint8, device="cuda")
    want_sc = torch.empty((B, 64 * 16), dtype=torch.uint8, device="cuda")
    b200kv.mx_quant_e4m3(out.view(B, 64 * 512), want8, want_sc)
    torch.cuda.synchronize()
    assert torch.equal(q8.view(B, -1), want8), "FP8 codes differ from the stand-alone quantiser's"
    assert torch.equal(sc.view(B, -1), want_sc), "scales differ from the stand-alone quantiser's"
    o8, osc = kvo.mx_quant_e4m3(from_dev_bf16(out).reshape(B, -1))
    assert np.array_equal(q8.view(B, -1).cpu().numpy(), o8) and np.array_equal(sc.view(B, -1).cpu().numpy(), osc)
    with pytest.raises(b200kv.B200KVError) as err:  # the two buffers come together
        args_q = (q8, None)
        b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out,
                          workspace=ws, variant=variant, status=status, quantised=args_q)
    assert err.value.code == b200kv.ERR_INVALID


@pytest.mark.parametrize("seed", range(4))
def test_random_batches_and_grid_sizes_match_the_reference(seed):
    """Many small random batches (lengths around the tile and block edges, empty sequences, one long sequence)
    on grids of 1 to 148 CTAs: the cut of the tile list, the slots of the partials and the merge must agree
    for every combination (grids larger than the number of tiles leave CTAs without work)."""
    rng = np.random.default_rng(1000 + seed)
    bs = 64
    for case in range(10):
        B = int(rng.integers(1, 24))
        choices = np.array([0, 1, 63, 64, 65, 127, 128, 129, 500, 1000, 2100])
        kv_len = rng.choice(choices, size=B).astype(np.int32)
        if case % 3 == 0:
            kv_len[int(rng.integers(0, B))] = int(rng.integers(3000, 9000))
        if not kv_len.any():
            kv_len[0] = 65
        blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 2
        table = scenarios.build_tables(kv_len, bs, blocks, order=rng.permutation(blocks).astype(np.int32))
        pool = kvo.make_pool(blocks * bs, seed=kvo.BASE_SEED + 31 * seed + case)
        q = kvo.make_q(B, seed=kvo.BASE_SEED + 7 * seed + case)
        ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, table, kv_len, bs, 1.0 / 24.0)
        for max_ctas in (int(rng.choice([1, 2, 3, 5, 7])), int(rng.choice([16, 31, 32, 64])), 0):
            out, lse = run_decode(q, pool, table, kv_len, bs, 1.0 / 24.0, b200kv.DECODE_TCGEN05, max_ctas=max_ctas)
            scenarios.check_attention(out, lse, ref_out, ref_lse,
                                      what=f"seed {seed} case {case} lens {kv_len.tolist()} ctas {max_ctas}")


def _fused_append_case(kv_len, bs, blocks, seed_scale, max_ctas, two_caches=False):
    """Pool + new rows; returns (device result, oracle result) of append-then-attend."""
    from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

    B = len(kv_len)
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = kvo.make_pool(blocks * bs)
    q = kvo.make_q(B, scale=seed_scale)
    new_rows = kvo.make_pool(B)[:, :576].copy()  # any bf16 rows will do; stream 1, other count
    new_rows[:, ::7] ^= 0x0040                    # and differ from what the pool holds at those rows
    last = kv_len.astype(np.int64) - 1
    live = kv_len > 0
    slots = np.full(B, -1, dtype=np.int32)
    slots[live] = (table[np.arange(B)[live], last[live] // bs].astype(np.int64) * bs + last[live] % bs).astype(np.int32)
    want_pool = pool.copy()
    assert kvo.append(want_pool, np.ascontiguousarray(new_rows[live, :512]), np.ascontiguousarray(new_rows[live, 512:]),
                      slots[live]) == 0
    ref_out, ref_lse = scenarios.ref_attention_f64(q, want_pool, table, kv_len, bs, 1.0 / 24.0)

    if two_caches:
        lat = to_dev_bf16(np.ascontiguousarray(pool[:, :512]))
        rope = to_dev_bf16(np.ascontiguousarray(pool[:, 512:]))
        view = b200kv.pool_view(lat, rope)
    else:
        dev_pool = to_dev_bf16(pool)
        view = b200kv.pool_view(dev_pool)
    new_lat = to_dev_bf16(np.ascontiguousarray(new_rows[:, :512]))
    new_rope = to_dev_bf16(np.ascontiguousarray(new_rows[:, 512:]))
    dq = to_dev_bf16(q)
    out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(B, 64, max_ctas), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    b200kv.mla_decode(dq, view, to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out, lse=lse, workspace=ws,
                      variant=b200kv.DECODE_TCGEN05, max_ctas=max_ctas, status=status, new_rows=(new_lat, new_rope))
    status_ok(status)
    if two_caches:
        got_pool = np.concatenate([from_dev_bf16(lat), from_dev_bf16(rope)], axis=1)
    else:
        got_pool = from_dev_bf16(dev_pool)
    return got_pool, want_pool, from_dev_bf16(out), lse.cpu().numpy(), ref_out, ref_lse


@pytest.mark.parametrize("max_ctas", [0, 5, 1])
def test_append_fused_into_the_attention_launch(max_ctas):
    """The decode launch writes each sequence's new row at position kv_len - 1 and attends over it: the pool
    equals the oracle's append bit for bit, the attention matches the reference on the appended pool. Lengths
    put the new row at the start, in the middle and at the end of a tile and of a block, in one-tile and
    one-token sequences, and leave an empty sequence alone."""
    bs = 64
    kv_len = np.array([4097, 1, 64, 65, 0, 128, 129, 1000, 63, 2048, 2], dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 5
    got_pool, want_pool, out, lse, ref_out, ref_lse = _fused_append_case(kv_len, bs, blocks, 4.0 / 24.0, max_ctas)
    assert np.array_equal(got_pool, want_pool)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what=f"fused append max_ctas={max_ctas}")
    assert (out[kv_len == 0] == 0).all()


def test_append_fused_with_the_reference_layout_of_two_caches():
    bs = 128
    kv_len = np.array([129, 128, 700, 1], dtype=np.int32)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 2
    got_pool, want_pool, out, lse, ref_out, ref_lse = _fused_append_case(kv_len, bs, blocks, 1.0 / 24.0, 0, two_caches=True)
    assert np.array_equal(got_pool, want_pool)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what="fused append, two caches")


def test_append_fused_is_refused_where_it_cannot_run():
    from gpu_util import to_dev_bf16, to_dev_i32

    bs, kv_len = 64, np.array([10], dtype=np.int32)
    table = scenarios.build_tables(kv_len, bs, 2)
    pool = to_dev_bf16(kvo.make_pool(2 * bs))
    q = to_dev_bf16(kvo.make_q(1))
    out = torch.empty((1, 64, 512), dtype=torch.bfloat16, device="cuda")
    rows = to_dev_bf16(kvo.make_pool(1))
    ws = torch.empty(b200kv.decode_workspace_bytes(1, 64, 0), dtype=torch.uint8, device="cuda")
    with pytest.raises(b200kv.B200KVError):  # the CUDA-core kernel has no fused append
        b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1 / 24, out=out,
                          workspace=ws, variant=b200kv.DECODE_SIMT, new_rows=(rows[:, :512], rows[:, 512:]))
    with pytest.raises(b200kv.B200KVError):  # nor a KV-range shard
        b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1 / 24, out=out,
                          workspace=ws, variant=b200kv.DECODE_TCGEN05, kv_begin=to_dev_i32(np.zeros(1)),
                          new_rows=(rows[:, :512], rows[:, 512:]))


def test_stable_tables_flag_changes_nothing_but_the_order_of_reads():
    """With B200KV_DECODE_STABLE_TABLES the kernel looks up its slice and first rows before it waits for the
    preceding kernel; behind a kernel that writes Q (as the projection before attention does) the results are
    the same, bit for bit."""
    from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

    bs = 64
    kv_len = scenarios.ragged_lengths(9, 1, 3000)
    blocks = int(sum(scenarios.blocks_for(int(n), bs) for n in kv_len)) + 3
    table = scenarios.fragmented_tables(kv_len, bs, blocks)
    pool = to_dev_bf16(kvo.make_pool(blocks * bs))
    q_src = to_dev_bf16(kvo.make_q(len(kv_len), scale=2.0 / 24.0))
    tbl, lens = to_dev_i32(table), to_dev_i32(kv_len)
    ws = torch.empty(b200kv.decode_workspace_bytes(len(kv_len), 64, 0), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    results = []
    for stable in (False, True):
        q = torch.zeros_like(q_src)
        out = torch.full((len(kv_len), 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((len(kv_len), 64), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        q.copy_(q_src)  # a kernel on the same stream writes Q just before the launch
        b200kv.mla_decode(q, b200kv.pool_view(pool), tbl, lens, bs, 1.0 / 24.0, out=out, lse=lse, workspace=ws,
                          variant=b200kv.DECODE_TCGEN05, status=status, stable_tables=stable)
        status_ok(status)
        results.append((from_dev_bf16(out), lse.cpu().numpy()))
    for other in results[1:]:
        assert np.array_equal(results[0][0], other[0])
        assert np.array_equal(results[0][1], other[1])
    ref_out, ref_lse = scenarios.ref_attention_f64(kvo.make_q(len(kv_len), scale=2.0 / 24.0), kvo.make_pool(blocks * bs),
                                                   table, kv_len, bs, 1.0 / 24.0)
    scenarios.check_attention(results[1][0], results[1][1], ref_out, ref_lse, what="stable tables")


def test_headline_configuration_in_full_with_fused_append():
    """The configuration every published number is quoted on, whole: 32 sequences x 4096 tokens, block 64,
    seeded permuted block tables, the default grid (one CTA per SM, cut by cost), the append fused into the
    launch. All 32 x 64 output rows are compared with the oracle (double accumulation) and the pool bit for bit."""
    from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

    bs, B, ctx = 64, 32, 4096
    blocks = B * (ctx // bs)
    kv_len = np.full(B, ctx, dtype=np.int32)
    table = kvo.permutation(blocks).reshape(B, ctx // bs)
    pool_np = kvo.make_pool(blocks * bs)
    q_np = kvo.make_q(B)
    new = kvo.normal_bf16(B * kvo.ROW, kvo.STREAM_NEW).reshape(B, kvo.ROW)
    slots = (table[:, -1].astype(np.int64) * bs + (ctx - 1) % bs).astype(np.int32)
    want_pool = pool_np.copy()
    assert kvo.append(want_pool, np.ascontiguousarray(new[:, :512]), np.ascontiguousarray(new[:, 512:]), slots) == 0
    want, want_lse = kvo.mla_decode(q_np, want_pool, table, kv_len, bs, 1.0 / 24.0, use_double=True)

    pool, q, new_d = to_dev_bf16(pool_np), to_dev_bf16(q_np), to_dev_bf16(new)
    out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(B), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    for stable in (False, True):  # without and with the benchmark's flags
        pool.copy_(to_dev_bf16(pool_np))
        out.fill_(float("nan"))
        b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out,
                          lse=lse, workspace=ws, variant=b200kv.DECODE_AUTO, max_ctas=0, status=status,
                          new_rows=(new_d[:, :512], new_d[:, 512:]), stable_tables=stable)
        status_ok(status)
        assert np.array_equal(from_dev_bf16(pool), want_pool), "pool differs from the oracle's append"
        scenarios.check_attention(from_dev_bf16(out), lse.cpu().numpy(), kvo.bf16_to_f32(want).astype(np.float64),
                                  want_lse.astype(np.float64), what=f"configs[1] in full, stable_tables={stable}",
                                  strict_abs=True, elementwise=True)


def test_fused_append_through_a_bad_table_entry_writes_nothing():
    """A sequence whose last block id points outside the pool: the launch records B200KV_DEV_BAD_BLOCK and
    leaves every pool row as it was (the separate append skips a bad slot the same way); it must not fall
    back to writing the new row into some other sequence's block."""
    from gpu_util import from_dev_bf16, to_dev_bf16, to_dev_i32

    bs = 64
    kv_len = np.array([200, 130], dtype=np.int32)
    blocks = 10
    table = scenarios.build_tables(kv_len, bs, blocks)
    table[1, (130 - 1) // bs] = 4000  # the block that should receive sequence 1's new row does not exist
    pool_np = kvo.make_pool(blocks * bs)
    pool, q = to_dev_bf16(pool_np), to_dev_bf16(kvo.make_q(2))
    new = to_dev_bf16(kvo.make_pool(2)[:, :576].copy())
    out = torch.zeros((2, 64, 512), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(2), dtype=torch.uint8, device="cuda")
    for max_ctas in (0, 1):
        status = b200kv.new_status()
        # sequence 0 alone would have been appended; run it without its new row's slot being touched either:
        # only the table of sequence 1 is bad, so sequence 0's row is the one legitimate write
        b200kv.mla_decode(q, b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(kv_len), bs, 1.0 / 24.0, out=out,
                          workspace=ws, variant=b200kv.DECODE_TCGEN05, max_ctas=max_ctas, status=status,
                          new_rows=(new[:, :512], new[:, 512:]))
        torch.cuda.synchronize()
        st = status.cpu().tolist()
        assert st[0] == b200kv.DEV_BAD_BLOCK and st[1] == 1 and st[3] == 4000, st
        want_pool = pool_np.copy()
        slot0 = int(table[0, (200 - 1) // bs]) * bs + (200 - 1) % bs
        want_pool[slot0] = from_dev_bf16(new)[0]
        assert np.array_equal(from_dev_bf16(pool), want_pool), "a pool row other than sequence 0's slot changed"


@pytest.mark.parametrize("variant", VARIANTS)
def test_length_beyond_the_table_row_is_reported_not_read(variant):
    """kv_len lives on the device, so the host cannot check it against max_blocks * block_size: a length that
    runs past the sequence's row of the block table is recorded as a bad block, and the entries of the next
    row (or the memory behind the table) are never used as block ids."""
    from gpu_util import to_dev_bf16, to_dev_i32

    bs = 64
    pool = to_dev_bf16(kvo.make_pool(8 * bs))
    table = np.array([[1, 2], [3, 4]], dtype=np.int32)
    for seq, lens in ((0, [3 * bs, 10]), (1, [10, 2 * bs + 1])):
        out = torch.zeros((2, 64, 512), dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(b200kv.decode_workspace_bytes(2), dtype=torch.uint8, device="cuda")
        status = b200kv.new_status()
        b200kv.mla_decode(to_dev_bf16(kvo.make_q(2)), b200kv.pool_view(pool), to_dev_i32(table), to_dev_i32(lens), bs,
                          1.0 / 24.0, out=out, workspace=ws, variant=variant, status=status)
        torch.cuda.synchronize()
        st = status.cpu().tolist()
        assert st[0] == b200kv.DEV_BAD_BLOCK and st[1] == seq and st[2] == 2 and st[3] == -1, st
