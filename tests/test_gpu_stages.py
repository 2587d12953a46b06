"""The stages beside the KV path on the GPU, through the C ABI: the fused producer (RMSNorm + rotary
embedding + paged write, and the query's rope slices) and the MX quantiser of the attention output.
Their arithmetic is fixed to the operation, so everything is compared bit for bit with the oracle."""
import numpy as np
import pytest
import torch

import b200kv
import kvo
from gpu_util import from_dev_bf16, status_ok, to_dev_bf16, to_dev_i32

pytestmark = pytest.mark.gpu


def rope_tables(tokens, first_pos=0):
    inv = 1.0 / (10000.0 ** (np.arange(32) / 32.0))
    ang = (first_pos + np.arange(tokens))[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1).astype(np.float32)
    return kvo.f32_to_bf16(cos), kvo.f32_to_bf16(sin)


def gamma_bits():
    return kvo.f32_to_bf16(1.0 + 0.1 * kvo.bf16_to_f32(kvo.normal_bf16(512, 7)))


@pytest.mark.parametrize("tokens,fused_pool", [(1, True), (32, True), (257, False), (4096, True)])
def test_fused_producer_matches_oracle_bit_for_bit(tokens, fused_pool):
    rows = max(2 * tokens, 256)
    pool_np = kvo.make_pool(rows)
    kv_a = kvo.normal_bf16(tokens * 576, 3).reshape(tokens, 576)
    kv_a[0, :512] = kvo.f32_to_bf16(kvo.bf16_to_f32(kv_a[0, :512]) * 100.0)
    gamma, (cos, sin) = gamma_bits(), rope_tables(tokens, first_pos=4000)
    slots = kvo.permutation(rows)[:tokens].astype(np.int32)
    if tokens > 8:
        slots[5] = -1          # padding: nothing written
        slots[7] = rows + 3    # outside the pool: recorded, nothing written
    heads = 64
    q_rope = kvo.normal_bf16(tokens * heads * 64, 2).reshape(tokens, heads, 64) if tokens <= 257 else None

    expect = pool_np.copy()
    bad = kvo.append_fused(expect, kv_a, gamma, cos, sin, slots)
    assert bad == (1 if tokens > 8 else 0)
    exp_latent, exp_rstd = kvo.rmsnorm512(kv_a, gamma)
    exp_rope = kvo.rope_half64(kv_a[:, None, 512:], cos, sin)[:, 0]

    if fused_pool:
        pool = to_dev_bf16(pool_np)
        view = b200kv.pool_view(pool)
    else:  # the reference's split caches: two arrays
        latent, rope = to_dev_bf16(pool_np[:, :512]), to_dev_bf16(pool_np[:, 512:])
        view = b200kv.pool_view(latent, rope)
    d_kv, d_gamma = to_dev_bf16(kv_a), to_dev_bf16(gamma)
    d_cos, d_sin, d_slots = to_dev_bf16(cos), to_dev_bf16(sin), to_dev_i32(slots)
    d_q = to_dev_bf16(q_rope) if q_rope is not None else None
    latent_out = torch.zeros((tokens, 512), dtype=torch.bfloat16, device="cuda")
    rope_out = torch.zeros((tokens, 64), dtype=torch.bfloat16, device="cuda")
    rstd = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    st = b200kv.new_status()
    for _ in range(2):  # twice: the write is idempotent, the q rotation is not, so rotate a fresh copy
        if q_rope is not None:
            d_q.copy_(to_dev_bf16(q_rope))
        b200kv.append_fused(view, d_kv, d_gamma, d_cos, d_sin, d_slots, q_rope=d_q, latent_out=latent_out,
                            rope_out=rope_out, rstd_out=rstd, status=st)
    torch.cuda.synchronize()
    got_status = st.cpu().tolist()
    if tokens > 8:
        assert got_status[0] == b200kv.DEV_BAD_SLOT and got_status[1] == 7 and got_status[2] == rows + 3
    else:
        status_ok(st)
    if fused_pool:
        got_pool = from_dev_bf16(pool)
    else:
        got_pool = np.concatenate([from_dev_bf16(latent), from_dev_bf16(rope)], axis=1)
    assert np.array_equal(got_pool, expect), "pool contents differ from the oracle"
    assert np.array_equal(from_dev_bf16(latent_out), exp_latent)
    assert np.array_equal(from_dev_bf16(rope_out), exp_rope)
    assert np.array_equal(rstd.cpu().numpy().view(np.uint32), exp_rstd.view(np.uint32))
    if q_rope is not None:
        assert np.array_equal(from_dev_bf16(d_q), kvo.rope_half64(q_rope, cos, sin))


def test_fused_producer_then_attention_reads_what_was_written():
    """The producer's rows are what the decode attention then sees: one step of both against the oracle."""
    import scenarios
    from gpu_util import run_decode

    bs, ctx = 64, 300
    blocks = scenarios.blocks_for(ctx, bs) + 2
    pool_np = kvo.make_pool(blocks * bs)
    table = kvo.permutation(blocks)[None, :].astype(np.int32)
    slot = int(table[0, (ctx - 1) // bs]) * bs + (ctx - 1) % bs
    kv_a = kvo.normal_bf16(576, 3).reshape(1, 576)
    gamma, (cos, sin) = gamma_bits(), rope_tables(1, first_pos=ctx - 1)
    expect = pool_np.copy()
    kvo.append_fused(expect, kv_a, gamma, cos, sin, np.array([slot], dtype=np.int32))
    pool = to_dev_bf16(pool_np)
    b200kv.append_fused(b200kv.pool_view(pool), to_dev_bf16(kv_a), to_dev_bf16(gamma), to_dev_bf16(cos), to_dev_bf16(sin),
                        to_dev_i32([slot]))
    torch.cuda.synchronize()
    got_pool = from_dev_bf16(pool)
    assert np.array_equal(got_pool, expect)
    q = kvo.make_q(1)
    kv_len = np.array([ctx], dtype=np.int32)
    out, lse = run_decode(q, got_pool, table, kv_len, bs, 1.0 / 24.0, b200kv.DECODE_TCGEN05)[:2]
    ref_out, ref_lse = scenarios.ref_attention_f64(q, expect, table, kv_len, bs, 1.0 / 24.0)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what="producer then attention")


@pytest.mark.parametrize("rows,cols", [(1, 32), (32, 32768), (5, 4096)])
def test_mx_quant_matches_oracle_bit_for_bit(rows, cols):
    x = kvo.normal_bf16(rows * cols, 2).reshape(rows, cols)
    x[0, :32] = 0
    if cols >= 128:
        x[0, 32:64] = kvo.f32_to_bf16(kvo.bf16_to_f32(x[0, 32:64]) * 1e30)
        x[0, 64:96] = kvo.f32_to_bf16(kvo.bf16_to_f32(x[0, 64:96]) * 1e-36)
        x[0, 100] = 0x7FC0
    if rows > 1:  # attention outputs are small: the benchmark's magnitude
        x[1] = kvo.f32_to_bf16(kvo.bf16_to_f32(x[1]) / 64.0)
    exp_q, exp_s = kvo.mx_quant_e4m3(x)
    d_x = to_dev_bf16(x)
    q = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    s = torch.zeros((rows, cols // 32), dtype=torch.uint8, device="cuda")
    b200kv.mx_quant_e4m3(d_x, q, s)
    torch.cuda.synchronize()
    assert np.array_equal(s.cpu().numpy(), exp_s), "scales differ"
    assert np.array_equal(q.cpu().numpy(), exp_q), "values differ"


def test_stage_entry_points_refuse_bad_arguments():
    pool = torch.zeros((128, 576), dtype=torch.bfloat16, device="cuda")
    view = b200kv.pool_view(pool)
    kv = torch.zeros((4, 576), dtype=torch.bfloat16, device="cuda")
    g = torch.zeros(512, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    slots = to_dev_i32([0, 1, 2, 3])
    with pytest.raises(b200kv.B200KVError) as err:
        narrow = torch.zeros((4, 568), dtype=torch.bfloat16, device="cuda")
        b200kv.append_fused(view, narrow, g, c, c, slots)            # rows narrower than 576
    assert err.value.code == b200kv.ERR_INVALID
    x = torch.zeros((2, 48), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(b200kv.B200KVError) as err:
        b200kv.mx_quant_e4m3(x, torch.zeros((2, 48), dtype=torch.uint8, device="cuda"),
                             torch.zeros((2, 2), dtype=torch.uint8, device="cuda"))  # 48 is not a multiple of 32
    assert err.value.code == b200kv.ERR_INVALID


def test_stage_operators_through_the_operator_abi():
    """aclnnRmsNorm, aclnnApplyRotaryPosEmbV2 and aclnnDynamicMxQuant with the reference's descriptor shapes
    (src/memory/static_arena_manager.cpp:475-495, 590-591) and plan arguments (src/pipeline/pipeline.cpp:212-225,
    250-258): plan, launch, compare with the oracle bit for bit. A shape the kernels do not cover (a 4096-wide
    norm) still plans, as a stand-in that leaves its output alone."""
    import ctypes
    from ctypes import POINTER, byref, c_char_p, c_double, c_int32, c_int64, c_uint64, c_void_p

    L = b200kv.lib
    L.aclCreateTensor.restype = c_void_p
    L.aclCreateTensor.argtypes = [POINTER(c_int64), c_uint64, c_int32, POINTER(c_int64), c_int64, c_int32,
                                  POINTER(c_int64), c_uint64, c_void_p]
    BF16, F32, FP8, E8M0 = 27, 0, 36, 37

    def tensor(t, dims, dtype):
        d = (c_int64 * len(dims))(*dims)
        h = L.aclCreateTensor(d, len(dims), dtype, None, 0, 2, d, len(dims), t.data_ptr())
        assert h
        return c_void_p(h)

    launch_args = [c_void_p, c_uint64, c_void_p, c_void_p]
    T, H = 4, 64
    ws, exe = c_uint64(9), c_void_p()

    # stage 6: kv_a_norm
    kv_a = kvo.normal_bf16(T * 576, 3).reshape(T, 576)
    gamma = gamma_bits()
    d_latent = to_dev_bf16(np.ascontiguousarray(kv_a[:, :512]))
    d_gamma = to_dev_bf16(gamma)
    y = torch.zeros((T, 512), dtype=torch.bfloat16, device="cuda")
    rstd = torch.zeros((T, 1), dtype=torch.float32, device="cuda")
    L.aclnnRmsNormGetWorkspaceSize.argtypes = [c_void_p, c_void_p, c_double, c_void_p, c_void_p, POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnRmsNorm.argtypes = launch_args
    assert L.aclnnRmsNormGetWorkspaceSize(tensor(d_latent, [T, 512], BF16), tensor(d_gamma, [512], BF16), 1e-6,
                                          tensor(y, [T, 512], BF16), tensor(rstd, [T, 1], F32), byref(ws), byref(exe)) == 0
    assert ws.value == 0 and L.aclnnRmsNorm(None, 0, exe, None) == 0
    torch.cuda.synchronize()
    exp_y, exp_r = kvo.rmsnorm512(kv_a, gamma)
    assert np.array_equal(from_dev_bf16(y), exp_y) and np.array_equal(rstd.cpu().numpy()[:, 0].view(np.uint32), exp_r.view(np.uint32))

    # the same operator on a hidden-size row: a stand-in, output untouched
    wide = torch.ones((T, 4096), dtype=torch.bfloat16, device="cuda")
    wide_out = torch.full((T, 4096), 7.0, dtype=torch.bfloat16, device="cuda")
    wide_g = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
    assert L.aclnnRmsNormGetWorkspaceSize(tensor(wide, [T, 4096], BF16), tensor(wide_g, [4096], BF16), 1e-6,
                                          tensor(wide_out, [T, 4096], BF16), None, byref(ws), byref(exe)) == 0
    assert L.aclnnRmsNorm(None, 0, exe, None) == 0
    torch.cuda.synchronize()
    assert bool((wide_out == 7.0).all())

    # stage 7: rope on q [T, 64, 64] and k [T, 1, 64]
    q_np = kvo.normal_bf16(T * H * 64, 2).reshape(T, H, 64)
    k_np = np.ascontiguousarray(kv_a[:, None, 512:])
    cos, sin = rope_tables(T, first_pos=77)
    d_q, d_k, d_cos, d_sin = to_dev_bf16(q_np), to_dev_bf16(k_np), to_dev_bf16(cos), to_dev_bf16(sin)
    L.aclnnApplyRotaryPosEmbV2GetWorkspaceSize.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_char_p,
                                                           POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnApplyRotaryPosEmbV2.argtypes = launch_args
    assert L.aclnnApplyRotaryPosEmbV2GetWorkspaceSize(tensor(d_q, [T, H, 64], BF16), tensor(d_k, [T, 1, 64], BF16),
                                                      tensor(d_cos, [T, 64], BF16), tensor(d_sin, [T, 64], BF16), 1,
                                                      b"half", byref(ws), byref(exe)) == 0
    assert L.aclnnApplyRotaryPosEmbV2(None, 0, exe, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(from_dev_bf16(d_q), kvo.rope_half64(q_np, cos, sin))
    assert np.array_equal(from_dev_bf16(d_k), kvo.rope_half64(k_np, cos, sin))

    # stage 10: attn_quant on [T, 64 x 512]
    cols = 64 * 512
    x_np = kvo.f32_to_bf16(kvo.bf16_to_f32(kvo.normal_bf16(T * cols, 2)) / 64.0).reshape(T, cols)
    d_x = to_dev_bf16(x_np)
    q8 = torch.zeros((T, cols), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((T, cols // 32), dtype=torch.uint8, device="cuda")
    L.aclnnDynamicMxQuantGetWorkspaceSize.argtypes = [c_void_p, c_int64, c_char_p, c_int64, c_int64, c_int64, c_void_p,
                                                      c_void_p, POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnDynamicMxQuant.argtypes = launch_args
    assert L.aclnnDynamicMxQuantGetWorkspaceSize(tensor(d_x, [T, cols], BF16), -1, b"rint", FP8, 32, 0,
                                                 tensor(q8, [T, cols], FP8), tensor(sc, [T, cols // 32], E8M0),
                                                 byref(ws), byref(exe)) == 0
    assert L.aclnnDynamicMxQuant(None, 0, exe, None) == 0
    torch.cuda.synchronize()
    exp_q, exp_s = kvo.mx_quant_e4m3(x_np)
    assert np.array_equal(q8.cpu().numpy(), exp_q) and np.array_equal(sc.cpu().numpy(), exp_s)


def _indexer_inputs(B, H, lens, bs, seed):
    import test_stage_oracle

    return test_stage_oracle._indexer_case(B, H, lens, bs, seed)


@pytest.mark.parametrize("lens,k", [([4096, 300, 5000, 17, 0, 9000], 512), ([70, 64], 2048), ([12000], 100),
                                    ([9000, 8193, 8192, 40000], 2048)])
def test_indexer_selection_matches_oracle_bit_for_bit(lens, k):
    """Exact scores: the selection equals the oracle's, position for position. Sequences of up to 8,192 tokens are
    selected by one CTA, longer ones in two levels (the best of every 8,192-token chunk, then the best of those):
    lengths on both sides of the chunk edge, a chunk that holds fewer tokens than k, five chunks."""
    B, H, bs = len(lens), 64, 64
    q, qs, w, key, ks, table, kv_len = _indexer_inputs(B, H, lens, bs, seed=11 + k)
    # ties on purpose: two tokens with identical keys and scales
    if lens[0] > 40:
        r = lambda t: int(table[0, t // bs]) * bs + t % bs
        key[r(31)] = key[r(5)]
        ks[r(31)] = ks[r(5)]
    exp_scores, exp_index, exp_n = kvo.indexer_topk(q, qs, w, key, ks, table, kv_len, bs, k)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    st = b200kv.new_status()
    index, n_sel = b200kv.indexer_topk(d(q), d(qs), to_dev_bf16(w), d(key), d(ks), to_dev_i32(table), to_dev_i32(kv_len),
                                       bs, int(max(lens)), k, status=st, variant=b200kv.INDEXER_EXACT)
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == 0
    assert np.array_equal(n_sel.cpu().numpy(), exp_n)
    assert np.array_equal(index.cpu().numpy(), exp_index), "selection differs from the oracle"


def _check_selection_up_to_rounding(index, n_sel, got_scores, exp_scores, exp_n, kv_len, k, eps_rel):
    """The tensor-core scores differ from the oracle's by rounding, so its selection is checked as a selection:
    per sequence the count, positions distinct and inside the sequence, the device's own scores in best-first
    order with ties by position, every score within eps of the oracle's (both when the scores are at hand),
    nothing better than the k-th oracle score (by more than eps) left out and nothing worse (by more than eps)
    taken."""
    assert np.array_equal(n_sel, exp_n)
    for b in range(len(kv_len)):
        n, m = int(kv_len[b]), int(n_sel[b])
        assert (index[b, m:] == -1).all()
        if n == 0:
            continue
        want = exp_scores[b, :n].astype(np.float64)
        eps = eps_rel * max(np.abs(want).max(), 1e-30)
        picked = index[b, :m].astype(np.int64)
        assert len(set(picked.tolist())) == m and picked.min() >= 0 and picked.max() < n
        if got_scores is not None:
            got = got_scores[b, :n].astype(np.float64)
            assert np.abs(want - got).max() <= eps, (b, np.abs(want - got).max(), eps)
            mine = got[picked]
            assert (np.diff(mine) <= 0).all(), "not best first by the kernel's own scores"
            same = np.diff(mine) == 0
            assert (np.diff(picked)[same] > 0).all(), "ties not by position"
        assert (np.diff(want[picked]) <= 2 * eps).all(), "not best first by the oracle's scores, up to rounding"
        if m < n:
            kth = np.sort(want)[::-1][m - 1]
            assert want[picked].min() >= kth - 2 * eps
            rest = np.setdiff1d(np.arange(n), picked)
            assert want[rest].max() <= kth + 2 * eps


@pytest.mark.parametrize("lens,heads,k", [([4096, 300, 5000, 17, 0, 9000], 64, 512), ([70, 64], 64, 2048), ([12000], 64, 100),
                                          ([1000, 129, 128, 1, 127], 16, 64), ([4097] * 8, 64, 512)])
def test_indexer_tensor_core_scores_and_selection(lens, heads, k):
    """The FP8 tcgen05 score kernel: scores within 1e-6 of the sequence's largest score of the oracle's fp32 chains
    (the tensor core sums the 128 exact products of a dot product in another order), and the selection made from
    them correct up to that. Fewer heads than the tile's 64, lengths around the tile (128) and block (64) edges, an
    empty sequence, fragmented tables."""
    B, bs = len(lens), 64
    q, qs, w, key, ks, table, kv_len = _indexer_inputs(B, heads, lens, bs, seed=101 + k)
    exp_scores, exp_index, exp_n = kvo.indexer_topk(q, qs, w, key, ks, table, kv_len, bs, k)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    st = b200kv.new_status()
    got = []
    index, n_sel = b200kv.indexer_topk(d(q), d(qs), to_dev_bf16(w), d(key), d(ks), to_dev_i32(table), to_dev_i32(kv_len),
                                       bs, int(max(lens)), k, status=st, variant=b200kv.INDEXER_TCGEN05, scores_out=got)
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == 0
    _check_selection_up_to_rounding(index.cpu().numpy(), n_sel.cpu().numpy(), got[0].cpu().numpy(), exp_scores, exp_n,
                                    kv_len, k, eps_rel=1e-6)


def test_indexer_tensor_core_variant_is_refused_where_it_cannot_run_and_reports_bad_blocks():
    B, heads, bs, k = 2, 64, 64, 16
    q, qs, w, key, ks, table, kv_len = _indexer_inputs(B, heads, [200, 64], bs, seed=5)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    with pytest.raises(b200kv.B200KVError) as err:  # blocks of 16 tokens: a 64-row key load would leave its block
        b200kv.indexer_topk(d(q), d(qs), to_dev_bf16(w), d(key), d(ks), to_dev_i32(table), to_dev_i32(kv_len), 16, 200, k,
                            variant=b200kv.INDEXER_TCGEN05)
    assert err.value.code == b200kv.ERR_INVALID
    bad = table.copy()
    bad[0, 1] = key.shape[0] // bs  # one block past the pool
    st = b200kv.new_status()
    got = []
    b200kv.indexer_topk(d(q), d(qs), to_dev_bf16(w), d(key), d(ks), to_dev_i32(bad), to_dev_i32(kv_len), bs, 200, k,
                        status=st, variant=b200kv.INDEXER_TCGEN05, scores_out=got)
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == b200kv.DEV_BAD_BLOCK
    assert np.isneginf(got[0].cpu().numpy()[0, 64:128]).all()  # the tokens of the missing block do not count


def test_sparse_attention_pipeline_indexer_then_resolved_rows_then_decode():
    """The whole sparse path on the device: top-k positions from the indexer, their pool rows, attention over
    exactly those rows. The selection (tensor-core scores) against the oracle's up to rounding, the attention
    against the float64 reference over the selected rows."""
    import scenarios
    from gpu_util import run_decode

    lens, bs, k = [3000, 700, 4096], 64, 512
    B = len(lens)
    q8, qs, w, key, ks, table, kv_len = _indexer_inputs(B, 64, lens, bs, seed=3)
    pool = kvo.make_pool(key.shape[0])                    # the latent KV pool shares the index cache's paging
    q = kvo.make_q(B)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rows_direct = torch.full((B, k), -9, dtype=torch.int32, device="cuda")
    index, n_sel = b200kv.indexer_topk(d(q8), d(qs), to_dev_bf16(w), d(key), d(ks), to_dev_i32(table), to_dev_i32(kv_len),
                                       bs, max(lens), k, rows_out=rows_direct)
    rows = b200kv.resolve_rows(to_dev_i32(table), bs, index, n_sel, pool.shape[0])
    torch.cuda.synchronize()
    assert torch.equal(rows, rows_direct), "the select kernel's own rows differ from resolve_rows on its positions"
    exp_scores, _, exp_n = kvo.indexer_topk(q8, qs, w, key, ks, table, kv_len, bs, k)
    got_index = index.cpu().numpy()
    _check_selection_up_to_rounding(got_index, n_sel.cpu().numpy(), None, exp_scores, exp_n, kv_len, k, eps_rel=1e-6)
    exp_rows = np.full((B, k), -1, dtype=np.int32)  # the rows of the device's selection
    for b in range(B):
        t = got_index[b, : exp_n[b]].astype(np.int64)
        exp_rows[b, : exp_n[b]] = table[b, t // bs].astype(np.int64) * bs + t % bs
    assert np.array_equal(rows.cpu().numpy(), exp_rows)
    ref_out, ref_lse = scenarios.ref_attention_f64(q, pool, exp_rows, exp_n, 1, 1.0 / 24.0)
    # the rows go from the resolver to the attention on the device: the tensor-core kernel gathers them
    from gpu_util import from_dev_bf16, status_ok
    status = b200kv.new_status()
    out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
    ws = torch.empty(b200kv.decode_workspace_bytes(B), dtype=torch.uint8, device="cuda")
    b200kv.mla_decode(to_dev_bf16(q), b200kv.pool_view(to_dev_bf16(pool)), None, n_sel, bs, 1.0 / 24.0, out=out, lse=lse,
                      workspace=ws, variant=b200kv.DECODE_TCGEN05, status=status, row_index=rows)
    status_ok(status)
    scenarios.check_attention(from_dev_bf16(out), lse.cpu().numpy(), ref_out, ref_lse, what="sparse pipeline, gathered")
    # and as a table of single-row blocks on the CUDA-core kernel
    out, lse = run_decode(q, pool, exp_rows, exp_n, 1, 1.0 / 24.0, b200kv.DECODE_AUTO)
    scenarios.check_attention(out, lse, ref_out, ref_lse, what="sparse pipeline")


def test_indexer_operator_through_the_operator_abi():
    """aclnnQuantLightningIndexer with the contract's shapes (mock/mock_ops.cpp:1118-1221): TND query [T, 64, 128]
    FP8, paged keys [blocks, block_size, 1, 128], out [T, 1, k]; plan, launch with the workspace the plan asked
    for, compare with the oracle's selection."""
    from ctypes import POINTER, byref, c_char_p, c_int32, c_int64, c_uint64, c_void_p

    L = b200kv.lib
    L.aclCreateTensor.restype = c_void_p
    L.aclCreateTensor.argtypes = [POINTER(c_int64), c_uint64, c_int32, POINTER(c_int64), c_int64, c_int32,
                                  POINTER(c_int64), c_uint64, c_void_p]
    BF16, F32, I32, FP8 = 27, 0, 3, 36

    def tensor(t, dims, dtype):
        d = (c_int64 * len(dims))(*dims)
        h = L.aclCreateTensor(d, len(dims), dtype, None, 0, 2, d, len(dims), t.data_ptr())
        assert h
        return c_void_p(h)

    lens, bs, k, H = [900, 64, 2000], 128, 256, 64
    T = len(lens)
    q, qs, w, key, ks, table, kv_len = _indexer_inputs(T, H, lens, bs, seed=21)
    blocks = key.shape[0] // bs
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_q, d_qs, d_w, d_key, d_ks = d(q), d(qs), to_dev_bf16(w), d(key), d(ks)
    d_table, d_len = to_dev_i32(table), to_dev_i32(kv_len)
    d_cum = to_dev_i32(np.arange(1, T + 1))
    out = torch.full((T, 1, k), -5, dtype=torch.int32, device="cuda")
    L.aclnnQuantLightningIndexerGetWorkspaceSize.argtypes = [c_void_p] * 8 + [c_int64, c_int64, c_char_p, c_char_p, c_int64,
                                                                               c_int64, c_int64, c_int64, c_void_p,
                                                                               POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnQuantLightningIndexer.argtypes = [c_void_p, c_uint64, c_void_p, c_void_p]
    ws_bytes, exe = c_uint64(0), c_void_p()
    rc = L.aclnnQuantLightningIndexerGetWorkspaceSize(
        tensor(d_q, [T, H, 128], FP8), tensor(d_key, [blocks, bs, 1, 128], FP8), tensor(d_w, [T, H], BF16),
        tensor(d_qs, [T, H], F32), tensor(d_ks, [blocks, bs, 1], F32), tensor(d_cum, [T], I32), tensor(d_len, [T], I32),
        tensor(d_table, [T, table.shape[1]], I32), 0, 0, b"TND", b"PA_BSND", k, 3, 2 ** 62, 2 ** 62,
        tensor(out, [T, 1, k], I32), byref(ws_bytes), byref(exe))
    assert rc == 0 and ws_bytes.value > 0
    ws = torch.empty(ws_bytes.value, dtype=torch.uint8, device="cuda")
    assert L.aclnnQuantLightningIndexer(ws.data_ptr(), ws_bytes.value, exe, None) == 0
    torch.cuda.synchronize()
    exp_scores, _, exp_n = kvo.indexer_topk(q, qs, w, key, ks, table, kv_len, bs, k)
    got = out.cpu().numpy()[:, 0, :]
    _check_selection_up_to_rounding(got, (got >= 0).sum(axis=1).astype(np.int32), None, exp_scores, exp_n, kv_len, k,
                                    eps_rel=1e-6)
