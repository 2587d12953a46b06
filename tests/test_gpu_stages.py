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
