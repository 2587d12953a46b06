"""The engine-facing operator ABI (include/b200kv_aclnn.h): plan once, repoint per layer, launch, as the
reference's StaticOpSlot does (src/core/op_table.cpp:230-270, src/pipeline/pipeline.cpp:390-416), with the
reference's own descriptor shapes (src/memory/static_arena_manager.cpp:480-497, 567-588). Results are held
against the oracle: the caches bit for bit, the attention within the path's tolerance."""
import ctypes
from ctypes import POINTER, byref, c_bool, c_char_p, c_double, c_int32, c_int64, c_uint64, c_void_p

import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, to_dev_bf16, to_dev_i32

pytestmark = pytest.mark.gpu

ACL_FLOAT32, ACL_INT32, ACL_BF16, ACL_FORMAT_ND = 0, 3, 27, 2
L = b200kv.lib


def _setup():
    L.aclCreateTensor.restype = c_void_p
    L.aclCreateTensor.argtypes = [POINTER(c_int64), c_uint64, c_int32, POINTER(c_int64), c_int64, c_int32,
                                  POINTER(c_int64), c_uint64, c_void_p]
    L.aclCreateTensorList.restype = c_void_p
    L.aclCreateTensorList.argtypes = [POINTER(c_void_p), c_uint64]
    L.aclCreateIntArray.restype = c_void_p
    L.aclCreateIntArray.argtypes = [POINTER(c_int64), c_uint64]
    L.aclSetTensorAddr.argtypes = [c_void_p, c_uint64, c_void_p, c_void_p]
    L.aclSetDynamicTensorAddr.argtypes = [c_void_p, c_uint64, c_uint64, c_void_p, c_void_p]
    L.aclSetAclOpExecutorRepeatable.argtypes = [c_void_p]
    L.aclDestroyAclOpExecutor.argtypes = [c_void_p]
    L.aclDestroyTensor.argtypes = [c_void_p]
    L.aclDestroyTensorList.argtypes = [c_void_p]
    L.aclDestroyIntArray.argtypes = [c_void_p]
    L.aclGetRecentErrMsg.restype = c_char_p
    L.aclnnScatterPaKvCacheGetWorkspaceSize.argtypes = [c_void_p] * 8 + [c_char_p, c_char_p, c_void_p, c_void_p,
                                                                         POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnScatterPaKvCache.argtypes = [c_void_p, c_uint64, c_void_p, c_void_p]
    L.aclnnFusedInferAttentionScoreV5GetWorkspaceSize.argtypes = (
        [c_void_p] * 31 + [c_int64, c_double, c_int64, c_int64, c_char_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                           c_bool, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, POINTER(c_uint64),
                           POINTER(c_void_p)])
    L.aclnnFusedInferAttentionScoreV5.argtypes = [c_void_p, c_uint64, c_void_p, c_void_p]
    L.aclrtSynchronizeStreamWithTimeout.argtypes = [c_void_p, c_int32]


def tensor(t: torch.Tensor, dims, dtype, strides=None):
    d = (c_int64 * len(dims))(*dims)
    s = None if strides is None else (c_int64 * len(dims))(*strides)
    h = L.aclCreateTensor(d, len(dims), dtype, s, 0, ACL_FORMAT_ND, d, len(dims), t.data_ptr())
    assert h
    return h


def plan_fia(query, key_list, value_list, seq_q, seq_kv, table, q_rope, key_rope, heads, scale, bs, lse_flag, out, lse):
    args = [query, key_list, value_list, None, None, seq_q, seq_kv] + [None] * 7 + [table] + [None] * 9 + \
           [q_rope, key_rope] + [None] * 5
    assert len(args) == 31
    ws, ex = c_uint64(0), c_void_p(0)
    rc = L.aclnnFusedInferAttentionScoreV5GetWorkspaceSize(*args, heads, scale, 65536, 0, b"TND", 1, 3, 0, bs, 0,
                                                           lse_flag, 0, 0, 0, 0, out, lse, byref(ws), byref(ex))
    return rc, ws.value, ex.value


def test_engine_call_sequence_plan_repoint_launch():
    """Batch 1, the reference's geometry: block 128, scale 1/sqrt(192), separate q_latent / q_rope tensors,
    slot = position; three layers share one plan and are reached by repointing the caches."""
    _setup()
    layers, bs, ctx_blocks, pos = 3, 128, 4, 300
    rows = ctx_blocks * bs
    scale = float(1.0 / np.sqrt(192.0))
    fused = [kvo.normal_bf16(rows * kvo.ROW, kvo.STREAM_KV, first=l * 977).reshape(rows, kvo.ROW) for l in range(layers)]
    lat_np = np.stack([np.ascontiguousarray(f[:, :512]) for f in fused])
    rope_np = np.stack([np.ascontiguousarray(f[:, 512:]) for f in fused])
    lat_np[:, pos:] = 0      # the arena is zero-filled beyond what has been written
    rope_np[:, pos:] = 0
    lat, rope = to_dev_bf16(lat_np), to_dev_bf16(rope_np)
    new_np = kvo.normal_bf16(layers * kvo.ROW, kvo.STREAM_NEW).reshape(layers, kvo.ROW)
    q_np = kvo.make_q(layers).reshape(layers, 64, kvo.ROW)
    kv_a = to_dev_bf16(new_np[0:1].copy())                 # act.kv_a: [1, 576] = latent | k_rope
    q_lat = to_dev_bf16(np.ascontiguousarray(q_np[0:1, :, :512]))
    q_rope = to_dev_bf16(np.ascontiguousarray(q_np[0:1, :, 512:]))
    slot = to_dev_i32([pos])
    table = to_dev_i32(np.arange(ctx_blocks, dtype=np.int32)[None])   # the identity the zero-filled table implies
    out = torch.zeros((1, 64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((1, 64, 1), dtype=torch.float32, device="cuda")

    t_key = tensor(kv_a, [1, 512], ACL_BF16)
    t_val = tensor(kv_a[:, 512:], [1, 1, 64], ACL_BF16)
    t_slot = tensor(slot, [1], ACL_INT32)
    t_kc = tensor(lat[0], [ctx_blocks, bs, 1, 512], ACL_BF16)
    t_vc = tensor(rope[0], [ctx_blocks, bs, 1, 64], ACL_BF16)
    ws, ex = c_uint64(0), c_void_p(0)
    rc = L.aclnnScatterPaKvCacheGetWorkspaceSize(t_key, t_kc, t_slot, t_val, t_vc, None, None, None, b"Norm", None,
                                                 None, None, byref(ws), byref(ex))
    assert rc == 0 and ws.value == 0, L.aclGetRecentErrMsg()
    scatter = ex.value
    assert L.aclSetAclOpExecutorRepeatable(scatter) == 0

    t_q = tensor(q_lat, [1, 64, 512], ACL_BF16)
    t_qr = tensor(q_rope, [1, 64, 64], ACL_BF16)
    k0 = tensor(lat[0], [ctx_blocks, bs, 1, 512], ACL_BF16)
    v0 = tensor(lat[0], [ctx_blocks, bs, 1, 512], ACL_BF16)
    key_list = L.aclCreateTensorList((c_void_p * 1)(k0), 1)
    value_list = L.aclCreateTensorList((c_void_p * 1)(v0), 1)
    t_kr = tensor(rope[0], [ctx_blocks, bs, 1, 64], ACL_BF16)
    t_tbl = tensor(table, [1, ctx_blocks], ACL_INT32)
    t_out = tensor(out, [1, 64, 512], ACL_BF16)
    t_lse = tensor(lse, [1, 64, 1], ACL_FLOAT32)
    seq_q = L.aclCreateIntArray((c_int64 * 1)(1), 1)
    seq_kv = L.aclCreateIntArray((c_int64 * 1)(pos + 1), 1)     # live length: the appended token is attended
    rc, fia_ws, fia = plan_fia(t_q, key_list, value_list, seq_q, seq_kv, t_tbl, t_qr, t_kr, 64, scale, bs, True,
                               t_out, t_lse)
    assert rc == 0 and fia_ws > 0, L.aclGetRecentErrMsg()
    assert L.aclSetAclOpExecutorRepeatable(fia) == 0
    workspace = torch.empty(fia_ws, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    for layer in range(layers):
        kv_a.copy_(to_dev_bf16(new_np[layer:layer + 1].copy()))
        q_lat.copy_(to_dev_bf16(np.ascontiguousarray(q_np[layer:layer + 1, :, :512])))
        q_rope.copy_(to_dev_bf16(np.ascontiguousarray(q_np[layer:layer + 1, :, 512:])))
        # the per-layer repointing of src/pipeline/pipeline.cpp:390-400
        assert L.aclSetTensorAddr(scatter, 1, t_kc, lat[layer].data_ptr()) == 0
        assert L.aclSetTensorAddr(scatter, 4, t_vc, rope[layer].data_ptr()) == 0
        assert L.aclSetDynamicTensorAddr(fia, 1, 0, key_list, lat[layer].data_ptr()) == 0
        assert L.aclSetDynamicTensorAddr(fia, 2, 0, value_list, lat[layer].data_ptr()) == 0
        assert L.aclSetTensorAddr(fia, 25, t_kr, rope[layer].data_ptr()) == 0
        assert L.aclnnScatterPaKvCache(None, 0, scatter, stream) == 0, L.aclGetRecentErrMsg()
        assert L.aclnnFusedInferAttentionScoreV5(workspace.data_ptr(), fia_ws, fia, stream) == 0, L.aclGetRecentErrMsg()
        assert L.aclrtSynchronizeStreamWithTimeout(stream, 30000) == 0

        want_l, want_r = lat_np[layer].copy(), rope_np[layer].copy()
        kvo.append(want_l, new_np[layer:layer + 1, :512].copy(), new_np[layer:layer + 1, 512:].copy(),
                   np.array([pos], np.int32), rope_pool=want_r)
        assert (from_dev_bf16(lat[layer]) == want_l).all() and (from_dev_bf16(rope[layer]) == want_r).all()
        ref, ref_lse = kvo.mla_decode(q_np[layer:layer + 1], want_l, np.arange(ctx_blocks, dtype=np.int32)[None],
                                      np.array([pos + 1], np.int32), bs, scale, use_double=True, rope_pool=want_r)
        scenarios.check_attention(from_dev_bf16(out), lse.cpu().numpy().reshape(1, 64),
                                  kvo.bf16_to_f32(ref).astype(np.float64), ref_lse.astype(np.float64),
                                  what=f"layer {layer}", strict_abs=True)

    # 32-byte alignment of replacement addresses, as StaticOpSlot::SetAddress demands
    assert L.aclSetTensorAddr(scatter, 1, t_kc, lat[0].data_ptr() + 16) == 161002
    for h in (t_key, t_val, t_slot, t_kc, t_vc, t_q, t_qr, t_kr, t_tbl, t_out, t_lse):
        L.aclDestroyTensor(h)
    L.aclDestroyTensorList(key_list)
    L.aclDestroyTensorList(value_list)
    L.aclDestroyIntArray(seq_q)
    L.aclDestroyIntArray(seq_kv)
    L.aclDestroyAclOpExecutor(scatter)
    L.aclDestroyAclOpExecutor(fia)


def test_plan_refuses_what_the_kernels_do_not_implement():
    _setup()
    bs, blocks = 64, 4
    lat = torch.zeros((blocks * bs, 512), dtype=torch.bfloat16, device="cuda")
    rope = torch.zeros((blocks * bs, 64), dtype=torch.bfloat16, device="cuda")
    q = torch.zeros((2, 64, 576), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((2, 64, 512), dtype=torch.bfloat16, device="cuda")
    table = torch.zeros((2, blocks), dtype=torch.int32, device="cuda")
    # fused query: q_latent and q_rope are strided views of one [2, 64, 576] buffer
    t_q = tensor(q, [2, 64, 512], ACL_BF16, strides=[64 * 576, 576, 1])
    t_qr = tensor(q[:, :, 512:], [2, 64, 64], ACL_BF16, strides=[64 * 576, 576, 1])
    k0 = tensor(lat, [blocks, bs, 1, 512], ACL_BF16)
    v0 = tensor(lat, [blocks, bs, 1, 512], ACL_BF16)
    kl = L.aclCreateTensorList((c_void_p * 1)(k0), 1)
    vl = L.aclCreateTensorList((c_void_p * 1)(v0), 1)
    t_kr = tensor(rope, [blocks, bs, 1, 64], ACL_BF16)
    t_tbl = tensor(table, [2, blocks], ACL_INT32)
    t_out = tensor(out, [2, 64, 512], ACL_BF16)
    seq_kv = L.aclCreateIntArray((c_int64 * 2)(10, 20), 2)
    rc, ws, ex = plan_fia(t_q, kl, vl, None, seq_kv, t_tbl, t_qr, t_kr, 64, 1.0 / 24.0, bs, False, t_out, None)
    assert rc == 0 and ex, L.aclGetRecentErrMsg()
    L.aclDestroyAclOpExecutor(ex)
    rc, _, _ = plan_fia(t_q, kl, vl, None, seq_kv, t_tbl, t_qr, t_kr, 64, -1.0, bs, False, t_out, None)
    assert rc == 161002                                       # non-positive scale
    rc, _, _ = plan_fia(t_q, kl, vl, None, seq_kv, None, t_qr, t_kr, 64, 1.0 / 24.0, bs, False, t_out, None)
    assert rc == 161001                                       # paged attention without a block table
    one = L.aclCreateIntArray((c_int64 * 1)(10), 1)
    rc, _, _ = plan_fia(t_q, kl, vl, None, one, t_tbl, t_qr, t_kr, 64, 1.0 / 24.0, bs, False, t_out, None)
    assert rc == 161002 and b"one length per sequence" in L.aclGetRecentErrMsg()
    ws_, ex_ = c_uint64(0), c_void_p(0)
    t_slot = tensor(table, [2], ACL_INT32)
    t_key = tensor(q, [2, 512], ACL_BF16, strides=[576, 1])
    t_val = tensor(q[:, :, 512:], [2, 1, 64], ACL_BF16, strides=[576, 64, 1])
    rc = L.aclnnScatterPaKvCacheGetWorkspaceSize(t_key, k0, t_slot, t_val, t_kr, None, None, None, b"Compress", None,
                                                 None, None, byref(ws_), byref(ex_))
    assert rc == 161002 and b"Norm" in L.aclGetRecentErrMsg()
