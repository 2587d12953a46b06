"""Helpers for the GPU parity tests: numpy (uint16 bf16 bits) <-> torch device tensors."""
from __future__ import annotations

import numpy as np
import torch

import b200kv


def to_dev_bf16(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> bf16 CUDA tensor of the same shape (bit-exact)."""
    t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    return t.view(torch.bfloat16)


def from_dev_bf16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def to_dev_i32(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def to_dev_i64(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int64)).cuda()


def status_ok(status: torch.Tensor):
    torch.cuda.synchronize()
    vals = status.cpu().tolist()
    assert vals[0] == 0, f"device status word reports {vals}"


def run_decode(q_u16, pool_u16, table, kv_len, bs, scale, variant, kv_begin=None, partial=False, rope_pool_u16=None,
               max_ctas=0):
    """Runs b200kv_mla_decode on the device; returns numpy results like kvo.mla_decode."""
    q = to_dev_bf16(q_u16)
    pool = to_dev_bf16(pool_u16)
    rope = None if rope_pool_u16 is None else to_dev_bf16(rope_pool_u16)
    view = b200kv.pool_view(pool, rope)
    B, H = q.shape[0], q.shape[1]
    tbl = to_dev_i32(table)
    lens = to_dev_i32(kv_len)
    begin = None if kv_begin is None else to_dev_i32(kv_begin)
    ws = torch.empty(b200kv.decode_workspace_bytes(B, H, max_ctas), dtype=torch.uint8, device="cuda")
    status = b200kv.new_status()
    if partial:
        po = torch.full((B, H, 512), float("nan"), dtype=torch.float32, device="cuda")
        pm = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        pl = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        b200kv.mla_decode(q, view, tbl, lens, bs, scale, kv_begin=begin, partial=(po, pm, pl), workspace=ws,
                          variant=variant, max_ctas=max_ctas, status=status)
        status_ok(status)
        return po.cpu().numpy(), pm.cpu().numpy(), pl.cpu().numpy()
    out = torch.full((B, H, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
    b200kv.mla_decode(q, view, tbl, lens, bs, scale, out=out, lse=lse, kv_begin=begin, workspace=ws, variant=variant,
                      max_ctas=max_ctas, status=status)
    status_ok(status)
    return from_dev_bf16(out), lse.cpu().numpy()
