"""ctypes binding of libb200kv.so, the C ABI of the B200 KV-cache path (include/b200kv.h).

The binding is plumbing for tests, the benchmark and Python callers: it turns torch tensors into raw
device pointers and the current CUDA stream into a handle, and calls the C entry points. There is no
fallback: if the library is missing, importing this package raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200kv.so")

LATENT_DIM = 512
ROPE_DIM = 64
ROW_DIM = LATENT_DIM + ROPE_DIM
HEADS = 64

OK = 0
ERR_NULLPTR = 161001
ERR_INVALID = 161002
ERR_RUNTIME = 361001

DEV_OK, DEV_BAD_SLOT, DEV_BAD_BLOCK, DEV_TIMEOUT, DEV_BAD_PLAN = 0, 1, 2, 3, 4

DECODE_AUTO, DECODE_SIMT, DECODE_TCGEN05 = 0, 1, 2


class B200KVError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"b200kv error {code}: {text}")
        self.code = code


class PoolView(Structure):
    _fields_ = [
        ("latent", c_void_p),
        ("rope", c_void_p),
        ("latent_row_stride", c_int64),
        ("rope_row_stride", c_int64),
        ("pool_rows", c_int64),
    ]


class DecodeArgs(Structure):
    _fields_ = [
        ("q", c_void_p),
        ("q_seq_stride", c_int64),
        ("q_head_stride", c_int64),
        ("pool", PoolView),
        ("block_table", c_void_p),
        ("max_blocks", c_int64),
        ("kv_len", c_void_p),
        ("kv_begin", c_void_p),
        ("batch", c_int32),
        ("heads", c_int32),
        ("block_size", c_int32),
        ("scale", c_float),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("partial_o", c_void_p),
        ("partial_m", c_void_p),
        ("partial_l", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("variant", c_int32),
        ("max_ctas", c_int32),
        ("new_latent", c_void_p),
        ("new_latent_stride", c_int64),
        ("new_rope", c_void_p),
        ("new_rope_stride", c_int64),
        ("flags", ctypes.c_uint32),
        ("row_index", c_void_p),
        ("row_index_stride", c_int64),
        ("out_fp8", c_void_p),
        ("out_scale", c_void_p),
    ]


class ProducerArgs(Structure):
    """b200kv_producer_args (include/b200kv.h)."""

    _fields_ = [
        ("pool", PoolView),
        ("kv_a", c_void_p), ("kv_a_stride", c_int64),
        ("gamma", c_void_p), ("eps", ctypes.c_float),
        ("cos", c_void_p), ("cos_stride", c_int64),
        ("sin", c_void_p), ("sin_stride", c_int64),
        ("slot_mapping", c_void_p), ("n_tokens", c_int64),
        ("q_rope", c_void_p), ("q_token_stride", c_int64), ("q_head_stride", c_int64), ("heads", c_int32),
        ("latent_out", c_void_p), ("latent_out_stride", c_int64),
        ("rope_out", c_void_p), ("rope_out_stride", c_int64),
        ("rstd_out", c_void_p),
    ]


class IndexerArgs(Structure):
    """b200kv_indexer_args (include/b200kv.h)."""

    _fields_ = [
        ("q", c_void_p), ("q_scale", c_void_p), ("weights", c_void_p), ("heads", c_int32),
        ("key_pool", c_void_p), ("key_stride", c_int64), ("k_scale", c_void_p), ("pool_rows", c_int64),
        ("block_table", c_void_p), ("max_blocks", c_int64), ("kv_len", c_void_p), ("batch", c_int32),
        ("block_size", c_int32), ("max_kv_len", c_int64), ("k", c_int32),
        ("index_out", c_void_p), ("n_selected_out", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("variant", c_int32),
        ("rows_out", c_void_p),
    ]


INDEXER_AUTO, INDEXER_EXACT, INDEXER_TCGEN05 = 0, 1, 2


class Reservation(Structure):
    _fields_ = [
        ("blocks_per_layer", c_int64),
        ("total_blocks", c_int64),
        ("latent_bytes", c_int64),
        ("rope_bytes", c_int64),
        ("block_table_bytes", c_int64),
        ("slot_mapping_bytes", c_int64),
    ]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python ascend-moe-engine_b200/build.py` "
            "(there is no CPU or eager fallback for this path)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.b200kv_last_error.restype = c_char_p
    lib.b200kv_abi_version.restype = c_int32
    lib.b200kv_append.restype = c_int32
    lib.b200kv_append.argtypes = [POINTER(PoolView), c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                  c_void_p, c_void_p]
    lib.b200kv_gather.restype = c_int32
    lib.b200kv_gather.argtypes = [POINTER(PoolView), c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                  c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p]
    lib.b200kv_mla_decode_workspace_bytes.restype = c_size_t
    lib.b200kv_mla_decode_workspace_bytes.argtypes = [c_int32, c_int32, c_int32]
    lib.b200kv_mla_decode.restype = c_int32
    lib.b200kv_mla_decode.argtypes = [POINTER(DecodeArgs), c_void_p, c_void_p]
    lib.b200kv_append_fused.restype = c_int32
    lib.b200kv_append_fused.argtypes = [POINTER(ProducerArgs), c_void_p, c_void_p]
    lib.b200kv_mx_quant_e4m3.restype = c_int32
    lib.b200kv_mx_quant_e4m3.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                         c_void_p]
    lib.b200kv_indexer_workspace_bytes.restype = c_size_t
    lib.b200kv_indexer_workspace_bytes.argtypes = [c_int32, c_int64]
    lib.b200kv_indexer_topk.restype = c_int32
    lib.b200kv_indexer_topk.argtypes = [POINTER(IndexerArgs), c_void_p, c_void_p]
    lib.b200kv_resolve_rows.restype = c_int32
    lib.b200kv_resolve_rows.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                        c_void_p, c_void_p, c_void_p]
    lib.b200kv_lse_merge.restype = c_int32
    lib.b200kv_lse_merge.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p]
    lib.b200kv_fill_normal_bf16.restype = c_int32
    lib.b200kv_fill_normal_bf16.argtypes = [c_void_p, c_int64, c_uint64, c_uint64, c_uint64, c_double, c_void_p]
    lib.b200kv_block_pool_create.restype = c_void_p
    lib.b200kv_block_pool_create.argtypes = [c_int32, c_int32, c_int32, c_int32, c_void_p]
    lib.b200kv_block_pool_destroy.argtypes = [c_void_p]
    lib.b200kv_block_pool_destroy.restype = None
    for name in ("admit", "release"):
        fn = getattr(lib, f"b200kv_block_pool_{name}")
        fn.restype = c_int32
        fn.argtypes = [c_void_p, c_int32]
    lib.b200kv_block_pool_grow.restype = c_int32
    lib.b200kv_block_pool_grow.argtypes = [c_void_p, c_int32, c_int32, c_void_p]
    lib.b200kv_block_pool_free_count.restype = c_int32
    lib.b200kv_block_pool_free_count.argtypes = [c_void_p]
    lib.b200kv_block_pool_seq_len.restype = c_int32
    lib.b200kv_block_pool_seq_len.argtypes = [c_void_p, c_int32]
    lib.b200kv_block_pool_table.restype = POINTER(c_int32)
    lib.b200kv_block_pool_table.argtypes = [c_void_p]
    lib.b200kv_block_pool_lens.restype = POINTER(c_int32)
    lib.b200kv_block_pool_lens.argtypes = [c_void_p]
    lib.b200kv_block_pool_export_free.restype = c_int32
    lib.b200kv_block_pool_export_free.argtypes = [c_void_p, c_void_p, c_int32]
    lib.b200kv_block_pool_validate.restype = c_int32
    lib.b200kv_block_pool_validate.argtypes = [c_void_p]
    lib.b200kv_plan_reservation.restype = c_int32
    lib.b200kv_plan_reservation.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int64, POINTER(Reservation)]
    lib.b200kv_utilisation.restype = c_double
    lib.b200kv_utilisation.argtypes = [c_int64, c_int64, c_int64]
    return lib


lib = _load()


def fault_inject(entry_point: str, after_calls: int = 0) -> None:
    """The call of `entry_point` after the next `after_calls` ones fails on the host with ERR_RUNTIME (tests)."""
    lib.b200kv_fault_inject.restype = c_int32
    lib.b200kv_fault_inject.argtypes = [c_char_p, c_int32]
    check(lib.b200kv_fault_inject(entry_point.encode(), after_calls))


def fault_clear() -> int:
    lib.b200kv_fault_clear.restype = c_int64
    return int(lib.b200kv_fault_clear())


def last_error() -> str:
    return (lib.b200kv_last_error() or b"").decode()


def check(code: int) -> None:
    if code != OK:
        raise B200KVError(code, last_error())


# ---------------------------------------------------------------------------------------------------
# Device operations on torch tensors
# ---------------------------------------------------------------------------------------------------
def _stream_handle(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def _ptr(t) -> int:
    return 0 if t is None else int(t.data_ptr())


def pool_view(latent, rope=None) -> PoolView:
    """A layer's pool as a view. `latent`: bf16 [rows, 576] (fused row: rope is columns 512..575) when
    `rope` is None, else bf16 [rows, >=512] with `rope` bf16 [rows, >=64] (the reference's two caches)."""
    assert latent.dim() == 2 and latent.stride(1) == 1
    view = PoolView()
    view.latent = _ptr(latent)
    view.latent_row_stride = latent.stride(0)
    view.pool_rows = latent.shape[0]
    if rope is None:
        assert latent.shape[1] == ROW_DIM
        view.rope = _ptr(latent) + LATENT_DIM * 2
        view.rope_row_stride = latent.stride(0)
    else:
        assert rope.dim() == 2 and rope.stride(1) == 1 and rope.shape[0] == latent.shape[0]
        view.rope = _ptr(rope)
        view.rope_row_stride = rope.stride(0)
    return view


def new_status(device="cuda"):
    import torch

    return torch.zeros(4, dtype=torch.int32, device=device)


def append(view: PoolView, latent_src, rope_src, slot_mapping, status=None, stream=None) -> None:
    """latent_src bf16 [T, >=512] and rope_src bf16 [T, >=64] (row strides taken from the tensors),
    slot_mapping int32 [T] on the device."""
    n = int(slot_mapping.shape[0])
    check(lib.b200kv_append(ctypes.byref(view), _ptr(latent_src), latent_src.stride(0) if n else LATENT_DIM,
                            _ptr(rope_src), rope_src.stride(0) if n else ROPE_DIM, _ptr(slot_mapping), n,
                            _stream_handle(stream), _ptr(status)))


def append_fused(view: PoolView, kv_a, gamma, cos, sin, slot_mapping, eps: float = 1e-6, q_rope=None,
                 latent_out=None, rope_out=None, rstd_out=None, status=None, stream=None) -> None:
    """The producer of the appended rows in one launch: kv_a bf16 [T, >=576] ([latent | rope] per token),
    gamma bf16 [512], cos / sin bf16 [T, 64] (or [64] shared by all tokens), slot_mapping int32 [T].
    q_rope bf16 [T, heads, 64] is rotated in place; latent_out [T, 512], rope_out [T, 64] and rstd_out fp32
    [T] receive copies of what was computed."""
    n = int(slot_mapping.shape[0])
    a = ProducerArgs()
    a.pool = view
    a.kv_a, a.kv_a_stride = _ptr(kv_a), kv_a.stride(0) if n else LATENT_DIM + ROPE_DIM
    a.gamma, a.eps = _ptr(gamma), eps
    a.cos, a.cos_stride = _ptr(cos), (cos.stride(0) if cos.dim() == 2 else 0)
    a.sin, a.sin_stride = _ptr(sin), (sin.stride(0) if sin.dim() == 2 else 0)
    a.slot_mapping, a.n_tokens = _ptr(slot_mapping), n
    if q_rope is not None:
        a.q_rope, a.q_token_stride, a.q_head_stride, a.heads = _ptr(q_rope), q_rope.stride(0), q_rope.stride(1), \
            int(q_rope.shape[1])
    if latent_out is not None:
        a.latent_out, a.latent_out_stride = _ptr(latent_out), latent_out.stride(0)
    if rope_out is not None:
        a.rope_out, a.rope_out_stride = _ptr(rope_out), rope_out.stride(0)
    a.rstd_out = _ptr(rstd_out)
    check(lib.b200kv_append_fused(ctypes.byref(a), _stream_handle(stream), _ptr(status)))


def mx_quant_e4m3(x, q, scales, stream=None) -> None:
    """x bf16 [rows, cols] -> q uint8 [rows, cols] (FP8 E4M3 codes), scales uint8 [rows, cols / 32] (E8M0)."""
    rows, cols = int(x.shape[0]), int(x.shape[1])
    check(lib.b200kv_mx_quant_e4m3(_ptr(x), x.stride(0), rows, cols, _ptr(q), q.stride(0), _ptr(scales),
                                   scales.stride(0), _stream_handle(stream)))


def gather(view: PoolView, block_table, kv_len, block_size: int, out_latent, out_rope, out_row_offsets,
           total_rows: int, status=None, stream=None) -> None:
    batch = int(kv_len.shape[0])
    check(lib.b200kv_gather(ctypes.byref(view), _ptr(block_table), block_table.stride(0) if batch else 1,
                            _ptr(kv_len), batch, block_size, _ptr(out_latent),
                            out_latent.stride(0) if total_rows else LATENT_DIM, _ptr(out_rope),
                            out_rope.stride(0) if total_rows else ROPE_DIM, _ptr(out_row_offsets), total_rows,
                            _stream_handle(stream), _ptr(status)))


def indexer_topk(q_fp8, q_scale, weights, key_pool, k_scale, block_table, kv_len, block_size: int, max_kv_len: int,
                 k: int, status=None, stream=None, variant: int = INDEXER_AUTO, scores_out=None, rows_out=None):
    """The k best-scoring tokens of every sequence: q_fp8 uint8 [B, H, 128], q_scale fp32 [B, H], weights bf16
    [B, H], key_pool uint8 [rows, >=128], k_scale fp32 [rows] -> (index int32 [B, k], n_selected int32 [B]).
    variant: INDEXER_EXACT for the bit-reproducible CUDA-core scores, INDEXER_TCGEN05 for the tensor cores.
    scores_out: a list that receives the workspace as an fp32 [B, stride] tensor of the scores (for tests).
    rows_out int32 [B, k]: also receives the selection as pool rows (see resolve_rows)."""
    import torch

    batch, heads = int(q_fp8.shape[0]), int(q_fp8.shape[1])
    index = torch.empty((batch, k), dtype=torch.int32, device=q_fp8.device)
    n_sel = torch.empty((batch,), dtype=torch.int32, device=q_fp8.device)
    ws = torch.empty(lib.b200kv_indexer_workspace_bytes(batch, max_kv_len), dtype=torch.uint8, device=q_fp8.device)
    a = IndexerArgs()
    a.q, a.q_scale, a.weights, a.heads = _ptr(q_fp8), _ptr(q_scale), _ptr(weights), heads
    a.key_pool, a.key_stride, a.k_scale, a.pool_rows = _ptr(key_pool), key_pool.stride(0), _ptr(k_scale), key_pool.shape[0]
    a.block_table, a.max_blocks, a.kv_len = _ptr(block_table), block_table.shape[1], _ptr(kv_len)
    a.batch, a.block_size, a.max_kv_len, a.k = batch, block_size, max_kv_len, k
    a.index_out, a.n_selected_out, a.workspace, a.workspace_bytes = _ptr(index), _ptr(n_sel), _ptr(ws), ws.numel()
    a.variant = variant
    a.rows_out = _ptr(rows_out)
    check(lib.b200kv_indexer_topk(ctypes.byref(a), _stream_handle(stream), _ptr(status)))
    if scores_out is not None:
        stride = (max_kv_len + 3) & ~3  # the scores lie first in the workspace, [batch][stride] fp32
        scores_out.append(ws[: batch * stride * 4].view(torch.float32).view(batch, stride))
    return index, n_sel


def resolve_rows(block_table, block_size: int, token_index, n_selected, pool_rows: int, rows=None, status=None,
                 stream=None):
    """Pool rows of the selected tokens: block_table int32 [B, max_blocks], token_index int32 [B, S] (logical
    positions), n_selected int32 [B] -> rows int32 [B, S] (-1 beyond n_selected). Attend over them with
    mla_decode(q, view, rows, n_selected, 1, scale, ...)."""
    import torch

    batch, max_sel = int(token_index.shape[0]), int(token_index.shape[1])
    if rows is None:
        rows = torch.empty((batch, max_sel), dtype=torch.int32, device=token_index.device)
    check(lib.b200kv_resolve_rows(_ptr(block_table), block_table.shape[1], block_size, _ptr(token_index), max_sel,
                                  _ptr(n_selected), batch, pool_rows, _ptr(rows), _stream_handle(stream), _ptr(status)))
    return rows


def decode_workspace_bytes(batch: int, heads: int = HEADS, max_ctas: int = 0) -> int:
    return int(lib.b200kv_mla_decode_workspace_bytes(batch, heads, max_ctas))


def mla_decode(q, view: PoolView, block_table, kv_len, block_size: int, scale: float, out=None, lse=None,
               kv_begin=None, partial=None, workspace=None, variant: int = DECODE_AUTO, max_ctas: int = 0,
               status=None, stream=None, new_rows=None, stable_tables: bool = False, row_index=None, quantised=None) -> None:
    """q bf16 [B, H, 576]; out bf16 [B, H, 512]; lse fp32 [B, H]; partial = (o fp32 [B,H,512], m, l).
    new_rows = (latent bf16 [B, 512], rope bf16 [B, 64]): the append fused into the launch, each sequence's
    new row written at its position kv_len - 1 before the attention reads it. stable_tables: the block table
    and the lengths were not written by the kernel just before this call on the stream (B200KV_DECODE_STABLE_TABLES).
    row_index int32 [B, max_selected]: attend over these pool rows (kv_len = how many per sequence) instead of the
    block table, which may then be None. quantised = (fp8 uint8 [B, H, 512], scales uint8 [B, H, 16]): the output's MX
    quantisation written by the same launch."""
    args = DecodeArgs()
    args.q = _ptr(q)
    args.q_seq_stride = q.stride(0)
    args.q_head_stride = q.stride(1)
    args.pool = view
    args.block_table = _ptr(block_table)
    args.max_blocks = 0 if block_table is None else block_table.stride(0)
    if row_index is not None:
        args.row_index, args.row_index_stride = _ptr(row_index), row_index.stride(0)
    if quantised is not None:
        args.out_fp8, args.out_scale = _ptr(quantised[0]), _ptr(quantised[1])
    args.kv_len = _ptr(kv_len)
    args.kv_begin = _ptr(kv_begin)
    args.batch = q.shape[0]
    args.heads = q.shape[1]
    args.block_size = block_size
    args.scale = scale
    args.out = _ptr(out)
    args.lse = _ptr(lse)
    if partial is not None:
        args.partial_o, args.partial_m, args.partial_l = (_ptr(t) for t in partial)
    args.workspace = _ptr(workspace)
    args.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    args.variant = variant
    args.max_ctas = max_ctas
    args.flags = 1 if stable_tables else 0
    if new_rows is not None:
        new_latent, new_rope = new_rows
        args.new_latent, args.new_latent_stride = _ptr(new_latent), new_latent.stride(0)
        args.new_rope, args.new_rope_stride = _ptr(new_rope), new_rope.stride(0)
    check(lib.b200kv_mla_decode(ctypes.byref(args), _stream_handle(stream), _ptr(status)))


def _decode_args(q, view: PoolView, block_table, kv_len, block_size: int, scale: float, out=None, lse=None, kv_begin=None,
                 workspace=None, max_ctas: int = 0, stable_tables: bool = False) -> DecodeArgs:
    args = DecodeArgs()
    args.q = _ptr(q)
    args.q_seq_stride = q.stride(0)
    args.q_head_stride = q.stride(1)
    args.pool = view
    args.block_table = _ptr(block_table)
    args.max_blocks = block_table.stride(0)
    args.kv_len = _ptr(kv_len)
    args.kv_begin = _ptr(kv_begin)
    args.batch = q.shape[0]
    args.heads = q.shape[1]
    args.block_size = block_size
    args.scale = scale
    args.out = _ptr(out)
    args.lse = _ptr(lse)
    args.workspace = _ptr(workspace)
    args.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    args.max_ctas = max_ctas
    args.flags = 1 if stable_tables else 0
    return args


def mla_decode_static(q, view: PoolView, block_table, kv_len, block_size: int, scale: float, out=None, lse=None,
                      kv_begin=None, partial=None, max_ctas: int = 0, status=None, stream=None) -> None:
    """b200kv_mla_decode_static: the same attention, with the library's built-in scratch instead of a
    workspace tensor; nothing is allocated on the device by the call."""
    lib.b200kv_mla_decode_static.restype = c_int32
    lib.b200kv_mla_decode_static.argtypes = [POINTER(DecodeArgs), c_void_p, c_void_p]
    args = DecodeArgs()
    args.q = _ptr(q)
    args.q_seq_stride = q.stride(0)
    args.q_head_stride = q.stride(1)
    args.pool = view
    args.block_table = _ptr(block_table)
    args.max_blocks = block_table.stride(0)
    args.kv_len = _ptr(kv_len)
    args.kv_begin = _ptr(kv_begin)
    args.batch = q.shape[0]
    args.heads = q.shape[1]
    args.block_size = block_size
    args.scale = scale
    args.out = _ptr(out)
    args.lse = _ptr(lse)
    if partial is not None:
        args.partial_o, args.partial_m, args.partial_l = (_ptr(t) for t in partial)
    args.max_ctas = max_ctas
    check(lib.b200kv_mla_decode_static(ctypes.byref(args), _stream_handle(stream), _ptr(status)))


def lse_merge(partial_o, partial_m, partial_l, out, lse=None, stream=None) -> None:
    """partial_o fp32 [P, rows, 512], partial_m / partial_l fp32 [P, rows] -> out bf16 [rows, 512]."""
    n_parts, rows = int(partial_m.shape[0]), int(partial_m.shape[1])
    check(lib.b200kv_lse_merge(_ptr(partial_o), _ptr(partial_m), _ptr(partial_l), n_parts, rows, _ptr(out),
                               _ptr(lse), _stream_handle(stream)))


def fill_normal_bf16(dst, seed: int, stream_id: int, first_element: int = 0, scale: float = 1.0, stream=None) -> None:
    check(lib.b200kv_fill_normal_bf16(_ptr(dst), dst.numel(), seed, stream_id, first_element, scale,
                                      _stream_handle(stream)))


# ---------------------------------------------------------------------------------------------------
# Host bookkeeping
# ---------------------------------------------------------------------------------------------------
class BlockPool:
    """KV block allocator: FIFO free list, per-sequence block tables (include/b200kv.h)."""

    def __init__(self, num_blocks: int, block_size: int, max_seqs: int, max_blocks_per_seq: int, free_order=None):
        import numpy as np

        order = None
        if free_order is not None:
            order = np.ascontiguousarray(free_order, dtype=np.int32)
            assert order.shape == (num_blocks,)
        self._h = lib.b200kv_block_pool_create(num_blocks, block_size, max_seqs, max_blocks_per_seq,
                                               None if order is None else order.ctypes.data)
        if not self._h:
            raise B200KVError(ERR_INVALID, last_error())
        self.num_blocks, self.block_size = num_blocks, block_size
        self.max_seqs, self.max_blocks_per_seq = max_seqs, max_blocks_per_seq

    def close(self) -> None:
        if self._h:
            lib.b200kv_block_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def admit(self, seq: int) -> None:
        check(lib.b200kv_block_pool_admit(self._h, seq))

    def grow(self, seq: int, n_tokens: int):
        import numpy as np

        slots = np.empty(max(n_tokens, 1), dtype=np.int32)
        check(lib.b200kv_block_pool_grow(self._h, seq, n_tokens, slots.ctypes.data))
        return slots[:n_tokens]

    def release(self, seq: int) -> None:
        check(lib.b200kv_block_pool_release(self._h, seq))

    def validate(self) -> None:
        check(lib.b200kv_block_pool_validate(self._h))

    @property
    def free_count(self) -> int:
        return int(lib.b200kv_block_pool_free_count(self._h))

    def seq_len(self, seq: int) -> int:
        return int(lib.b200kv_block_pool_seq_len(self._h, seq))

    def table(self):
        import numpy as np

        ptr = lib.b200kv_block_pool_table(self._h)
        return np.ctypeslib.as_array(ptr, shape=(self.max_seqs, self.max_blocks_per_seq)).copy()

    def lens(self):
        import numpy as np

        ptr = lib.b200kv_block_pool_lens(self._h)
        return np.ctypeslib.as_array(ptr, shape=(self.max_seqs,)).copy()

    def free_list(self):
        import numpy as np

        out = np.empty(self.num_blocks, dtype=np.int32)
        n = lib.b200kv_block_pool_export_free(self._h, out.ctypes.data, self.num_blocks)
        return out[:n].copy()


class KvCache(Structure):
    _fields_ = [
        ("geometry", Reservation),
        ("layers", c_int64),
        ("block_size", c_int64),
        ("max_seqs", c_int64),
        ("block_table_handle", c_int64),
        ("slot_mapping_handle", c_int64),
        ("latent_handle", c_int64),
        ("rope_handle", c_int64),
        ("max_blocks_per_seq", c_int64),
        ("seq_lens_handle", c_int64),
    ]


ARENA_DEVICE, ARENA_HOST_SIM = 0, 1


class Arena:
    """Three-phase static arena (reserve -> commit -> seal) behind the C ABI."""

    def __init__(self, backend: int = ARENA_DEVICE):
        lib.b200kv_arena_create.restype = c_void_p
        lib.b200kv_arena_create.argtypes = [c_int32]
        lib.b200kv_arena_destroy.argtypes = [c_void_p]
        lib.b200kv_arena_destroy.restype = None
        lib.b200kv_arena_reserve.restype = c_int64
        lib.b200kv_arena_reserve.argtypes = [c_void_p, c_char_p, c_size_t, c_size_t]
        lib.b200kv_arena_address.restype = c_void_p
        lib.b200kv_arena_address.argtypes = [c_void_p, c_int64]
        lib.b200kv_arena_offset.restype = c_int64
        lib.b200kv_arena_offset.argtypes = [c_void_p, c_int64]
        for name in ("reserved_bytes", "bytes"):
            fn = getattr(lib, f"b200kv_arena_{name}")
            fn.restype = c_size_t
            fn.argtypes = [c_void_p]
        for name in ("commit", "allocations", "commit_workspace", "seal", "sealed", "validate"):
            fn = getattr(lib, f"b200kv_arena_{name}")
            fn.restype = c_int32
            fn.argtypes = [c_void_p]
        lib.b200kv_arena_note_workspace.restype = c_int32
        lib.b200kv_arena_note_workspace.argtypes = [c_void_p, c_uint64]
        lib.b200kv_arena_workspace_fits.restype = c_int32
        lib.b200kv_arena_workspace_fits.argtypes = [c_void_p, c_uint64]
        lib.b200kv_arena_workspace.restype = c_void_p
        lib.b200kv_arena_workspace.argtypes = [c_void_p]
        lib.b200kv_arena_workspace_bytes.restype = c_uint64
        lib.b200kv_arena_workspace_bytes.argtypes = [c_void_p]
        lib.b200kv_kv_cache_reserve.restype = c_int32
        lib.b200kv_kv_cache_reserve.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                POINTER(KvCache)]
        lib.b200kv_kv_cache_layer_view.restype = c_int32
        lib.b200kv_kv_cache_layer_view.argtypes = [c_void_p, POINTER(KvCache), c_int64, POINTER(PoolView)]
        self._h = lib.b200kv_arena_create(backend)
        if not self._h:
            raise B200KVError(ERR_INVALID, last_error())

    def close(self):
        if self._h and lib is not None:  # (the module may already be gone at interpreter exit)
            lib.b200kv_arena_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def reserve(self, name: str, nbytes: int, align: int = 0) -> int:
        handle = int(lib.b200kv_arena_reserve(self._h, name.encode(), nbytes, align))
        if handle < 0:
            raise B200KVError(-handle, last_error())
        return handle

    def commit(self):
        check(lib.b200kv_arena_commit(self._h))

    def address(self, handle: int) -> int:
        addr = lib.b200kv_arena_address(self._h, handle)
        if not addr:
            raise B200KVError(ERR_INVALID, last_error())
        return int(addr)

    def offset(self, handle: int) -> int:
        return int(lib.b200kv_arena_offset(self._h, handle))

    @property
    def reserved_bytes(self) -> int:
        return int(lib.b200kv_arena_reserved_bytes(self._h))

    @property
    def nbytes(self) -> int:
        return int(lib.b200kv_arena_bytes(self._h))

    @property
    def allocations(self) -> int:
        return int(lib.b200kv_arena_allocations(self._h))

    def note_workspace(self, nbytes: int):
        check(lib.b200kv_arena_note_workspace(self._h, nbytes))

    def commit_workspace(self):
        check(lib.b200kv_arena_commit_workspace(self._h))

    @property
    def workspace(self) -> int:
        return int(lib.b200kv_arena_workspace(self._h) or 0)

    @property
    def workspace_bytes(self) -> int:
        return int(lib.b200kv_arena_workspace_bytes(self._h))

    def workspace_fits(self, nbytes: int):
        check(lib.b200kv_arena_workspace_fits(self._h, nbytes))

    def seal(self):
        check(lib.b200kv_arena_seal(self._h))

    @property
    def sealed(self) -> bool:
        return bool(lib.b200kv_arena_sealed(self._h))

    def validate(self):
        check(lib.b200kv_arena_validate(self._h))

    def reserve_kv_cache(self, max_context: int, block_size: int, layers: int = 43, max_seqs: int = 1,
                         tokens_per_step: int = 1) -> KvCache:
        cache = KvCache()
        check(lib.b200kv_kv_cache_reserve(self._h, max_context, block_size, layers, max_seqs, tokens_per_step,
                                          ctypes.byref(cache)))
        return cache

    def reserve_kv_cache_batched(self, num_blocks: int, block_size: int, layers: int, max_seqs: int,
                                 max_blocks_per_seq: int, tokens_per_step: int) -> KvCache:
        lib.b200kv_kv_cache_reserve_batched.restype = c_int32
        lib.b200kv_kv_cache_reserve_batched.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                        POINTER(KvCache)]
        cache = KvCache()
        check(lib.b200kv_kv_cache_reserve_batched(self._h, num_blocks, block_size, layers, max_seqs, max_blocks_per_seq,
                                                  tokens_per_step, ctypes.byref(cache)))
        return cache

    def tensor(self, handle: int, shape, dtype):
        """The committed span `handle` (or an address) as a torch tensor over the arena's memory, no copy."""
        return device_tensor(self.address(handle), shape, dtype)

    def layer_view(self, cache: KvCache, layer: int) -> PoolView:
        view = PoolView()
        check(lib.b200kv_kv_cache_layer_view(self._h, ctypes.byref(cache), layer, ctypes.byref(view)))
        return view


class EngineConfig(Structure):
    """b200kv_engine_config (include/b200kv.h)."""

    _fields_ = [("layers", c_int32), ("max_seqs", c_int32), ("num_blocks", c_int32), ("block_size", c_int32),
                ("max_blocks_per_seq", c_int32), ("max_step_tokens", c_int32), ("scale", c_float), ("eps", c_float),
                ("backend", c_int32)]


class Engine:
    """The KV path as the engine drives it, batched (b200kv_engine_*): Build once, then per step begin_step, per
    layer layer_append / layer_attend, end_step. Device tensors are torch tensors; nothing here allocates them."""

    def __init__(self, layers: int, max_seqs: int, num_blocks: int, block_size: int, max_blocks_per_seq: int,
                 max_step_tokens: int, scale: float, eps: float = 1e-6, backend: int = 0):
        lib.b200kv_engine_create.restype = c_void_p
        lib.b200kv_engine_create.argtypes = [POINTER(EngineConfig)]
        lib.b200kv_engine_destroy.restype = None
        lib.b200kv_engine_destroy.argtypes = [c_void_p]
        for name in ("arena", "cache", "block_pool", "status"):
            fn = getattr(lib, f"b200kv_engine_{name}")
            fn.restype = c_void_p
            fn.argtypes = [c_void_p]
        for name in ("admit", "release"):
            fn = getattr(lib, f"b200kv_engine_{name}")
            fn.restype = c_int32
            fn.argtypes = [c_void_p, c_int32]
        lib.b200kv_engine_begin_step.restype = c_int32
        lib.b200kv_engine_begin_step.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_void_p]
        lib.b200kv_engine_layer_append.restype = c_int32
        lib.b200kv_engine_layer_append.argtypes = [c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                                   c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p]
        lib.b200kv_engine_layer_attend.restype = c_int32
        lib.b200kv_engine_layer_attend.argtypes = [c_void_p, c_int32, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                                   c_void_p, c_void_p]
        lib.b200kv_engine_end_step.restype = c_int32
        lib.b200kv_engine_end_step.argtypes = [c_void_p]
        lib.b200kv_engine_stats_json.restype = c_int64
        lib.b200kv_engine_stats_json.argtypes = [c_void_p, c_char_p, c_int64]
        lib.b200kv_arena_allocations.restype = c_int32
        lib.b200kv_arena_allocations.argtypes = [c_void_p]
        lib.b200kv_arena_address.restype = c_void_p
        lib.b200kv_arena_address.argtypes = [c_void_p, c_int64]
        lib.b200kv_arena_sealed.restype = c_int32
        lib.b200kv_arena_sealed.argtypes = [c_void_p]
        self.config = EngineConfig(layers, max_seqs, num_blocks, block_size, max_blocks_per_seq, max_step_tokens, scale,
                                   eps, backend)
        self._h = lib.b200kv_engine_create(ctypes.byref(self.config))
        if not self._h:
            raise B200KVError(ERR_INVALID, last_error())

    def close(self):
        if self._h and lib is not None:
            lib.b200kv_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    @property
    def cache(self) -> KvCache:
        return ctypes.cast(lib.b200kv_engine_cache(self._h), POINTER(KvCache)).contents

    @property
    def allocations(self) -> int:
        return int(lib.b200kv_arena_allocations(lib.b200kv_engine_arena(self._h)))

    @property
    def sealed(self) -> bool:
        return bool(lib.b200kv_arena_sealed(lib.b200kv_engine_arena(self._h)))

    def span_address(self, handle: int) -> int:
        return int(lib.b200kv_arena_address(lib.b200kv_engine_arena(self._h), handle))

    def admit(self, seq: int):
        check(lib.b200kv_engine_admit(self._h, seq))

    def release(self, seq: int):
        check(lib.b200kv_engine_release(self._h, seq))

    def seq_len(self, seq: int) -> int:
        return int(lib.b200kv_block_pool_seq_len(lib.b200kv_engine_block_pool(self._h), seq))

    def table(self):
        import numpy as np

        ptr = lib.b200kv_block_pool_table(lib.b200kv_engine_block_pool(self._h))
        c = self.config
        return np.ctypeslib.as_array(ptr, shape=(c.max_seqs, c.max_blocks_per_seq)).copy()

    def begin_step(self, seqs, new_tokens=None, stream=None):
        import numpy as np

        ids = np.ascontiguousarray(seqs, dtype=np.int32)
        grow = None if new_tokens is None else np.ascontiguousarray(new_tokens, dtype=np.int32)
        check(lib.b200kv_engine_begin_step(self._h, ids.ctypes.data, None if grow is None else grow.ctypes.data, len(ids),
                                           _stream_handle(stream) if self.config.backend == 0 else None))

    def layer_append(self, layer: int, kv_a, gamma, cos, sin, q_rope=None, stream=None):
        check(lib.b200kv_engine_layer_append(
            self._h, layer, _ptr(kv_a), kv_a.stride(0), _ptr(gamma), _ptr(cos), cos.stride(0) if cos.dim() == 2 else 0,
            _ptr(sin), sin.stride(0) if sin.dim() == 2 else 0, _ptr(q_rope),
            0 if q_rope is None else q_rope.stride(0), 0 if q_rope is None else q_rope.stride(1), _stream_handle(stream)))

    def layer_attend(self, layer: int, q, out, out_fp8=None, out_scales=None, stream=None):
        check(lib.b200kv_engine_layer_attend(self._h, layer, _ptr(q), q.stride(0), q.stride(1), _ptr(out), _ptr(out_fp8),
                                             _ptr(out_scales), _stream_handle(stream)))

    def end_step(self):
        check(lib.b200kv_engine_end_step(self._h))

    def abort_step(self):
        lib.b200kv_engine_abort_step.restype = c_int32
        lib.b200kv_engine_abort_step.argtypes = [c_void_p]
        check(lib.b200kv_engine_abort_step(self._h))

    def free_list(self):
        import numpy as np

        pool = lib.b200kv_engine_block_pool(self._h)
        out = np.empty(self.config.num_blocks, dtype=np.int32)
        n = lib.b200kv_block_pool_export_free(pool, out.ctypes.data, self.config.num_blocks)
        return out[:n].copy()

    def status(self):
        """The engine's device status word as a tensor over the arena."""
        import torch

        return device_tensor(int(lib.b200kv_engine_status(self._h)), (4,), torch.int32)

    def stats_json(self) -> str:
        buf = ctypes.create_string_buffer(512)
        lib.b200kv_engine_stats_json(self._h, buf, 512)
        return buf.value.decode()


class _RawDeviceMemory:
    """Memory someone else owns, described for torch through the CUDA array interface."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


def device_tensor(address: int, shape, dtype):
    """A torch tensor of `shape` and `dtype` over device memory at `address` that the caller keeps alive (an
    arena span, an arena workspace). Nothing is allocated or copied."""
    import math

    import torch

    count = math.prod(shape)
    nbytes = count * torch.empty((), dtype=dtype).element_size()
    if nbytes == 0:
        return torch.empty(shape, dtype=dtype, device="cuda")
    raw = torch.as_tensor(_RawDeviceMemory(address, nbytes), device="cuda")
    return raw.view(dtype).view(*shape)


def plan_reservation(max_context: int, block_size: int, layers: int = 43, max_seqs: int = 1,
                     tokens_per_step: int = 1) -> Reservation:
    out = Reservation()
    check(lib.b200kv_plan_reservation(max_context, block_size, layers, max_seqs, tokens_per_step, ctypes.byref(out)))
    return out


def utilisation(active_tokens: int, blocks_per_layer: int, block_size: int) -> float:
    return float(lib.b200kv_utilisation(active_tokens, blocks_per_layer, block_size))
