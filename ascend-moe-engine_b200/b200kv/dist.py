"""Multi-GPU plumbing for the two ways the path shards (one process per GPU, torch.distributed).

Batched decode partitions whole sequences over ranks and needs no collective on the data path. A single
long sequence is split by KV range: each rank attends over its block range, the per-rank partial
(m, l, O) triples are all-gathered, and every rank merges them with the log-sum-exp reduction.
The partition arithmetic is the C library's (b200kv_partition_sequences, b200kv_split_kv_range).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int32, c_int64, c_void_p

import numpy as np

from . import check, lib, lse_merge

lib.b200kv_partition_sequences.restype = c_int32
lib.b200kv_partition_sequences.argtypes = [c_void_p, c_int32, c_int32, c_void_p, c_void_p]
lib.b200kv_split_kv_range.restype = c_int32
lib.b200kv_split_kv_range.argtypes = [c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]


def partition_sequences(kv_len, n_ranks: int):
    """Returns (rank_of_seq int32 [n], tokens_per_rank int64 [n_ranks])."""
    lens = np.ascontiguousarray(kv_len, dtype=np.int32)
    ranks = np.empty(len(lens), dtype=np.int32)
    loads = np.zeros(n_ranks, dtype=np.int64)
    check(lib.b200kv_partition_sequences(lens.ctypes.data, len(lens), n_ranks, ranks.ctypes.data, loads.ctypes.data))
    return ranks, loads


def split_kv_range(kv_len: int, block_size: int, n_ranks: int, rank: int):
    """Returns (begin, length) of `rank`'s contiguous block range of a kv_len-token sequence."""
    begin, length = c_int32(), c_int32()
    check(lib.b200kv_split_kv_range(kv_len, block_size, n_ranks, rank, ctypes.byref(begin), ctypes.byref(length)))
    return int(begin.value), int(length.value)


def all_gather_partials(partial_o, partial_m, partial_l, group=None):
    """All-gathers one rank's partial (o [rows,512] fp32, m [rows], l [rows]) into stacked
    ([world, rows, 512], [world, rows], [world, rows]) tensors on every rank. One collective moves all
    three: they travel as a single [rows, 514] buffer per rank (131,584 bytes at 64 rows)."""
    import torch
    import torch.distributed as dist

    rows = partial_m.numel()
    packed = torch.cat([partial_o.reshape(rows, -1), partial_m.reshape(rows, 1), partial_l.reshape(rows, 1)], dim=1)
    world = dist.get_world_size(group)
    flat = torch.empty((world * rows, packed.shape[1]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed.contiguous(), group=group)
    gathered = flat.view(world, rows, packed.shape[1])
    width = partial_o.reshape(rows, -1).shape[1]
    return gathered[:, :, :width].contiguous(), gathered[:, :, width].contiguous(), gathered[:, :, width + 1].contiguous()


def merge_across_ranks(partial_o, partial_m, partial_l, out, lse=None, group=None, stream=None):
    """KV-range split epilogue on the device: all-gather (NCCL) then the LSE merge kernel; every rank
    ends with the full result in `out` (bf16 [rows, 512]) and `lse`."""
    o, m, l = all_gather_partials(partial_o, partial_m, partial_l, group)
    lse_merge(o, m, l, out, lse, stream=stream)
    return out


lib.b200kv_peer_exchange_bytes.restype = ctypes.c_size_t
lib.b200kv_peer_exchange_bytes.argtypes = [c_int32, c_int64]
lib.b200kv_peer_buffer_alloc.restype = c_int32
lib.b200kv_peer_buffer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(c_void_p), c_void_p]
lib.b200kv_peer_buffer_open.restype = c_int32
lib.b200kv_peer_buffer_open.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
lib.b200kv_peer_buffer_close.restype = c_int32
lib.b200kv_peer_buffer_close.argtypes = [c_void_p]
lib.b200kv_peer_buffer_free.restype = c_int32
lib.b200kv_peer_buffer_free.argtypes = [c_void_p]
lib.b200kv_mla_decode_peer.restype = c_int32
lib.b200kv_mla_decode_peer.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p]
lib.b200kv_peer_merge.restype = c_int32
lib.b200kv_peer_merge.argtypes = [c_void_p, c_int32, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p]


class PeerExchange:
    """The KV-range split epilogue over peer memory (b200kv_peer_merge): every rank pushes its partials into
    all ranks' exchange buffers over NVLink and merges what arrives in its own; no collective on the data
    path. Construction is collective (the 64-byte memory handles are all-gathered once); `merge` is then a
    pair of kernel launches on the caller's stream and may be captured in a CUDA graph."""

    def __init__(self, rows: int, group=None):
        import torch.distributed as dist

        self.rows = int(rows)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        nbytes = lib.b200kv_peer_exchange_bytes(self.world, self.rows)
        if nbytes == 0:
            raise ValueError(f"peer exchange of {self.world} ranks x {self.rows} rows is not supported")
        own = c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.b200kv_peer_buffer_alloc(nbytes, ctypes.byref(own), handle))
        self._own = own
        handles = [bytes(handle)]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
        self._opened = []
        table = (c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                table[r] = own.value
                continue
            mapped = c_void_p()
            raw = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
            check(lib.b200kv_peer_buffer_open(raw, ctypes.byref(mapped)))
            self._opened.append(mapped)
            table[r] = mapped.value
        self._table = table
        if self.world > 1:
            dist.barrier(group=group)  # every rank has mapped every buffer before anyone pushes

    def merge(self, partial_o, partial_m, partial_l, out, lse=None, status=None, stream=None):
        """partial_o fp32 [rows, 512], partial_m / partial_l fp32 [rows] of this rank's shard -> out bf16
        [rows, 512] (and lse fp32 [rows]) of the whole sequence, on every rank."""
        from . import _ptr, _stream_handle

        check(lib.b200kv_peer_merge(self._table, self.world, self.rank, self.rows, _ptr(partial_o), _ptr(partial_m),
                                    _ptr(partial_l), _ptr(out), _ptr(lse), _stream_handle(stream), _ptr(status)))
        return out

    def decode_merge(self, q, view, block_table, kv_len, block_size: int, scale: float, out, lse=None, kv_begin=None,
                     workspace=None, max_ctas: int = 0, status=None, stream=None, stable_tables: bool = False):
        """b200kv_mla_decode_peer: attention over this rank's shard (kv_begin / kv_len) and the merge across the
        ranks in one call; q bf16 [B, 64, 576] with B * 64 == rows, out bf16 [B, 64, 512] on every rank."""
        from . import _decode_args, _ptr, _stream_handle

        args = _decode_args(q, view, block_table, kv_len, block_size, scale, out=out, lse=lse, kv_begin=kv_begin,
                            workspace=workspace, max_ctas=max_ctas, stable_tables=stable_tables)
        check(lib.b200kv_mla_decode_peer(ctypes.byref(args), self._table, self.world, self.rank,
                                         _stream_handle(stream), _ptr(status)))
        return out

    def close(self):
        """Collective in spirit: call it on every rank once no rank can still be pushing."""
        for mapped in self._opened:
            lib.b200kv_peer_buffer_close(mapped)
        self._opened = []
        if self._own is not None:
            lib.b200kv_peer_buffer_free(self._own)
            self._own = None
