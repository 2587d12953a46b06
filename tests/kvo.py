"""Loader and numpy-facing wrappers for the CPU oracle (oracle/kv_oracle.cpp).

Test infrastructure only. The oracle is compiled -march=native, so one build is kept per host CPU
(keyed by the CPU flags) and rebuilt when the source changes.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
from ctypes import c_double, c_float, c_int32, c_int64, c_uint64, c_void_p

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

LATENT, ROPE, ROW, HEADS = 512, 64, 576, 64
BASE_SEED = 20251008
STREAM_KV, STREAM_Q, STREAM_NEW, STREAM_PERM, STREAM_LEN, STREAM_CHURN = 1, 2, 3, 4, 5, 6


def _cpu_key() -> str:
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:12]


def build() -> str:
    """Builds (or finds up to date) the oracle for this host's CPU. Several processes may call this at once
    (one per rank of a multi-GPU run): the build runs under an exclusive file lock, so none of them loads a
    library that another is still writing."""
    import fcntl

    build_dir = os.path.join("_build", _cpu_key())
    os.makedirs(os.path.join(ORACLE_DIR, "_build"), exist_ok=True)
    with open(os.path.join(ORACLE_DIR, "_build", ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            res = subprocess.run(["make", "-s", f"BUILD_DIR={build_dir}"], cwd=ORACLE_DIR, capture_output=True, text=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + res.stdout + res.stderr)
    return os.path.join(ORACLE_DIR, build_dir, "libkv_oracle.so")


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        L.kvo_fill_normal_bf16.argtypes = [c_void_p, c_int64, c_uint64, c_uint64, c_uint64, c_double]
        L.kvo_draw_u64.argtypes = [c_void_p, c_int64, c_uint64, c_uint64, c_uint64]
        L.kvo_permutation.argtypes = [c_void_p, c_int32, c_uint64, c_uint64]
        L.kvo_f32_to_bf16.argtypes = [c_void_p, c_void_p, c_int64]
        L.kvo_bf16_to_f32.argtypes = [c_void_p, c_void_p, c_int64]
        L.kvo_blocks_per_layer.restype = c_int64
        L.kvo_blocks_per_layer.argtypes = [c_int64, c_int64]
        L.kvo_total_blocks.restype = c_int64
        L.kvo_total_blocks.argtypes = [c_int64, c_int64, c_int64]
        L.kvo_utilisation.restype = c_double
        L.kvo_utilisation.argtypes = [c_int64, c_int64, c_int64]
        L.kvo_pool_bytes.argtypes = [c_int64] * 5 + [c_void_p, c_void_p]
        L.kvo_append.restype = c_int64
        L.kvo_append.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                 c_int64, c_int64, c_int64, c_int64]
        L.kvo_gather.restype = c_int64
        L.kvo_gather.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                 c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64]
        L.kvo_mla_decode.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                     c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                     c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        L.kvo_rmsnorm512.argtypes = [c_void_p, c_int64, c_void_p, c_float, c_int64, c_void_p, c_int64, c_void_p]
        L.kvo_rope_half64.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                      c_void_p, c_int64, c_int64]
        L.kvo_append_fused.restype = c_int64
        L.kvo_append_fused.argtypes = [c_void_p, c_int64, c_void_p, c_float, c_void_p, c_int64, c_void_p, c_int64,
                                       c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64]
        L.kvo_mx_quant_e4m3.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        L.kvo_f32_to_e4m3.restype = ctypes.c_uint8
        L.kvo_f32_to_e4m3.argtypes = [c_float]
        L.kvo_indexer_scores.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p,
                                         c_int64, c_void_p, c_int32, c_int32, c_void_p, c_int64]
        L.kvo_topk_tokens.argtypes = [c_void_p, c_int64, c_void_p, c_int32, c_int32, c_void_p, c_void_p]
        L.kvo_lse_merge.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]
        L.kvo_num_threads.restype = c_int32
        L.kvo_set_num_threads.argtypes = [c_int32]
        L.kvo_book_create.restype = c_void_p
        L.kvo_book_create.argtypes = [c_int32, c_int32, c_int32, c_int32, c_void_p]
        L.kvo_book_destroy.argtypes = [c_void_p]
        L.kvo_book_admit.argtypes = [c_void_p, c_int32]
        L.kvo_book_grow.argtypes = [c_void_p, c_int32, c_int32, c_void_p]
        L.kvo_book_release.argtypes = [c_void_p, c_int32]
        L.kvo_book_free_count.argtypes = [c_void_p]
        L.kvo_book_export.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


# ---- generators -------------------------------------------------------------------------------------
def normal_bf16(count: int, stream: int, first: int = 0, scale: float = 1.0, seed: int = BASE_SEED) -> np.ndarray:
    """bf16 bit patterns (uint16) of scale*N(0,1) for element counters first..first+count-1."""
    out = np.empty(count, dtype=np.uint16)
    lib().kvo_fill_normal_bf16(_p(out), count, seed, stream, first, scale)
    return out


def draws(count: int, stream: int, first: int = 0, seed: int = BASE_SEED) -> np.ndarray:
    out = np.empty(count, dtype=np.uint64)
    lib().kvo_draw_u64(_p(out), count, seed, stream, first)
    return out


def permutation(count: int, stream: int = STREAM_PERM, seed: int = BASE_SEED) -> np.ndarray:
    out = np.empty(count, dtype=np.int32)
    lib().kvo_permutation(_p(out), count, seed, stream)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().kvo_f32_to_bf16(_p(a), _p(out), a.size)
    return out


# ---- the path -------------------------------------------------------------------------------------------
def append(pool: np.ndarray, latent_src: np.ndarray, rope_src: np.ndarray, slots: np.ndarray,
           rope_pool: np.ndarray | None = None) -> int:
    """pool: uint16 [rows, 576] fused rows (rope_pool None) or [rows, 512] + rope_pool [rows, 64]. In place."""
    assert pool.dtype == np.uint16 and pool.flags.c_contiguous
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    if rope_pool is None:
        rp, rs = pool.ctypes.data + LATENT * 2, pool.shape[1]
    else:
        rp, rs = rope_pool.ctypes.data, rope_pool.shape[1]
    return int(lib().kvo_append(_p(latent_src), latent_src.strides[0] // 2, _p(rope_src), rope_src.strides[0] // 2,
                                _p(pool), pool.shape[1], rp, rs, _p(slots), len(slots), pool.shape[0], LATENT, ROPE))


def gather(pool: np.ndarray, block_table: np.ndarray, kv_len: np.ndarray, block_size: int,
           rope_pool: np.ndarray | None = None):
    """Returns (latent uint16 [sum len, 512], rope uint16 [sum len, 64], row offsets int64 [B])."""
    block_table = np.ascontiguousarray(block_table, dtype=np.int32)
    kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
    offsets = np.zeros(len(kv_len), dtype=np.int64)
    offsets[1:] = np.cumsum(kv_len[:-1])
    total = int(kv_len.sum())
    out_l = np.zeros((total, LATENT), dtype=np.uint16)
    out_r = np.zeros((total, ROPE), dtype=np.uint16)
    if rope_pool is None:
        rp, rs = pool.ctypes.data + LATENT * 2, pool.shape[1]
    else:
        rp, rs = rope_pool.ctypes.data, rope_pool.shape[1]
    bad = lib().kvo_gather(_p(pool), pool.shape[1], rp, rs, pool.shape[0], _p(block_table), block_table.shape[1],
                           _p(kv_len), len(kv_len), block_size, _p(out_l), LATENT, _p(out_r), ROPE, _p(offsets),
                           LATENT, ROPE)
    assert bad == 0
    return out_l, out_r, offsets


def mla_decode(q: np.ndarray, pool: np.ndarray, block_table: np.ndarray, kv_len: np.ndarray, block_size: int,
               scale: float, kv_begin: np.ndarray | None = None, use_double: bool = False, partial: bool = False,
               rope_pool: np.ndarray | None = None):
    """q uint16 [B, H, 576]. Returns (out uint16 [B,H,512], lse f32 [B,H]) or with partial=True
    (o f32 [B,H,512], m f32 [B,H], l f32 [B,H])."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    block_table = np.ascontiguousarray(block_table, dtype=np.int32)
    kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
    if kv_begin is not None:
        kv_begin = np.ascontiguousarray(kv_begin, dtype=np.int32)
    B, H = q.shape[0], q.shape[1]
    out = np.zeros((B, H, LATENT), dtype=np.uint16)
    lse = np.zeros((B, H), dtype=np.float32)
    po = np.zeros((B, H, LATENT), dtype=np.float32) if partial else None
    pm = np.zeros((B, H), dtype=np.float32) if partial else None
    pl = np.zeros((B, H), dtype=np.float32) if partial else None
    if rope_pool is None:
        rp, rs = pool.ctypes.data + LATENT * 2, pool.shape[1]
    else:
        rp, rs = rope_pool.ctypes.data, rope_pool.shape[1]
    lib().kvo_mla_decode(_p(q), H * ROW, ROW, _p(pool), pool.shape[1], rp, rs, _p(block_table), block_table.shape[1],
                         _p(kv_len), _p(kv_begin), B, H, block_size, LATENT, ROPE, scale, int(use_double), _p(out),
                         _p(lse), _p(po), _p(pm), _p(pl))
    if partial:
        return po, pm, pl
    return out, lse


def lse_merge(po: np.ndarray, pm: np.ndarray, pl: np.ndarray):
    """po f32 [P, rows, 512], pm/pl f32 [P, rows] -> (out uint16 [rows,512], lse f32 [rows])."""
    po = np.ascontiguousarray(po, dtype=np.float32)
    pm = np.ascontiguousarray(pm, dtype=np.float32)
    pl = np.ascontiguousarray(pl, dtype=np.float32)
    parts, rows = pm.shape
    out = np.zeros((rows, LATENT), dtype=np.uint16)
    lse = np.zeros(rows, dtype=np.float32)
    lib().kvo_lse_merge(_p(po), _p(pm), _p(pl), parts, rows, LATENT, _p(out), _p(lse))
    return out, lse


class Book:
    """The bookkeeping model (free-list FIFO, tables) of the oracle."""

    def __init__(self, num_blocks, block_size, max_seqs, max_blocks_per_seq, free_order=None):
        order = None if free_order is None else np.ascontiguousarray(free_order, dtype=np.int32)
        self._h = lib().kvo_book_create(num_blocks, block_size, max_seqs, max_blocks_per_seq, _p(order))
        self.num_blocks, self.max_seqs, self.max_blocks_per_seq = num_blocks, max_seqs, max_blocks_per_seq

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvo_book_destroy(self._h)
            self._h = None

    def admit(self, seq):
        return lib().kvo_book_admit(self._h, seq)

    def grow(self, seq, n):
        slots = np.empty(max(n, 1), dtype=np.int32)
        rc = lib().kvo_book_grow(self._h, seq, n, _p(slots))
        return rc, slots[:n]

    def release(self, seq):
        return lib().kvo_book_release(self._h, seq)

    @property
    def free_count(self):
        return lib().kvo_book_free_count(self._h)

    def export(self):
        table = np.zeros((self.max_seqs, self.max_blocks_per_seq), dtype=np.int32)
        lens = np.zeros(self.max_seqs, dtype=np.int32)
        free = np.zeros(self.num_blocks, dtype=np.int32)
        lib().kvo_book_export(self._h, _p(table), _p(lens), _p(free))
        return table, lens, free[: self.free_count]


# ---- scenario builders shared by tests and the benchmark's checks -----------------------------------------
def make_pool(rows: int, stream: int = STREAM_KV, seed: int = BASE_SEED) -> np.ndarray:
    return normal_bf16(rows * ROW, stream, 0, 1.0, seed).reshape(rows, ROW)


def make_q(batch: int, heads: int = HEADS, scale: float = 1.0 / 24.0, seed: int = BASE_SEED) -> np.ndarray:
    return normal_bf16(batch * heads * ROW, STREAM_Q, 0, scale, seed).reshape(batch, heads, ROW)


def rmsnorm512(x: np.ndarray, gamma: np.ndarray, eps: float = 1e-6):
    """x uint16 [T, >=512] (bf16 bits), gamma uint16 [512] -> (y uint16 [T, 512], rstd float32 [T])."""
    x = np.ascontiguousarray(x)
    y = np.empty((x.shape[0], 512), dtype=np.uint16)
    rstd = np.empty(x.shape[0], dtype=np.float32)
    lib().kvo_rmsnorm512(_p(x), x.shape[1], _p(np.ascontiguousarray(gamma)), eps, x.shape[0], _p(y), 512, _p(rstd))
    return y, rstd


def rope_half64(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x uint16 [T, V, 64], cos / sin uint16 [T, 64] -> rotated uint16 [T, V, 64]."""
    x = np.ascontiguousarray(x)
    cos, sin = np.ascontiguousarray(cos), np.ascontiguousarray(sin)
    y = np.empty_like(x)
    T, V, _ = x.shape
    lib().kvo_rope_half64(_p(x), V * 64, 64, _p(cos), 64, _p(sin), 64, T, V, _p(y), V * 64, 64)
    return y


def append_fused(pool: np.ndarray, kv_a: np.ndarray, gamma: np.ndarray, cos: np.ndarray, sin: np.ndarray,
                 slots: np.ndarray, eps: float = 1e-6) -> int:
    """Normalises, rotates and writes rows of kv_a uint16 [T, 576] into pool uint16 [rows, 576] in place;
    returns the number of slots outside the pool."""
    kv_a = np.ascontiguousarray(kv_a)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    cos, sin = np.ascontiguousarray(cos), np.ascontiguousarray(sin)
    base = pool.ctypes.data
    return int(lib().kvo_append_fused(_p(kv_a), kv_a.shape[1], _p(np.ascontiguousarray(gamma)), eps, _p(cos), 64,
                                      _p(sin), 64, _p(slots), kv_a.shape[0], base, pool.shape[1],
                                      base + 2 * LATENT, pool.shape[1], pool.shape[0]))


def mx_quant_e4m3(x: np.ndarray):
    """x uint16 [rows, cols] (bf16 bits, cols % 32 == 0) -> (q uint8 [rows, cols], scales uint8 [rows, cols/32])."""
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    q = np.empty((rows, cols), dtype=np.uint8)
    scales = np.empty((rows, cols // 32), dtype=np.uint8)
    lib().kvo_mx_quant_e4m3(_p(x), cols, rows, cols, _p(q), cols, _p(scales), cols // 32)
    return q, scales


def indexer_topk(q_fp8: np.ndarray, q_scale: np.ndarray, weights: np.ndarray, key_pool: np.ndarray, k_scale: np.ndarray,
                 block_table: np.ndarray, kv_len: np.ndarray, block_size: int, k: int):
    """q_fp8 uint8 [B, H, 128], q_scale f32 [B, H], weights uint16 (bf16) [B, H], key_pool uint8 [rows, 128],
    k_scale f32 [rows] -> (scores f32 [B, max_len], index int32 [B, k], n_selected int32 [B])."""
    q_fp8, key_pool = np.ascontiguousarray(q_fp8), np.ascontiguousarray(key_pool)
    q_scale, k_scale = np.ascontiguousarray(q_scale, dtype=np.float32), np.ascontiguousarray(k_scale, dtype=np.float32)
    weights = np.ascontiguousarray(weights, dtype=np.uint16)
    block_table = np.ascontiguousarray(block_table, dtype=np.int32)
    kv_len = np.ascontiguousarray(kv_len, dtype=np.int32)
    B, H = q_fp8.shape[0], q_fp8.shape[1]
    max_len = max(int(kv_len.max()), 1)
    scores = np.full((B, max_len), -np.inf, dtype=np.float32)
    lib().kvo_indexer_scores(_p(q_fp8), _p(q_scale), _p(weights), H, _p(key_pool), key_pool.shape[1], _p(k_scale),
                             _p(block_table), block_table.shape[1], _p(kv_len), B, block_size, _p(scores), max_len)
    index = np.empty((B, k), dtype=np.int32)
    n_sel = np.empty(B, dtype=np.int32)
    lib().kvo_topk_tokens(_p(scores), max_len, _p(kv_len), B, k, _p(index), _p(n_sel))
    return scores, index, n_sel
