"""Seeded scenario builders shared by the CPU and GPU tests (numpy only)."""
from __future__ import annotations

import numpy as np

import kvo


def blocks_for(length: int, block_size: int) -> int:
    return (length + block_size - 1) // block_size


def build_tables(kv_len, block_size: int, num_blocks: int, order=None):
    """Hands out blocks to sequences in admission order from `order` (default: seeded permutation).
    Returns int32 [B, max_blocks] (unused entries 0)."""
    kv_len = np.asarray(kv_len, dtype=np.int64)
    if order is None:
        order = kvo.permutation(num_blocks)
    need = [blocks_for(int(n), block_size) for n in kv_len]
    assert sum(need) <= num_blocks
    max_blocks = max(1, max(need))
    table = np.zeros((len(kv_len), max_blocks), dtype=np.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = order[at:at + n]
        at += n
    return table


def fragmented_tables(kv_len, block_size: int, num_blocks: int):
    """Round-robin hand-out from a shuffled free list: sequence b's blocks are interleaved with the
    others', as after long-running churn."""
    kv_len = np.asarray(kv_len, dtype=np.int64)
    order = list(kvo.permutation(num_blocks))
    need = [blocks_for(int(n), block_size) for n in kv_len]
    max_blocks = max(1, max(need))
    table = np.zeros((len(kv_len), max_blocks), dtype=np.int32)
    have = [0] * len(kv_len)
    at = 0
    progressing = True
    while progressing:
        progressing = False
        for b in range(len(kv_len)):
            if have[b] < need[b]:
                table[b, have[b]] = order[at]
                at += 1
                have[b] += 1
                progressing = True
    return table


def ragged_lengths(count: int, lo: int, hi: int, first: int = 0):
    """len = lo + x % (hi - lo + 1) from the lengths stream."""
    x = kvo.draws(count, kvo.STREAM_LEN, first)
    return (lo + (x % np.uint64(hi - lo + 1))).astype(np.int32)


def ref_attention_f64(q_u16, pool_u16, table, kv_len, block_size, scale, kv_begin=None):
    """Independent float64 restatement in numpy (not the oracle's code): returns out f64 [B,H,512], lse f64 [B,H]."""
    q = kvo.bf16_to_f32(q_u16).astype(np.float64)
    B, H, _ = q.shape
    out = np.zeros((B, H, kvo.LATENT))
    lse = np.full((B, H), -np.inf)
    for b in range(B):
        n = int(kv_len[b])
        if n == 0:
            continue
        begin = 0 if kv_begin is None else int(kv_begin[b])
        toks = np.arange(begin, begin + n)
        rows = table[b, toks // block_size].astype(np.int64) * block_size + toks % block_size
        kv = kvo.bf16_to_f32(pool_u16[rows]).astype(np.float64)
        s = scale * (q[b] @ kv.T)
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(axis=1, keepdims=True)
        out[b] = (p @ kv[:, : kvo.LATENT]) / l
        lse[b] = (m + np.log(l))[:, 0]
    return out, lse


# Every call of check_attention leaves a record here: (what, max abs err, worst excess over the row-max bound,
# worst excess over the per-element bound). conftest.py prints them at the end of a run and writes them to the
# file named by B200KV_TOLERANCE_REPORT, when that is set.
TOLERANCE_RECORDS = []


def check_attention(out_u16, lse, ref_out, ref_lse, abs_tol=2e-3, rel_tol=1e-2, lse_tol=1e-3, what="",
                    strict_abs=False, elementwise=None):
    """The tolerance the path is held to (bf16 in, fp32 accumulate, bf16 out), in three forms:

    per element  |got - ref| <= 2e-3 + 1e-2 * |ref|            asserted with elementwise=True, and always
                                                                implied by strict_abs
    per row      |got - ref| <= 2e-3 + 1e-2 * max_row |ref|    always asserted: an output row is a softmax-weighted
                                                                average of value rows, so its error is relative to
                                                                the magnitude of the values averaged, not to an
                                                                element of the row that happens to cancel
    absolute     |got - ref| <= 2e-3                            strict_abs: inputs drawn from the benchmark's
                                                                distribution (outputs well below 0.2 in magnitude)

    lse is within 1e-3. elementwise=None measures the per-element form without asserting it (adversarial
    inputs whose rows hold large values beside cancelling ones); the record says by how much it held or not."""
    got = kvo.bf16_to_f32(np.asarray(out_u16)).astype(np.float64)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - ref_out)
    row_scale = np.abs(ref_out).max(axis=-1, keepdims=True) if err.size else 0.0
    bound = abs_tol + rel_tol * row_scale
    worst = float((err - bound).max()) if err.size else -1.0
    worst_elem = float((err - (abs_tol + rel_tol * np.abs(ref_out))).max()) if err.size else -1.0
    max_abs = float(err.max()) if err.size else 0.0
    TOLERANCE_RECORDS.append({"what": what, "max_abs_err": max_abs, "row_bound_excess": worst,
                              "element_bound_excess": worst_elem, "strict_abs": bool(strict_abs),
                              "max_abs_ref": float(np.abs(ref_out).max()) if err.size else 0.0})
    assert worst <= 0.0, f"{what}: |err| exceeds {abs_tol} + {rel_tol}*rowmax|ref| by {worst:.3e} (max abs err {max_abs:.3e})"
    if strict_abs:
        assert max_abs <= abs_tol, f"{what}: max abs err {max_abs:.3e} > {abs_tol}"
    if elementwise:
        assert worst_elem <= 0.0, f"{what}: |err| exceeds {abs_tol} + {rel_tol}*|ref| per element by {worst_elem:.3e}"
    if lse is not None:
        finite = np.isfinite(ref_lse)
        assert (np.isfinite(np.asarray(lse)) == finite).all(), f"{what}: lse finiteness differs"
        if finite.any():
            lerr = float(np.abs(np.asarray(lse, dtype=np.float64)[finite] - ref_lse[finite]).max())
            assert lerr <= lse_tol, f"{what}: lse err {lerr:.3e} > {lse_tol}"
    return max_abs
