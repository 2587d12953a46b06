"""The oracle's statements of the stages beside the KV path (RMSNorm, rotary embedding "half", block-32 MX
quantisation), held against independent numpy restatements in float64 and against the definitions of the
formats (CPU). The reference runs these as closed operators, so no vector of its own exists: parity unpinned."""
import numpy as np

import kvo


def f32(a):
    return kvo.bf16_to_f32(np.asarray(a))


def bf16_ulp(ref_f64):
    """Spacing of bf16 at |ref| (8 significant bits)."""
    a = np.maximum(np.abs(ref_f64), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


def e4m3_value(code):
    code = np.asarray(code, dtype=np.int64)
    sign = np.where(code & 0x80, -1.0, 1.0)
    e, m = (code >> 3) & 15, code & 7
    v = np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e - 7.0))
    return np.where((e == 15) & (m == 7), np.nan, sign * v)


def test_rmsnorm_matches_float64_within_one_bf16_step():
    x = kvo.normal_bf16(40 * 576, 3).reshape(40, 576)
    x[3, :512] = kvo.f32_to_bf16(f32(x[3, :512]) * 300.0)   # a large row
    x[4, :512] = 0                                           # an all-zero row: rstd = 1/sqrt(eps)
    gamma = kvo.f32_to_bf16(1.0 + 0.1 * f32(kvo.normal_bf16(512, 7)))
    y, rstd = kvo.rmsnorm512(x, gamma, 1e-6)
    xf, gf = f32(x[:, :512]).astype(np.float64), f32(gamma).astype(np.float64)
    ref_r = 1.0 / np.sqrt((xf * xf).mean(axis=1) + 1e-6)
    assert np.allclose(rstd, ref_r, rtol=3e-7, atol=0)
    ref = xf * ref_r[:, None] * gf
    err = np.abs(f32(y).astype(np.float64) - ref)
    assert (err <= 1.01 * bf16_ulp(ref)).all()           # at most one step off the exact value
    assert (err <= 0.51 * bf16_ulp(ref)).mean() > 0.97    # and almost always the nearest one
    assert rstd[4] == np.float32(1.0 / np.sqrt(np.float32(1e-6))) and not y[4].any()


def test_rope_half_is_a_rotation_of_the_pairs():
    T, V = 6, 5
    x = kvo.normal_bf16(T * V * 64, 2).reshape(T, V, 64)
    angle = np.linspace(0.0, 5.0, T * 32).reshape(T, 32)
    cos = kvo.f32_to_bf16(np.concatenate([np.cos(angle), np.cos(angle)], axis=1).astype(np.float32))
    sin = kvo.f32_to_bf16(np.concatenate([np.sin(angle), np.sin(angle)], axis=1).astype(np.float32))
    y = kvo.rope_half64(x, cos, sin)
    xf, cf, sf = f32(x).astype(np.float64), f32(cos).astype(np.float64), f32(sin).astype(np.float64)
    ref = np.empty_like(xf)
    ref[..., :32] = xf[..., :32] * cf[:, None, :32] - xf[..., 32:] * sf[:, None, :32]
    ref[..., 32:] = xf[..., 32:] * cf[:, None, 32:] + xf[..., :32] * sf[:, None, 32:]
    err = np.abs(f32(y).astype(np.float64) - ref)
    assert (err <= 0.5 * bf16_ulp(ref) + 1e-12 + 2.0 ** -24 * np.abs(ref)).all()   # one rounding to bf16
    # zero angle leaves the vector alone; a quarter turn swaps the halves with a sign
    one, zero = kvo.f32_to_bf16(np.ones(64, np.float32)), np.zeros(64, np.uint16)
    assert np.array_equal(kvo.rope_half64(x[:1], one[None], zero[None]), x[:1])
    quarter = kvo.rope_half64(x[:1], zero[None], one[None])
    assert np.array_equal(f32(quarter[..., :32]), -f32(x[:1, :, 32:])) and np.array_equal(quarter[..., 32:], x[:1, :, :32])


def test_e4m3_conversion_is_round_to_nearest_even_and_saturates():
    codes = np.arange(256)
    values = e4m3_value(codes)
    finite = np.sort(np.unique(np.abs(values[~np.isnan(values)])))
    assert finite[-1] == 448.0 and finite[1] == 2.0 ** -9
    L = kvo.lib()
    for c in codes:                                   # every representable value maps to itself
        if not np.isnan(values[c]) and values[c] != 0:
            assert L.kvo_f32_to_e4m3(float(values[c])) == c
    mids = (finite[:-1] + finite[1:]) / 2              # ties go to the even code
    for lo, mid in zip(finite[:-1], mids):
        got = L.kvo_f32_to_e4m3(float(mid))
        lo_code = L.kvo_f32_to_e4m3(float(lo))
        assert got == (lo_code if lo_code % 2 == 0 else lo_code + 1), (lo, mid, got)
    assert L.kvo_f32_to_e4m3(1e9) == 0x7E and L.kvo_f32_to_e4m3(-464.0) == 0xFE and L.kvo_f32_to_e4m3(float("nan")) & 0x7F == 0x7F
    assert L.kvo_f32_to_e4m3(2.0 ** -10) == 0 and L.kvo_f32_to_e4m3(2.0 ** -10 * 1.01) == 1 and L.kvo_f32_to_e4m3(-0.0) == 0x80


def test_mx_quant_blocks_follow_the_scale_rule():
    rows, cols = 7, 256
    x = kvo.normal_bf16(rows * cols, 2).reshape(rows, cols)
    x[0, :32] = 0                                                       # all-zero block
    x[1, :32] = kvo.f32_to_bf16(f32(x[1, :32]) * 1e30)                  # huge values
    x[2, :32] = kvo.f32_to_bf16(f32(x[2, :32]) * 1e-30)                 # tiny values
    x[3, 5] = 0x7FC0                                                    # a NaN poisons its block
    x[4, :32] = kvo.f32_to_bf16(np.full(32, 448.0, np.float32))         # exactly the largest code
    q, s = kvo.mx_quant_e4m3(x)
    xf = f32(x).astype(np.float64).reshape(rows, cols // 32, 32)
    amax = np.abs(xf).max(axis=2)
    for r in range(rows):
        for b in range(cols // 32):
            if np.isnan(amax[r, b]):
                assert s[r, b] == 0xFF and ((q[r, 32 * b:32 * b + 32] & 0x7F) == 0x7F).all()
                continue
            e = -127 if amax[r, b] == 0 else int(np.clip(np.floor(np.log2(amax[r, b])) - 8, -127, 127))
            assert s[r, b] == e + 127, (r, b)
            back = e4m3_value(q[r, 32 * b:32 * b + 32]) * 2.0 ** e
            scaled = xf[r, b] * 2.0 ** -e
            # the largest element lands in [256, 512): nothing is lost to the scale but the 3-bit mantissa
            assert np.abs(scaled).max() < 512
            step = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(scaled), 2.0 ** -6))) - 3)
            ok = np.abs(e4m3_value(q[r, 32 * b:32 * b + 32]) - np.clip(scaled, -448, 448)) <= 0.5 * step + 1e-12
            assert ok.all(), (r, b)
            assert np.isfinite(back).all()
    assert s[0, 0] == 0 and not q[0, :32].any() and (q[4, :32] == 0x7E).all() and s[4, 0] == 127


def _indexer_case(B, H, lens, bs, seed=5):
    rng = np.random.default_rng(seed)
    blocks = int(sum((int(n) + bs - 1) // bs for n in lens)) + 2
    table = np.zeros((B, max(1, max((int(n) + bs - 1) // bs for n in lens))), dtype=np.int32)
    order = rng.permutation(blocks)
    at = 0
    for b, n in enumerate(lens):
        nb = (int(n) + bs - 1) // bs
        table[b, :nb] = order[at:at + nb]
        at += nb
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)   # every finite E4M3 code
    q = rng.choice(codes[(codes & 0x7F) < 0x50], size=(B, H, 128)).astype(np.uint8)
    key = rng.choice(codes[(codes & 0x7F) < 0x50], size=(blocks * bs, 128)).astype(np.uint8)
    q_scale = rng.uniform(0.01, 0.1, size=(B, H)).astype(np.float32)
    k_scale = rng.uniform(0.01, 0.1, size=(blocks * bs,)).astype(np.float32)
    weights = kvo.f32_to_bf16(rng.normal(0.0, 1.0, size=(B, H)).astype(np.float32))
    return q, q_scale, weights, key, k_scale, table, np.asarray(lens, dtype=np.int32)


def test_indexer_scores_and_selection_match_a_float64_restatement():
    B, H, bs, k = 3, 16, 16, 24
    q, qs, w, key, ks, table, lens = _indexer_case(B, H, [100, 7, 33], bs)
    scores, index, n_sel = kvo.indexer_topk(q, qs, w, key, ks, table, lens, bs, k)
    qf, kf = e4m3_value(q), e4m3_value(key)
    wf = f32(w).astype(np.float64)
    for b in range(B):
        n = int(lens[b])
        rows = table[b, np.arange(n) // bs].astype(np.int64) * bs + np.arange(n) % bs
        dots = kf[rows] @ qf[b].T                                    # [n, H]
        ref = (np.maximum(dots * (qs[b].astype(np.float64)[None, :] * ks[rows].astype(np.float64)[:, None]), 0.0)
               * wf[b][None, :]).sum(axis=1)
        assert np.allclose(scores[b, :n], ref, rtol=2e-5, atol=1e-5)
        assert n_sel[b] == min(k, n) and (index[b, n_sel[b]:] == -1).all()
        picked = index[b, : n_sel[b]]
        assert len(set(picked.tolist())) == len(picked)
        got = scores[b, picked]
        assert (np.diff(got) <= 0).all()                              # best first
        rest = np.setdiff1d(np.arange(n), picked)
        if len(rest):
            assert scores[b, rest].max() <= got.min()                 # nothing better was left out
        for i in range(len(picked) - 1):                              # ties: lower position first
            if got[i] == got[i + 1]:
                assert picked[i] < picked[i + 1]
