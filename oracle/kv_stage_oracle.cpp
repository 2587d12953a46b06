// CPU oracle for the stages on either side of the KV path: the producer of the appended row (RMSNorm of
// the 512-wide latent, partial rotary embedding of the 64-wide rope slice and of the query's rope slices)
// and the consumer of the attention output (block-32 MX quantisation to FP8 E4M3 with E8M0 scales).
//
// THIS FILE IS TEST INFRASTRUCTURE, like kv_oracle.cpp: nothing in the product library links or calls it.
//
// PARITY UNPINNED: the reference runs these stages as closed operators (aclnnRmsNorm,
// aclnnApplyRotaryPosEmbV2, aclnnDynamicMxQuant; stages 6, 7 and 10 of src/pipeline/pipeline.cpp:212-258)
// and its mock launches do nothing, so its tree holds no numeric vector for them. What is restated here is
// what the call sites fix: epsilon and the gamma operand (pipeline.cpp:215-216), rotary mode "half" on
// [T, heads, 64] and [T, 1, 64] slices with one cos/sin row of 64 per token (pipeline.cpp:51, 222-223;
// src/memory/static_arena_manager.cpp:484-488, 590-591), and block 32, round-to-nearest-even, FP8 E4M3
// values with E8M0 scales by the OCP microscaling rule (pipeline.cpp:49, 253-256; static_arena_manager.cpp
// :492-495). The arithmetic is SPECIFIED to the operation, so that the CUDA kernels can match it bit for
// bit; this file must be compiled with floating-point contraction off (see the Makefile):
//
//   RMSNorm of a 512-wide row x with weight g (both bf16), 32 lanes as on the device:
//     lane L accumulates a = fma(x_i, x_i, a) over i = 8L..8L+7, then i = 256+8L..256+8L+7, from a = 0;
//     the 32 partial sums are combined by a butterfly: for off in 16, 8, 4, 2, 1: a_L += a_(L xor off);
//     r = 1 / sqrt(a * (1/512) + eps)   (IEEE division and square root, fp32);
//     y_i = bf16( (x_i * r) * g_i )     (two fp32 multiplications, then round to nearest even).
//   Rotary embedding, mode "half", of a 64-wide vector x with rows c (cos) and s (sin), for i in 0..31:
//     y_i      = bf16( fma(-x_(i+32), s_i,      x_i * c_i) )
//     y_(i+32) = bf16( fma( x_i,      s_(i+32), x_(i+32) * c_(i+32)) )
//   MX quantisation of 32 values (bf16 -> fp32 exactly): m = max |x_i| (NaN makes the scale NaN);
//     e = floor(log2 m) - 8, clamped to [-127, 127] (m = 0 gives -127); scale byte = e + 127;
//     q_i = fp8_e4m3( x_i * 2^(-e) ), round to nearest even, saturating at +-448, NaN -> 0x7F | sign.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>

namespace {

inline float Bf16ToF32(uint16_t v) {
  uint32_t bits = static_cast<uint32_t>(v) << 16;
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

inline uint16_t F32ToBf16(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((bits >> 16) | 0x0040u);  // quiet NaN
  const uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return static_cast<uint16_t>(bits >> 16);
}

// fp32 -> FP8 E4M3 (1-4-3, bias 7, no infinities, 0x7F/0xFF = NaN), round to nearest even, saturating.
inline uint8_t F32ToE4m3(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  const uint8_t sign = static_cast<uint8_t>((bits >> 24) & 0x80u);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint8_t>(sign | 0x7fu);
  const float a = std::fabs(f);
  if (a >= 448.0f) {
    // Everything at or above the largest finite value saturates (464 would be the rounding boundary to the
    // NaN code; saturation wins there too).
    return static_cast<uint8_t>(sign | 0x7eu);
  }
  if (a == 0.0f) return sign;
  int exp2;
  std::frexp(a, &exp2);  // a = m * 2^exp2, m in [0.5, 1)
  int e = exp2 - 1;      // floor(log2 a)
  if (e < -6) e = -6;    // subnormal range shares the exponent of the smallest normal
  // Quantum is 2^(e-3); the value in quanta, rounded to nearest even.
  const float quanta = std::ldexp(a, 3 - e);
  float rounded = std::nearbyint(quanta);  // default rounding mode is to nearest even
  int mant = static_cast<int>(rounded);
  int exp_field;
  if (e == -6 && mant < 8) {
    exp_field = 0;  // subnormal: mant in 0..7
  } else {
    if (mant == 16) {  // rounded up into the next binade
      mant = 8;
      ++e;
    }
    exp_field = e + 7;
    mant -= 8;
  }
  if (exp_field > 15 || (exp_field == 15 && mant > 6)) return static_cast<uint8_t>(sign | 0x7eu);
  return static_cast<uint8_t>(sign | (exp_field << 3) | mant);
}

float RmsScale(const uint16_t* x, float eps) {
  float lanes[32];
  for (int lane = 0; lane < 32; ++lane) {
    float a = 0.0f;
    for (int half = 0; half < 2; ++half) {
      for (int j = 0; j < 8; ++j) {
        const float v = Bf16ToF32(x[256 * half + 8 * lane + j]);
        a = std::fmaf(v, v, a);
      }
    }
    lanes[lane] = a;
  }
  for (int off = 16; off > 0; off >>= 1) {
    float next[32];
    for (int lane = 0; lane < 32; ++lane) next[lane] = lanes[lane] + lanes[lane ^ off];
    std::memcpy(lanes, next, sizeof(lanes));
  }
  const float mean = lanes[0] * (1.0f / 512.0f);
  return 1.0f / std::sqrt(mean + eps);
}

void RopeHalf(const uint16_t* x, const uint16_t* c, const uint16_t* s, uint16_t* y) {
  uint16_t out[64];
  for (int i = 0; i < 32; ++i) {
    const float x1 = Bf16ToF32(x[i]), x2 = Bf16ToF32(x[i + 32]);
    const float lo = x1 * Bf16ToF32(c[i]);
    const float hi = x2 * Bf16ToF32(c[i + 32]);
    out[i] = F32ToBf16(std::fmaf(-x2, Bf16ToF32(s[i]), lo));
    out[i + 32] = F32ToBf16(std::fmaf(x1, Bf16ToF32(s[i + 32]), hi));
  }
  std::memcpy(y, out, sizeof(out));
}

}  // namespace

extern "C" {

// y[t][0..511] = RMSNorm(x[t]) * gamma, rstd[t] = the row's reciprocal RMS (or null).
// Follows stage 6 of the reference (src/pipeline/pipeline.cpp:212-218): x = kv_a[:, :512], eps 1e-6.
void kvo_rmsnorm512(const uint16_t* x, int64_t x_stride, const uint16_t* gamma, float eps, int64_t rows, uint16_t* y,
                    int64_t y_stride, float* rstd) {
  for (int64_t t = 0; t < rows; ++t) {
    const uint16_t* row = x + t * x_stride;
    const float r = RmsScale(row, eps);
    if (rstd != nullptr) rstd[t] = r;
    for (int i = 0; i < 512; ++i) {
      const float scaled = Bf16ToF32(row[i]) * r;
      y[t * y_stride + i] = F32ToBf16(scaled * Bf16ToF32(gamma[i]));
    }
  }
}

// Rotary embedding, mode "half", of vectors x[t][v][0..63] (v < vectors) with the token's cos/sin row.
// Follows stage 7 of the reference (src/pipeline/pipeline.cpp:219-225): q_rope [T, 64 heads, 64] and
// k_rope [T, 1, 64], both rotated in place with rope_cos / rope_sin [T, 64].
void kvo_rope_half64(const uint16_t* x, int64_t token_stride, int64_t vector_stride, const uint16_t* cos,
                     int64_t cos_stride, const uint16_t* sin, int64_t sin_stride, int64_t tokens, int64_t vectors,
                     uint16_t* y, int64_t y_token_stride, int64_t y_vector_stride) {
  for (int64_t t = 0; t < tokens; ++t) {
    for (int64_t v = 0; v < vectors; ++v) {
      RopeHalf(x + t * token_stride + v * vector_stride, cos + t * cos_stride, sin + t * sin_stride,
               y + t * y_token_stride + v * y_vector_stride);
    }
  }
}

// The fused producer: row t of kv_a ([latent 512 | rope 64], stride kv_a_stride) is normalised and rotated
// and written to pool row slot[t] (negative: skipped). Returns the number of slots outside the pool.
// Follows stages 6-8 of the reference (src/pipeline/pipeline.cpp:212-234) taken together.
int64_t kvo_append_fused(const uint16_t* kv_a, int64_t kv_a_stride, const uint16_t* gamma, float eps, const uint16_t* cos,
                         int64_t cos_stride, const uint16_t* sin, int64_t sin_stride, const int32_t* slots,
                         int64_t tokens, uint16_t* latent_pool, int64_t latent_row_stride, uint16_t* rope_pool,
                         int64_t rope_row_stride, int64_t pool_rows) {
  int64_t bad = 0;
  for (int64_t t = 0; t < tokens; ++t) {
    const int64_t slot = slots[t];
    if (slot < 0) continue;
    if (slot >= pool_rows) {
      ++bad;
      continue;
    }
    kvo_rmsnorm512(kv_a + t * kv_a_stride, kv_a_stride, gamma, eps, 1, latent_pool + slot * latent_row_stride,
                   latent_row_stride, nullptr);
    RopeHalf(kv_a + t * kv_a_stride + 512, cos + t * cos_stride, sin + t * sin_stride, rope_pool + slot * rope_row_stride);
  }
  return bad;
}

// Block-32 MX quantisation along the last axis: x bf16 [rows][cols] (cols % 32 == 0) -> q FP8 E4M3
// [rows][cols], scales E8M0 [rows][cols / 32].
// Follows stage 10 of the reference (src/pipeline/pipeline.cpp:250-258): attn_flat [T, 64 x 512] ->
// attn_fp8 + attn_mx_scale [T, 1024].
void kvo_mx_quant_e4m3(const uint16_t* x, int64_t x_stride, int64_t rows, int64_t cols, uint8_t* q, int64_t q_stride,
                       uint8_t* scales, int64_t scale_stride) {
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < cols / 32; ++b) {
      const uint16_t* src = x + r * x_stride + 32 * b;
      float amax = 0.0f;
      bool nan = false;
      for (int i = 0; i < 32; ++i) {
        const float v = std::fabs(Bf16ToF32(src[i]));
        if (std::isnan(v)) nan = true;
        if (v > amax) amax = v;  // infinities included
      }
      int e;
      if (nan) {
        scales[r * scale_stride + b] = 0xff;
        for (int i = 0; i < 32; ++i) q[r * q_stride + 32 * b + i] = static_cast<uint8_t>(((src[i] >> 8) & 0x80u) | 0x7fu);
        continue;
      }
      if (amax == 0.0f) {
        e = -127;
      } else if (std::isinf(amax)) {
        e = 127;
      } else {
        int exp2;
        std::frexp(amax, &exp2);
        e = exp2 - 1 - 8;
        if (e < -127) e = -127;
        if (e > 127) e = 127;
      }
      scales[r * scale_stride + b] = static_cast<uint8_t>(e + 127);
      for (int i = 0; i < 32; ++i) {
        const float scaled = std::ldexp(Bf16ToF32(src[i]), -e);  // exact unless it overflows (then it saturates)
        q[r * q_stride + 32 * b + i] = F32ToE4m3(scaled);
      }
    }
  }
}

// Single conversions, for the tests of the conversion itself.
uint8_t kvo_f32_to_e4m3(float f) { return F32ToE4m3(f); }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Sparse-selection indexer in front of attention (the reference vendors it and plans it but does not apply
// it: include/moe/pipeline/pipeline.hpp:57-66; operator contract mock/mock_ops.cpp:1118-1221; formula
// third_party/ops_transformer/attention/quant_lightning_indexer/README.md: out = Top-k over tokens of
// sum_h W_h * ReLU(ScaleQ_h * ScaleK_t * (Q_h . K_t)) with FP8 E4M3 Q and K of width 128, N2 = 1).
// PARITY UNPINNED (a closed operator on the device, a no-op in the mock). The arithmetic is specified:
//   dot_h  = fma chain over d = 0..127 from 0, fp32, FP8 values converted exactly;
//   s_h    = max(0, (qs_h * ks_t) * dot_h)          (two fp32 multiplications);
//   score  = fma chain over h = 0..heads-1 of w_h * s_h from 0;  a NaN score counts as -infinity;
//   order  = by score descending, ties by token index ascending; the first k tokens are the selection.
// ---------------------------------------------------------------------------------------------
namespace {
inline float E4m3ToF32(uint8_t v) {
  const int e = (v >> 3) & 15, m = v & 7;
  float a;
  if (e == 15 && m == 7) a = std::numeric_limits<float>::quiet_NaN();
  else if (e == 0) a = std::ldexp(static_cast<float>(m), -9);
  else a = std::ldexp(1.0f + static_cast<float>(m) / 8.0f, e - 7);
  return (v & 0x80) ? -a : a;
}
}  // namespace

extern "C" {

// scores[b][t] for t < kv_len[b] (the rest untouched). q: fp8 [B][heads][128]; q_scale fp32 [B][heads];
// weights bf16 [B][heads]; key pool fp8 [rows][key_stride]; k_scale fp32 [rows]; paged by block_table.
void kvo_indexer_scores(const uint8_t* q, const float* q_scale, const uint16_t* weights, int32_t heads, const uint8_t* key_pool,
                        int64_t key_stride, const float* k_scale, const int32_t* block_table, int64_t max_blocks,
                        const int32_t* kv_len, int32_t batch, int32_t block_size, float* scores, int64_t score_stride) {
  for (int32_t b = 0; b < batch; ++b) {
    for (int32_t t = 0; t < kv_len[b]; ++t) {
      const int64_t row = static_cast<int64_t>(block_table[b * max_blocks + t / block_size]) * block_size + t % block_size;
      const uint8_t* k = key_pool + row * key_stride;
      float score = 0.0f;
      for (int32_t h = 0; h < heads; ++h) {
        const uint8_t* qh = q + (static_cast<int64_t>(b) * heads + h) * 128;
        float dot = 0.0f;
        for (int d = 0; d < 128; ++d) dot = std::fmaf(E4m3ToF32(qh[d]), E4m3ToF32(k[d]), dot);
        const float scaled = (q_scale[b * heads + h] * k_scale[row]) * dot;
        const float s = scaled > 0.0f ? scaled : 0.0f;  // NaN compares false: 0
        score = std::fmaf(Bf16ToF32(weights[b * heads + h]), s, score);
      }
      scores[b * score_stride + t] = score;
    }
  }
}

// index[b][0..k) = the k best tokens of sequence b (by score descending, then index ascending), -1 beyond
// min(k, kv_len[b]); n_selected[b] = min(k, kv_len[b]).
void kvo_topk_tokens(const float* scores, int64_t score_stride, const int32_t* kv_len, int32_t batch, int32_t k,
                     int32_t* index, int32_t* n_selected) {
  for (int32_t b = 0; b < batch; ++b) {
    const int32_t n = kv_len[b];
    // insertion into a sorted list of at most k entries: small and obviously right
    int32_t kept = 0;
    for (int32_t t = 0; t < n; ++t) {
      float s = scores[b * score_stride + t];
      if (std::isnan(s)) s = -std::numeric_limits<float>::infinity();
      int32_t pos = kept;
      while (pos > 0) {
        const int32_t other = index[b * k + pos - 1];
        float so = scores[b * score_stride + other];
        if (std::isnan(so)) so = -std::numeric_limits<float>::infinity();
        if (so > s || (so == s && other < t)) break;
        --pos;
      }
      if (pos >= k) continue;
      const int32_t last = kept < k ? kept : k - 1;
      for (int32_t i = last; i > pos; --i) index[b * k + i] = index[b * k + i - 1];
      index[b * k + pos] = t;
      if (kept < k) ++kept;
    }
    for (int32_t i = kept; i < k; ++i) index[b * k + i] = -1;
    n_selected[b] = kept;
  }
}

}  // extern "C"
