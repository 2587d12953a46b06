// CPU oracle for the decode-time KV-cache path: seeded inputs, KV block bookkeeping, scatter-append,
// block-table gather, absorbed-MLA decode attention and the log-sum-exp merge of split partials.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA path is compared with and the CPU
// baseline that is timed beside it; nothing in the product library links, loads or calls it.
//
// PARITY UNPINNED: the reference engine delegates this arithmetic to closed operator libraries
// (aclnnScatterPaKvCache, aclnnFusedInferAttentionScoreV5; CANN 9.2.0-beta.2) and its mock backend
// launches are no-ops (mock/mock_ops.cpp:29-31, 1225-1262), so the reference tree holds no numeric
// golden vector for this path. What follows restates the *semantics* the reference's call sites and
// descriptors define, each function citing the lines it follows; only the structural known-answers
// (block counts, utilisation) can be pinned, and tests/test_oracle_pins.py checks those.
//
// Build: see oracle/Makefile (g++ -O3 -march=native -fopenmp -shared).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------------------------------------
// bf16 <-> fp32 (round to nearest even, NaN kept quiet)
// ---------------------------------------------------------------------------------------------
inline float Bf16ToF32(uint16_t v) {
  uint32_t bits = static_cast<uint32_t>(v) << 16;
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

inline uint16_t F32ToBf16(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((bits >> 16) | 0x0040u);
  const uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return static_cast<uint16_t>(bits >> 16);
}

// ---------------------------------------------------------------------------------------------
// Counter-based generator: splitmix64 keyed by (seed, stream), Box-Muller in double, RNE to bf16.
// The base seed of the benchmarks is the reference harness's prompt seed
// (python/benchmarks/bench_runner.py:107).
// ---------------------------------------------------------------------------------------------
constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

inline uint64_t Mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

inline uint64_t StreamKey(uint64_t seed, uint64_t stream) { return Mix64(seed ^ (stream * kGolden + kGolden)); }

inline uint64_t Draw(uint64_t key, uint64_t counter) { return Mix64(key + (counter + 1) * kGolden); }

inline double NormalAt(uint64_t key, uint64_t element) {
  const uint64_t pair = element >> 1;
  const double u1 = static_cast<double>((Draw(key, 2 * pair) >> 11) + 1) * 0x1.0p-53;  // (0, 1]
  const double u2 = static_cast<double>(Draw(key, 2 * pair + 1) >> 11) * 0x1.0p-53;    // [0, 1)
  const double radius = std::sqrt(-2.0 * std::log(u1));
  const double angle = 6.283185307179586476925286766559 * u2;
  return (element & 1u) ? radius * std::sin(angle) : radius * std::cos(angle);
}

}  // namespace

extern "C" {

// dst[i] = bf16(scale * N(0,1)) for element counters first_element + i of stream (seed, stream).
void kvo_fill_normal_bf16(uint16_t* dst, int64_t count, uint64_t seed, uint64_t stream, uint64_t first_element,
                          double scale) {
  const uint64_t key = StreamKey(seed, stream);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    const double z = NormalAt(key, first_element + static_cast<uint64_t>(i)) * scale;
    dst[i] = F32ToBf16(static_cast<float>(z));
  }
}

// Raw 64-bit draws (used for lengths, churn choices).
void kvo_draw_u64(uint64_t* dst, int64_t count, uint64_t seed, uint64_t stream, uint64_t first_counter) {
  const uint64_t key = StreamKey(seed, stream);
  for (int64_t i = 0; i < count; ++i) dst[i] = Draw(key, first_counter + static_cast<uint64_t>(i));
}

// Fisher-Yates permutation of 0..count-1 driven by the same stream.
void kvo_permutation(int32_t* dst, int32_t count, uint64_t seed, uint64_t stream) {
  const uint64_t key = StreamKey(seed, stream);
  for (int32_t i = 0; i < count; ++i) dst[i] = i;
  for (int32_t i = count - 1; i > 0; --i) {
    const uint64_t j = Draw(key, static_cast<uint64_t>(i)) % static_cast<uint64_t>(i + 1);
    std::swap(dst[i], dst[j]);
  }
}

void kvo_f32_to_bf16(const float* src, uint16_t* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = F32ToBf16(src[i]);
}

void kvo_bf16_to_f32(const uint16_t* src, float* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = Bf16ToF32(src[i]);
}

// ---------------------------------------------------------------------------------------------
// KV reservation geometry (src/memory/static_arena_manager.cpp:197, 232-240, 315-318): blocks per
// layer = ceil(max_context / block_size); the pool is layer-major, two co-indexed caches.
// ---------------------------------------------------------------------------------------------
int64_t kvo_blocks_per_layer(int64_t max_context, int64_t block_size) {
  return (max_context + block_size - 1) / block_size;
}

// Total blocks the diagnostics report (src/pipeline/pipeline.cpp:134-136): per-layer blocks x layers.
int64_t kvo_total_blocks(int64_t max_context, int64_t block_size, int64_t layers) {
  return kvo_blocks_per_layer(max_context, block_size) * layers;
}

// Utilisation after `position` has been written (src/pipeline/pipeline.cpp:532-534):
// (position + 1) / (blocks x block_size).
double kvo_utilisation(int64_t position, int64_t max_context, int64_t block_size) {
  const int64_t capacity = kvo_blocks_per_layer(max_context, block_size) * block_size;
  return static_cast<double>(position + 1) / static_cast<double>(capacity);
}

// Bytes of the two KV spans (src/memory/static_arena_manager.cpp:315-318).
void kvo_pool_bytes(int64_t max_context, int64_t block_size, int64_t layers, int64_t latent_dim, int64_t rope_dim,
                    int64_t* latent_bytes, int64_t* rope_bytes) {
  const int64_t rows = kvo_blocks_per_layer(max_context, block_size) * block_size * layers;
  *latent_bytes = rows * latent_dim * 2;
  *rope_bytes = rows * rope_dim * 2;
}

// ---------------------------------------------------------------------------------------------
// Append (stage kv_cache_write, src/pipeline/pipeline.cpp:226-234; contract
// include/moe/core/op_table.hpp:339-372, mode "Norm"): for each token row t,
//   latent_cache[slot[t] / bs][slot[t] % bs][:] = latent[t][:],  rope_cache likewise.
// A cache is addressed as flat rows here (block*bs + offset == slot). Rows whose slot is negative
// are skipped (padding); a slot >= pool_rows is reported and skipped.
// Strides are in elements. Returns the number of out-of-range slots.
// ---------------------------------------------------------------------------------------------
int64_t kvo_append(const uint16_t* latent_src, int64_t src_latent_stride, const uint16_t* rope_src,
                   int64_t src_rope_stride, uint16_t* latent_pool, int64_t latent_row_stride, uint16_t* rope_pool,
                   int64_t rope_row_stride, const int32_t* slot_mapping, int64_t n_tokens, int64_t pool_rows,
                   int64_t latent_dim, int64_t rope_dim) {
  int64_t bad = 0;
  for (int64_t t = 0; t < n_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    if (slot >= pool_rows) {
      ++bad;
      continue;
    }
    std::memcpy(latent_pool + slot * latent_row_stride, latent_src + t * src_latent_stride,
                static_cast<size_t>(latent_dim) * 2);
    std::memcpy(rope_pool + slot * rope_row_stride, rope_src + t * src_rope_stride,
                static_cast<size_t>(rope_dim) * 2);
  }
  return bad;
}

// ---------------------------------------------------------------------------------------------
// Gather: logical token j of sequence b lives in physical row
//   block_table[b * max_blocks + j / bs] * bs + j % bs
// (the block_table argument of the attention stage, src/pipeline/pipeline.cpp:241,244; the only
// source-visible statement of the addressing is the vendored indexer,
// third_party/ops_transformer/attention/quant_lightning_indexer/op_kernel/arch35/
// quant_lightning_indexer_service_cube.h:243-268). Output rows of sequence b start at
// out_row_offsets[b]. Returns the number of out-of-range block ids (rows skipped).
// ---------------------------------------------------------------------------------------------
int64_t kvo_gather(const uint16_t* latent_pool, int64_t latent_row_stride, const uint16_t* rope_pool,
                   int64_t rope_row_stride, int64_t pool_rows, const int32_t* block_table, int64_t max_blocks,
                   const int32_t* kv_len, int64_t batch, int64_t block_size, uint16_t* out_latent,
                   int64_t out_latent_stride, uint16_t* out_rope, int64_t out_rope_stride,
                   const int64_t* out_row_offsets, int64_t latent_dim, int64_t rope_dim) {
  int64_t bad = 0;
#pragma omp parallel for schedule(dynamic) reduction(+ : bad)
  for (int64_t b = 0; b < batch; ++b) {
    for (int64_t j = 0; j < kv_len[b]; ++j) {
      const int64_t block = block_table[b * max_blocks + j / block_size];
      const int64_t row = block * block_size + j % block_size;
      if (block < 0 || row >= pool_rows) {
        ++bad;
        continue;
      }
      const int64_t dst = out_row_offsets[b] + j;
      std::memcpy(out_latent + dst * out_latent_stride, latent_pool + row * latent_row_stride,
                  static_cast<size_t>(latent_dim) * 2);
      std::memcpy(out_rope + dst * out_rope_stride, rope_pool + row * rope_row_stride,
                  static_cast<size_t>(rope_dim) * 2);
    }
  }
  return bad;
}

// ---------------------------------------------------------------------------------------------
// Absorbed-MLA decode attention (stage attention, src/pipeline/pipeline.cpp:235-249; formula
// softmax(scale Q K^T) V, include/moe/core/op_table.hpp:377; key = latent (+) rope through the
// query_rope / key_rope arguments, op_table.hpp:407-408; value list = latent cache,
// src/memory/static_arena_manager.cpp:579-580; out [T,64,512] bf16 and lse [T,64,1] fp32,
// static_arena_manager.cpp:491,496-497; one query token per sequence, kTokensPerStep = 1).
//
// Per sequence b and head h, over logical tokens j in [kv_begin[b], kv_begin[b] + kv_len[b]):
//   s_j = scale * (q_lat[h] . c_j + q_rope[h] . r_j),  m = max_j s_j,  p_j = exp(s_j - m),
//   l = sum_j p_j,  out[h] = (sum_j p_j c_j) / l  (bf16, RNE),  lse[h] = m + log(l).
// bf16 inputs are widened to fp32; scores, exp, sums and PV accumulate in fp32 (double when
// `use_double`). The un-normalised partial (m, l, O = sum p_j c_j) is also returned when the
// partial_* pointers are non-null, for the KV-range split. kv_begin may be null (all zero).
// A sequence with kv_len 0 yields out = 0, lse = -inf, partial m = -inf, l = 0.
// q layout: q[b*q_seq_stride + h*q_head_stride + k], k < latent_dim is q_lat, then q_rope.
// ---------------------------------------------------------------------------------------------
void kvo_mla_decode(const uint16_t* q, int64_t q_seq_stride, int64_t q_head_stride, const uint16_t* latent_pool,
                    int64_t latent_row_stride, const uint16_t* rope_pool, int64_t rope_row_stride,
                    const int32_t* block_table, int64_t max_blocks, const int32_t* kv_len, const int32_t* kv_begin,
                    int64_t batch, int64_t heads, int64_t block_size, int64_t latent_dim, int64_t rope_dim,
                    float scale, int32_t use_double, uint16_t* out_bf16, float* lse, float* partial_o,
                    float* partial_m, float* partial_l) {
  const int64_t work = batch * heads;
#pragma omp parallel
  {
    std::vector<float> scores;
    std::vector<double> acc_d(static_cast<size_t>(latent_dim));
    std::vector<float> acc_f(static_cast<size_t>(latent_dim));
    std::vector<float> qf(static_cast<size_t>(latent_dim + rope_dim));
#pragma omp for schedule(dynamic, 1)
    for (int64_t item = 0; item < work; ++item) {
      const int64_t b = item / heads;
      const int64_t h = item % heads;
      const int64_t len = kv_len[b];
      const int64_t begin = kv_begin ? kv_begin[b] : 0;
      const uint16_t* qrow = q + b * q_seq_stride + h * q_head_stride;
      for (int64_t k = 0; k < latent_dim + rope_dim; ++k) qf[static_cast<size_t>(k)] = Bf16ToF32(qrow[k]);
      scores.resize(static_cast<size_t>(len));
      float m = -std::numeric_limits<float>::infinity();
      for (int64_t j = 0; j < len; ++j) {
        const int64_t tok = begin + j;
        const int64_t row = static_cast<int64_t>(block_table[b * max_blocks + tok / block_size]) * block_size +
                            tok % block_size;
        const uint16_t* c = latent_pool + row * latent_row_stride;
        const uint16_t* r = rope_pool + row * rope_row_stride;
        float s;
        if (use_double) {
          double acc = 0.0;
          for (int64_t k = 0; k < latent_dim; ++k) acc += static_cast<double>(qf[k]) * Bf16ToF32(c[k]);
          for (int64_t k = 0; k < rope_dim; ++k) acc += static_cast<double>(qf[latent_dim + k]) * Bf16ToF32(r[k]);
          s = static_cast<float>(acc * static_cast<double>(scale));
        } else {
          float acc = 0.0f;
          for (int64_t k = 0; k < latent_dim; ++k) acc += qf[k] * Bf16ToF32(c[k]);
          for (int64_t k = 0; k < rope_dim; ++k) acc += qf[latent_dim + k] * Bf16ToF32(r[k]);
          s = acc * scale;
        }
        scores[static_cast<size_t>(j)] = s;
        m = std::max(m, s);
      }
      std::fill(acc_d.begin(), acc_d.end(), 0.0);
      std::fill(acc_f.begin(), acc_f.end(), 0.0f);
      double l_d = 0.0;
      float l_f = 0.0f;
      for (int64_t j = 0; j < len; ++j) {
        const int64_t tok = begin + j;
        const int64_t row = static_cast<int64_t>(block_table[b * max_blocks + tok / block_size]) * block_size +
                            tok % block_size;
        const uint16_t* c = latent_pool + row * latent_row_stride;
        if (use_double) {
          const double p = std::exp(static_cast<double>(scores[j]) - static_cast<double>(m));
          l_d += p;
          for (int64_t k = 0; k < latent_dim; ++k) acc_d[k] += p * Bf16ToF32(c[k]);
        } else {
          const float p = std::exp(scores[j] - m);
          l_f += p;
          for (int64_t k = 0; k < latent_dim; ++k) acc_f[k] += p * Bf16ToF32(c[k]);
        }
      }
      const double l = use_double ? l_d : static_cast<double>(l_f);
      const int64_t o = (b * heads + h) * latent_dim;
      for (int64_t k = 0; k < latent_dim; ++k) {
        const double num = use_double ? acc_d[k] : static_cast<double>(acc_f[k]);
        if (partial_o) partial_o[o + k] = static_cast<float>(num);
        if (out_bf16) {
          const float val = len > 0 ? (use_double ? static_cast<float>(num / l) : acc_f[k] / l_f) : 0.0f;
          out_bf16[o + k] = F32ToBf16(val);
        }
      }
      if (partial_m) partial_m[b * heads + h] = m;
      if (partial_l) partial_l[b * heads + h] = static_cast<float>(l);
      if (lse) {
        lse[b * heads + h] = len > 0 ? (use_double ? static_cast<float>(static_cast<double>(m) + std::log(l_d))
                                                   : m + std::log(l_f))
                                     : -std::numeric_limits<float>::infinity();
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Log-sum-exp merge of n_parts partials per (sequence, head):
//   M = max_r m_r,  L = sum_r l_r e^{m_r - M},  out = (sum_r O_r e^{m_r - M}) / L,  lse = M + log L.
// Layout: partial_o [n_parts][batch*heads][dim], partial_m / partial_l [n_parts][batch*heads].
// Parts with l == 0 (empty shard) contribute nothing. All parts empty: out = 0, lse = -inf.
// ---------------------------------------------------------------------------------------------
void kvo_lse_merge(const float* partial_o, const float* partial_m, const float* partial_l, int64_t n_parts,
                   int64_t rows, int64_t dim, uint16_t* out_bf16, float* lse) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float big = -std::numeric_limits<float>::infinity();
    for (int64_t p = 0; p < n_parts; ++p) {
      if (partial_l[p * rows + r] > 0.0f) big = std::max(big, partial_m[p * rows + r]);
    }
    float total = 0.0f;
    std::vector<float> acc(static_cast<size_t>(dim), 0.0f);
    for (int64_t p = 0; p < n_parts; ++p) {
      const float l = partial_l[p * rows + r];
      if (!(l > 0.0f)) continue;
      const float w = std::exp(partial_m[p * rows + r] - big);
      total += l * w;
      const float* o = partial_o + (p * rows + r) * dim;
      for (int64_t k = 0; k < dim; ++k) acc[k] += o[k] * w;
    }
    for (int64_t k = 0; k < dim; ++k) out_bf16[r * dim + k] = F32ToBf16(total > 0.0f ? acc[k] / total : 0.0f);
    if (lse) lse[r] = total > 0.0f ? big + std::log(total) : -std::numeric_limits<float>::infinity();
  }
}

int32_t kvo_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void kvo_set_num_threads(int32_t n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// ---------------------------------------------------------------------------------------------
// KV block bookkeeping model. The reference reserves one block table per step and never writes it
// (src/memory/static_arena_manager.cpp:298, 581-582; slot = position, src/pipeline/pipeline.cpp:517),
// so batched tables, a free list and admission / release have no counterpart there; the closest
// reference pattern is the expert slot pool with its invariant check
// (src/memory/exclusive_staging.cpp:313-399, 529-572). This model defines the semantics the product's
// fixed-capacity block pool must reproduce bit for bit:
//   * the free list is a FIFO queue, initialised to the caller's order;
//   * grow(seq, n): while the table is too short for len + n tokens, pop the queue head and append
//     it to the table; token j's slot is table[j / bs] * bs + j % bs; all-or-nothing when the queue
//     runs short (returns -1, no change);
//   * release(seq): push the table's blocks to the queue tail in table order, clear the row to 0.
// Deliberately written with growable std containers, unlike the product.
// ---------------------------------------------------------------------------------------------
struct KvoBook {
  int32_t num_blocks;
  int32_t block_size;
  int32_t max_seqs;
  int32_t max_blocks_per_seq;
  std::deque<int32_t> free_list;
  std::vector<std::vector<int32_t>> tables;
  std::vector<int64_t> lens;
  std::vector<uint8_t> live;
};

KvoBook* kvo_book_create(int32_t num_blocks, int32_t block_size, int32_t max_seqs, int32_t max_blocks_per_seq,
                         const int32_t* free_order) {
  auto* book = new KvoBook();
  book->num_blocks = num_blocks;
  book->block_size = block_size;
  book->max_seqs = max_seqs;
  book->max_blocks_per_seq = max_blocks_per_seq;
  for (int32_t i = 0; i < num_blocks; ++i) book->free_list.push_back(free_order ? free_order[i] : i);
  book->tables.resize(static_cast<size_t>(max_seqs));
  book->lens.assign(static_cast<size_t>(max_seqs), 0);
  book->live.assign(static_cast<size_t>(max_seqs), 0);
  return book;
}

void kvo_book_destroy(KvoBook* book) { delete book; }

int32_t kvo_book_admit(KvoBook* book, int32_t seq) {
  if (seq < 0 || seq >= book->max_seqs || book->live[seq]) return -1;
  book->live[seq] = 1;
  book->lens[seq] = 0;
  book->tables[seq].clear();
  return 0;
}

// Grows sequence `seq` by n tokens; writes their slots to slots_out[0..n). Returns 0, or -1 with no
// state change (unknown sequence, table row too short, or free list too short).
int32_t kvo_book_grow(KvoBook* book, int32_t seq, int32_t n_tokens, int32_t* slots_out) {
  if (seq < 0 || seq >= book->max_seqs || !book->live[seq] || n_tokens < 0) return -1;
  const int64_t new_len = book->lens[seq] + n_tokens;
  const int64_t need = (new_len + book->block_size - 1) / book->block_size;
  const int64_t have = static_cast<int64_t>(book->tables[seq].size());
  if (need > book->max_blocks_per_seq) return -1;
  if (need - have > static_cast<int64_t>(book->free_list.size())) return -1;
  for (int64_t i = have; i < need; ++i) {
    book->tables[seq].push_back(book->free_list.front());
    book->free_list.pop_front();
  }
  for (int64_t j = book->lens[seq]; j < new_len; ++j) {
    const int64_t block = book->tables[seq][static_cast<size_t>(j / book->block_size)];
    slots_out[j - book->lens[seq]] = static_cast<int32_t>(block * book->block_size + j % book->block_size);
  }
  book->lens[seq] = new_len;
  return 0;
}

int32_t kvo_book_release(KvoBook* book, int32_t seq) {
  if (seq < 0 || seq >= book->max_seqs || !book->live[seq]) return -1;
  for (int32_t block : book->tables[seq]) book->free_list.push_back(block);
  book->tables[seq].clear();
  book->lens[seq] = 0;
  book->live[seq] = 0;
  return 0;
}

int32_t kvo_book_free_count(const KvoBook* book) { return static_cast<int32_t>(book->free_list.size()); }

// Exports the dense table [max_seqs][max_blocks_per_seq] (unused entries 0, matching the arena's
// zero fill, src/memory/static_arena.cpp:114-116), the lengths, and the free list in queue order.
void kvo_book_export(const KvoBook* book, int32_t* table, int32_t* lens, int32_t* free_out) {
  std::fill(table, table + static_cast<int64_t>(book->max_seqs) * book->max_blocks_per_seq, 0);
  for (int32_t s = 0; s < book->max_seqs; ++s) {
    for (size_t i = 0; i < book->tables[s].size(); ++i) table[s * book->max_blocks_per_seq + i] = book->tables[s][i];
    lens[s] = static_cast<int32_t>(book->lens[s]);
  }
  for (size_t i = 0; i < book->free_list.size(); ++i) free_out[i] = book->free_list[i];
}

}  // extern "C"
