// Sparse-selection indexer in front of attention: for every sequence, the k tokens of its paged history
// that score highest against the step's index query,
//   score_t = sum_h w_h * ReLU(qs_h * ks_t * (Q_h . K_t)),   Q_h, K_t FP8 E4M3 vectors of 128,
// as token positions, best first. The reference vendors this operator (aclnnQuantLightningIndexer) and
// plans it but does not apply it (include/moe/pipeline/pipeline.hpp:57-66). The positions go to
// b200kv_resolve_rows and from there to the decode attention over single-row blocks.
//
// The score kernel in this file runs on CUDA cores and is the reproducible one (the tensor-core score kernel
// is kv_indexer_tc.cu; b200kv_indexer_topk chooses). The arithmetic is fixed
// to the operation (one thread owns a token and runs the same fp32 fma chains as the CPU statement: over
// d = 0..127 for each head, then over the heads), so scores are bit-identical with the oracle and the
// selection is exact: tokens are ordered by (score descending, position ascending) as 64-bit keys; a radix
// select finds the k-th key and a bitonic sort in shared memory orders the k that are taken.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200kv {
namespace {

constexpr int kIndexDim = 128;
constexpr int kMaxIndexHeads = 64;
constexpr int kScoreThreads = 128;
constexpr int kSortThreads = 1024;
constexpr int kMaxK = 2048;

__device__ __forceinline__ float E4m3ToFloat(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

struct ScoreParams {
  const uint8_t* q;        // [B][heads][128] fp8
  const float* q_scale;    // [B][heads]
  const __nv_bfloat16* w;  // [B][heads]
  int32_t heads;
  const uint8_t* key_pool;  // [rows][key_stride] fp8
  int64_t key_stride;
  const float* k_scale;  // [rows]
  int64_t pool_rows;
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  int32_t block_size;
  float* scores;  // [B][score_stride]
  int64_t score_stride;
  int32_t* status;
};

// Grid (token tiles of 128, sequence). The sequence's query (as fp32) and per-head coefficients sit in
// shared memory; a thread keeps its token's key row in registers and runs the chains.
__global__ void __launch_bounds__(kScoreThreads) IndexerScoreKernel(ScoreParams p) {
  GridDependencyTrigger();
  GridDependencyWait();
  __shared__ __align__(16) float q_s[kMaxIndexHeads * kIndexDim];
  __shared__ float qs_s[kMaxIndexHeads];
  __shared__ float w_s[kMaxIndexHeads];
  const int b = blockIdx.y;
  const int len = p.kv_len[b];
  const int t0 = blockIdx.x * kScoreThreads;
  if (t0 >= len) return;
  for (int i = threadIdx.x; i < p.heads * kIndexDim; i += kScoreThreads) {
    q_s[i] = E4m3ToFloat(p.q[static_cast<int64_t>(b) * p.heads * kIndexDim + i]);
  }
  for (int i = threadIdx.x; i < p.heads; i += kScoreThreads) {
    qs_s[i] = p.q_scale[b * p.heads + i];
    w_s[i] = __bfloat162float(p.w[b * p.heads + i]);
  }
  __syncthreads();
  const int t = t0 + threadIdx.x;
  if (t >= len) return;
  const int64_t column = t / p.block_size;
  const int64_t block = column < p.max_blocks ? p.block_table[static_cast<int64_t>(b) * p.max_blocks + column] : -1;
  const int64_t row = block * p.block_size + t % p.block_size;
  if (block < 0 || row >= p.pool_rows) {
    RecordError(p.status, B200KV_DEV_BAD_BLOCK, b, static_cast<int32_t>(column), static_cast<int32_t>(block));
    p.scores[b * p.score_stride + t] = -INFINITY;
    return;
  }
  float k[kIndexDim];
  {
    const int4* src = reinterpret_cast<const int4*>(p.key_pool + row * p.key_stride);
#pragma unroll
    for (int c = 0; c < kIndexDim / 16; ++c) {
      const int4 v = src[c];
      const uint32_t words[4] = {static_cast<uint32_t>(v.x), static_cast<uint32_t>(v.y), static_cast<uint32_t>(v.z),
                                 static_cast<uint32_t>(v.w)};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) k[16 * c + 4 * j + e] = E4m3ToFloat((words[j] >> (8 * e)) & 0xffu);
      }
    }
  }
  const float ks = p.k_scale[row];
  float score = 0.0f;
  for (int h = 0; h < p.heads; ++h) {
    const float4* qh = reinterpret_cast<const float4*>(q_s + h * kIndexDim);
    float dot = 0.0f;
#pragma unroll
    for (int d4 = 0; d4 < kIndexDim / 4; ++d4) {
      const float4 qv = qh[d4];
      dot = __fmaf_rn(qv.x, k[4 * d4], dot);
      dot = __fmaf_rn(qv.y, k[4 * d4 + 1], dot);
      dot = __fmaf_rn(qv.z, k[4 * d4 + 2], dot);
      dot = __fmaf_rn(qv.w, k[4 * d4 + 3], dot);
    }
    const float scaled = __fmul_rn(__fmul_rn(qs_s[h], ks), dot);
    const float s = scaled > 0.0f ? scaled : 0.0f;
    score = __fmaf_rn(w_s[h], s, score);
  }
  p.scores[b * p.score_stride + t] = score;
}

// Key that sorts ascending into (score descending, position ascending): high word = the complement of the
// score's order-preserving integer image, low word = the position. A NaN score counts as -infinity; +0 and
// -0 compare equal.
__device__ __forceinline__ uint64_t SortKey(float score, uint32_t position) {
  if (score != score) score = -INFINITY;
  score += 0.0f;
  uint32_t bits = __float_as_uint(score);
  bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // ascending with the value
  return (static_cast<uint64_t>(~bits) << 32) | position;
}

// One CTA per sequence. The k best tokens are the k smallest 64-bit keys, all distinct. A radix select finds
// the k-th smallest key: the key's bits from the top in digits of 11, 11, 10 (the score) and 11, 11, 10 (the
// position), each pass a histogram of the digit over the tokens that match the digits found so far, a block scan
// of the histogram, and the digit in which the wanted rank falls. The passes stop as soon as every token that
// still matches is wanted (with distinct scores: after the three score digits). Tokens whose key is at most
// the one found are then collected, exactly k of them, and sorted (bitonic, the short-range steps on registers).
// A thread keeps the score images of its first eight tokens
// in registers, so sequences of up to 8,192 tokens are read from memory once; work is linear in the length.
constexpr int kRadixBins = 2048;
constexpr int kBinsPerThread = kRadixBins / kSortThreads;
constexpr int kHeldPerThread = 8;
constexpr int kSelectChunk = kHeldPerThread * kSortThreads;  // 8,192 tokens: what one CTA reads once and keeps

// Long sequences in two levels, so that more than one CTA works on a sequence: the k best of every chunk of
// 8,192 tokens (kLevel 1: one CTA a chunk, its keys written unsorted to the candidate area), then the k best
// of the candidates (kLevel 2: one CTA a sequence, elements are the 64-bit keys themselves). The k best of the
// whole are among the k best of each chunk, so the result is that of one level (kLevel 0), which sequences of
// up to a chunk use.
struct SelectParams {
  const float* scores;
  int64_t score_stride;
  const int32_t* kv_len;
  int32_t k;
  int32_t chunks;           // per sequence (levels 1 and 2)
  uint64_t* candidates;     // [batch][chunks][k] keys (levels 1 and 2)
  int32_t* index;           // [batch][k]
  int32_t* n_selected;      // [batch]
  const int32_t* block_table;
  int64_t max_blocks;
  int32_t block_size;
  int64_t pool_rows;
  int32_t* rows_out;        // [batch][k] or null
  int32_t* status;
};

template <int kLevel>
__global__ void __launch_bounds__(kSortThreads) IndexerSelectKernel(SelectParams p) {
  GridDependencyTrigger();
  __shared__ uint64_t keys[kMaxK];
  __shared__ uint32_t hist[kRadixBins];
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t chosen[2][3];  // per pass parity: digit, elements before it, elements in it
  __shared__ uint32_t n_taken;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < kRadixBins; i += kSortThreads) hist[i] = 0;
  if (tid == 0) n_taken = 0;
  GridDependencyWait();
  const int b = kLevel == 1 ? blockIdx.y : blockIdx.x;
  const int chunk = kLevel == 1 ? blockIdx.x : 0;
  const int len = p.kv_len[b];
  const int k = p.k;
  // The elements this CTA selects among, n of them, and how many it keeps.
  const int first = kLevel == 1 ? chunk * kSelectChunk : 0;  // first token (levels 0 and 1)
  int n;
  if (kLevel == 0) {
    n = len;
  } else if (kLevel == 1) {
    n = len - first < kSelectChunk ? len - first : kSelectChunk;
    if (n < 0) n = 0;
  } else {
    n = p.chunks * k;
  }
  const int kept = kLevel == 2 ? (len < k ? len : k) : (n < k ? n : k);
  const float* row = p.scores + b * p.score_stride + first;
  const uint64_t* cand_in = p.candidates + static_cast<int64_t>(b) * p.chunks * k;
  uint64_t* cand_out = p.candidates + (static_cast<int64_t>(b) * p.chunks + chunk) * k;
  if (kLevel != 1) {
    if (tid == 0) p.n_selected[b] = kept;
    for (int i = kept + tid; i < k; i += kSortThreads) {
      p.index[b * k + i] = -1;
      if (p.rows_out != nullptr) p.rows_out[b * k + i] = -1;
    }
  } else {
    for (int i = kept + tid; i < k; i += kSortThreads) cand_out[i] = ~0ull;  // empties sort last
  }
  if (kept == 0) return;
  // Levels 0 and 1: the high word of the key (ascending = better) of this thread's elements tid, tid + 1024, ...,
  // the first eight held in registers. Level 2 reads its few keys from memory every time.
  uint32_t held[kHeldPerThread];
  if (kLevel != 2) {
#pragma unroll
    for (int j = 0; j < kHeldPerThread; ++j) {
      const int e = tid + j * kSortThreads;
      held[j] = e < n ? static_cast<uint32_t>(SortKey(row[e], 0u) >> 32) : 0u;
    }
  }
  auto held_key = [&](int j, int e) -> uint64_t {  // j = e / 1024 (compile-time inside unrolled loops)
    return (static_cast<uint64_t>(held[j]) << 32) | static_cast<uint32_t>(first + e);
  };
  auto read_key = [&](int e) -> uint64_t {
    return kLevel == 2 ? cand_in[e] : SortKey(row[e], static_cast<uint32_t>(first + e));
  };
  constexpr int kFirstRead = kLevel == 2 ? 0 : kSelectChunk;  // elements from here on are read, not held
  __syncthreads();  // the histogram is clear

  uint64_t bound = ~0ull;  // every element is wanted when there are at most `kept`
  if (n > kept) {
    uint64_t prefix = 0, mask = 0;
    uint32_t rank = static_cast<uint32_t>(kept);  // 1-based rank, among the elements that match `prefix`, of the key wanted
    for (int pass = 0; pass < 6; ++pass) {
      const int shift = pass == 0 ? 53 : pass == 1 ? 42 : pass == 2 ? 32 : pass == 3 ? 21 : pass == 4 ? 10 : 0;
      const uint32_t digit_mask = (pass == 2 || pass == 5) ? 1023u : 2047u;
      // (Scores of one sequence are close together, so in the top digits most tokens fall into a few bins;
      // shared-memory atomics on one address still cost less here than finding a warp's equal digits first with
      // match.any, which was measured: 2.5 us more per launch.)
      if (kLevel != 2) {
#pragma unroll
        for (int j = 0; j < kHeldPerThread; ++j) {
          const int e = tid + j * kSortThreads;
          if (e < n) {
            const uint64_t key = held_key(j, e);
            if ((key & mask) == prefix) atomicAdd(&hist[static_cast<uint32_t>(key >> shift) & digit_mask], 1u);
          }
        }
      }
      for (int e = tid + kFirstRead; e < n; e += kSortThreads) {
        const uint64_t key = read_key(e);
        if ((key & mask) == prefix) atomicAdd(&hist[static_cast<uint32_t>(key >> shift) & digit_mask], 1u);
      }
      __syncthreads();
      // A thread owns a few consecutive bins (and clears them for the next pass); a scan over the threads gives the
      // elements before its bins: shuffles inside the warp, and every warp adds up the warps before it for itself.
      uint32_t count[kBinsPerThread], mine = 0;
#pragma unroll
      for (int i = 0; i < kBinsPerThread; ++i) {
        count[i] = hist[kBinsPerThread * tid + i];
        hist[kBinsPerThread * tid + i] = 0;
        mine += count[i];
      }
      uint32_t incl = mine;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
      }
      if (lane == 31) warp_sum[warp] = incl;
      __syncthreads();
      uint32_t earlier = lane < warp ? warp_sum[lane] : 0u;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) earlier += __shfl_xor_sync(0xffffffffu, earlier, off);
      uint32_t before = earlier + incl - mine;
      if (before < rank && rank <= before + mine) {  // one thread: the rank falls in its bins
#pragma unroll
        for (int i = 0; i < kBinsPerThread; ++i) {
          if (before < rank && rank <= before + count[i]) {
            chosen[pass & 1][0] = kBinsPerThread * tid + i;
            chosen[pass & 1][1] = before;
            chosen[pass & 1][2] = count[i];
          }
          before += count[i];
        }
      }
      __syncthreads();
      prefix |= static_cast<uint64_t>(chosen[pass & 1][0]) << shift;
      mask |= static_cast<uint64_t>(digit_mask) << shift;
      rank -= chosen[pass & 1][1];
      bound = prefix;  // after the last pass the prefix is the key itself
      if (rank == chosen[pass & 1][2]) {  // all that still match are wanted: the bound is the largest key with this prefix
        bound = prefix | ~mask;
        break;
      }
    }
  }
  // Exactly `kept` keys are at most the bound. A warp reserves the slots of its takers with one addition.
  auto take = [&](bool wanted, uint64_t key) {  // every lane of the warp calls
    const unsigned takers = __ballot_sync(0xffffffffu, wanted);
    if (takers == 0u) return;
    uint32_t slot0 = 0;
    if (lane == __ffs(takers) - 1) slot0 = atomicAdd(&n_taken, static_cast<uint32_t>(__popc(takers)));
    slot0 = __shfl_sync(0xffffffffu, slot0, __ffs(takers) - 1);
    const uint32_t slot = slot0 + __popc(takers & ((1u << lane) - 1u));
    if (wanted && slot < static_cast<uint32_t>(kMaxK)) keys[slot] = key;
  };
  if (kLevel != 2) {
#pragma unroll
    for (int j = 0; j < kHeldPerThread; ++j) {
      const int e = tid + j * kSortThreads;
      if (warp * 32 + j * kSortThreads >= n) break;
      const uint64_t key = held_key(j, e);
      take(e < n && key <= bound, key);
    }
  }
  for (int e0 = warp * 32 + kFirstRead; e0 < n; e0 += kSortThreads) {
    const int e = e0 + lane;
    const uint64_t key = e < n ? read_key(e) : ~0ull;
    take(e < n && key <= bound, key);
  }
  __syncthreads();
  if (kLevel == 1) {  // the chunk's best, in any order: the next level selects and sorts
    for (int i = tid; i < kept; i += kSortThreads) cand_out[i] = keys[i];
    return;
  }
  // The collected keys in order: a bitonic sort, ascending, of the list padded to a power of two. Element e
  // belongs to thread e % 1024 (two elements a thread when k > 1024). Steps whose partner is less than 32 away
  // stay inside a warp and run on registers with shuffles, a whole run of them between two barriers; only the
  // steps with a partner 32 or more away (10 of the 45 for 512 keys) go through shared memory.
  int padded = 32;
  while (padded < kept) padded <<= 1;
  for (int i = kept + tid; i < padded; i += kSortThreads) keys[i] = ~0ull;
  __syncthreads();
  for (int size = 2; size <= padded; size <<= 1) {
    int stride = size >> 1;
    for (; stride >= 32; stride >>= 1) {
      for (int i = tid; i < padded / 2; i += kSortThreads) {
        const int lo = 2 * i - (i & (stride - 1));  // index of the pair's lower element
        const int hi = lo + stride;
        const bool ascending = (lo & size) == 0;
        const uint64_t a = keys[lo], c = keys[hi];
        if ((a > c) == ascending) {
          keys[lo] = c;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
    for (int e = tid; e < padded; e += kSortThreads) {  // the same trip count for every lane of a warp
      uint64_t mine = keys[e];
      const bool ascending = (e & size) == 0;
      for (int s2 = stride; s2 > 0; s2 >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, mine, s2);
        const bool lower = (e & s2) == 0;  // this element is the pair's lower one
        const bool take_other = lower ? ((mine > other) == ascending) : ((other > mine) == ascending);
        if (take_other) mine = other;
      }
      keys[e] = mine;
    }
    __syncthreads();
  }
  for (int i = tid; i < kept; i += kSortThreads) {
    const int32_t t = static_cast<int32_t>(keys[i] & 0xffffffffu);
    p.index[b * k + i] = t;
    if (p.rows_out != nullptr) {  // the selection as pool rows, what ResolveRowsKernel would make of it
      const int64_t column = t / p.block_size;
      const int64_t block = column < p.max_blocks ? p.block_table[static_cast<int64_t>(b) * p.max_blocks + column] : -1;
      const int64_t r = block * p.block_size + t % p.block_size;
      int32_t out_row = -1;
      if (block < 0 || r >= p.pool_rows) {
        RecordError(p.status, B200KV_DEV_BAD_BLOCK, b, i, t);
      } else {
        out_row = static_cast<int32_t>(r);
      }
      p.rows_out[b * k + i] = out_row;
    }
  }
}

}  // namespace
}  // namespace b200kv

namespace b200kv {
bool IndexerTcSupports(int32_t heads, int32_t block_size, int64_t key_stride, int64_t pool_rows);
int32_t LaunchIndexerScoreTc(const void* q, const float* q_scale, const void* weights, int32_t heads, const void* key_pool,
                             int64_t key_stride, const float* k_scale, int64_t pool_rows, const int32_t* block_table,
                             int64_t max_blocks, const int32_t* kv_len, int32_t batch, int32_t block_size, int64_t max_kv_len,
                             float* scores, int64_t score_stride, cudaStream_t stream, int32_t* status);
}  // namespace b200kv

using namespace b200kv;

namespace {
// Scores [batch][stride] fp32, then (sequences longer than one chunk) the candidate keys [batch][chunks][kMaxK].
int64_t ScoreStrideOf(int64_t max_kv_len) { return (max_kv_len + 3) & ~3ll; }
int64_t ChunksOf(int64_t max_kv_len) { return (max_kv_len + kSelectChunk - 1) / kSelectChunk; }
size_t ScoreBytesOf(int32_t batch, int64_t max_kv_len) {
  return (static_cast<size_t>(batch) * static_cast<size_t>(ScoreStrideOf(max_kv_len)) * sizeof(float) + 15) & ~static_cast<size_t>(15);
}
}  // namespace

extern "C" size_t b200kv_indexer_workspace_bytes(int32_t batch, int64_t max_kv_len) {
  if (batch <= 0 || max_kv_len <= 0) return 0;
  const int64_t chunks = ChunksOf(max_kv_len);
  return ScoreBytesOf(batch, max_kv_len) +
         (chunks > 1 ? static_cast<size_t>(batch) * static_cast<size_t>(chunks) * kMaxK * sizeof(uint64_t) : 0);
}

extern "C" int32_t b200kv_indexer_topk(const b200kv_indexer_args* args, void* stream, b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_indexer_topk")) return rc;
  if (args == nullptr) {
    SetLastError("indexer_topk: args is null");
    return B200KV_ERR_NULLPTR;
  }
  const b200kv_indexer_args& a = *args;
  if (a.batch == 0) return B200KV_OK;
  if (a.q == nullptr || a.q_scale == nullptr || a.weights == nullptr || a.key_pool == nullptr || a.k_scale == nullptr ||
      a.block_table == nullptr || a.kv_len == nullptr || a.index_out == nullptr || a.n_selected_out == nullptr ||
      a.workspace == nullptr) {
    SetLastError("indexer_topk: q, q_scale, weights, key_pool, k_scale, block_table, kv_len, outputs and workspace must "
                 "be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (a.batch < 0 || a.heads < 1 || a.heads > kMaxIndexHeads || a.k < 1 || a.k > kMaxK || a.block_size <= 0 ||
      a.max_blocks <= 0 || a.max_kv_len <= 0 || a.pool_rows <= 0 || a.key_stride < kIndexDim || a.key_stride % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(a.key_pool) & 15u) != 0 ||
      a.workspace_bytes < b200kv_indexer_workspace_bytes(a.batch, a.max_kv_len)) {
    SetLastError("indexer_topk refused: batch %d, heads %d (1..%d), k %d (1..%d), block_size %d, max_kv_len %lld, key stride "
                 "%lld (>= 128, multiple of 16, 16-byte aligned pool), workspace %zu of %zu bytes",
                 a.batch, a.heads, kMaxIndexHeads, a.k, kMaxK, a.block_size, static_cast<long long>(a.max_kv_len),
                 static_cast<long long>(a.key_stride), a.workspace_bytes,
                 b200kv_indexer_workspace_bytes(a.batch, a.max_kv_len));
    return B200KV_ERR_INVALID;
  }
  const bool tc_ok = IndexerTcSupports(a.heads, a.block_size, a.key_stride, a.pool_rows) &&
                     (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0;  // its TMA loads want a 16-byte aligned query
  if ((a.variant != B200KV_INDEXER_AUTO && a.variant != B200KV_INDEXER_EXACT && a.variant != B200KV_INDEXER_TCGEN05) ||
      (a.variant == B200KV_INDEXER_TCGEN05 && !tc_ok)) {
    SetLastError("indexer_topk refused: variant %d (the tensor-core score kernel needs heads <= 64, block_size %% 64 == 0 and a "
                 "16-byte aligned q; heads %d, block_size %d)", a.variant, a.heads, a.block_size);
    return B200KV_ERR_INVALID;
  }
  const bool use_tc = tc_ok && a.variant != B200KV_INDEXER_EXACT;
  ScoreParams p{};
  p.q = static_cast<const uint8_t*>(a.q);
  p.q_scale = a.q_scale;
  p.w = static_cast<const __nv_bfloat16*>(a.weights);
  p.heads = a.heads;
  p.key_pool = static_cast<const uint8_t*>(a.key_pool);
  p.key_stride = a.key_stride;
  p.k_scale = a.k_scale;
  p.pool_rows = a.pool_rows;
  p.block_table = a.block_table;
  p.max_blocks = a.max_blocks;
  p.kv_len = a.kv_len;
  p.block_size = a.block_size;
  p.scores = static_cast<float*>(a.workspace);
  p.score_stride = ScoreStrideOf(a.max_kv_len);
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_tc) {
    if (int32_t rc = LaunchIndexerScoreTc(a.q, a.q_scale, a.weights, a.heads, a.key_pool, a.key_stride, a.k_scale, a.pool_rows,
                                          a.block_table, a.max_blocks, a.kv_len, a.batch, a.block_size, a.max_kv_len, p.scores,
                                          p.score_stride, s, status)) {
      return rc;
    }
  } else {
    const dim3 grid(static_cast<unsigned>((a.max_kv_len + kScoreThreads - 1) / kScoreThreads), static_cast<unsigned>(a.batch));
    if (int32_t rc = CheckCuda(LaunchOverlapped(IndexerScoreKernel, grid, dim3(kScoreThreads), 0, s, p), "indexer score launch")) {
      return rc;
    }
  }
  SelectParams sp{};
  sp.scores = p.scores;
  sp.score_stride = p.score_stride;
  sp.kv_len = a.kv_len;
  sp.k = a.k;
  sp.chunks = static_cast<int32_t>(ChunksOf(a.max_kv_len));
  sp.candidates = reinterpret_cast<uint64_t*>(static_cast<char*>(a.workspace) + ScoreBytesOf(a.batch, a.max_kv_len));
  sp.index = a.index_out;
  sp.n_selected = a.n_selected_out;
  sp.block_table = a.block_table;
  sp.max_blocks = a.max_blocks;
  sp.block_size = a.block_size;
  sp.pool_rows = a.pool_rows;
  sp.rows_out = a.rows_out;
  sp.status = static_cast<int32_t*>(status);
  if (sp.chunks <= 1) {
    return CheckCuda(LaunchOverlapped(IndexerSelectKernel<0>, dim3(static_cast<unsigned>(a.batch)), dim3(kSortThreads), 0, s, sp),
                     "indexer top-k launch");
  }
  if (int32_t rc = CheckCuda(LaunchOverlapped(IndexerSelectKernel<1>, dim3(static_cast<unsigned>(sp.chunks), static_cast<unsigned>(a.batch)),
                                              dim3(kSortThreads), 0, s, sp),
                             "indexer top-k (chunks) launch")) {
    return rc;
  }
  return CheckCuda(LaunchOverlapped(IndexerSelectKernel<2>, dim3(static_cast<unsigned>(a.batch)), dim3(kSortThreads), 0, s, sp),
                   "indexer top-k (candidates) launch");
}
