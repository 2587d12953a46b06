// Sparse-selection indexer in front of attention: for every sequence, the k tokens of its paged history
// that score highest against the step's index query,
//   score_t = sum_h w_h * ReLU(qs_h * ks_t * (Q_h . K_t)),   Q_h, K_t FP8 E4M3 vectors of 128,
// as token positions, best first. The reference vendors this operator (aclnnQuantLightningIndexer) and
// plans it but does not apply it (include/moe/pipeline/pipeline.hpp:57-66). The positions go to
// b200kv_resolve_rows and from there to the decode attention over single-row blocks.
//
// First version, on CUDA cores: correctness and a defined result come first here. The arithmetic is fixed
// to the operation (one thread owns a token and runs the same fp32 fma chains as the CPU statement: over
// d = 0..127 for each head, then over the heads), so scores are bit-identical with the oracle and the
// selection is exact: tokens are ordered by (score descending, position ascending) with a bitonic sort of
// 64-bit keys in shared memory, 4,096 candidates at a time merged with the best k so far.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200kv {
namespace {

constexpr int kIndexDim = 128;
constexpr int kMaxIndexHeads = 64;
constexpr int kScoreThreads = 128;
constexpr int kSortThreads = 1024;
constexpr int kSortSlots = 8192;   // keys sorted at once: 4,096 new candidates + up to 2,048 kept, padded
constexpr int kChunk = 4096;
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

constexpr uint64_t kEmptyKey = ~0ull;  // sorts last

// One CTA per sequence: candidates come in chunks of 4,096, the best k so far stay in the first k slots.
__global__ void __launch_bounds__(kSortThreads)
    IndexerTopkKernel(const float* scores, int64_t score_stride, const int32_t* kv_len, int32_t k, int32_t* index,
                      int32_t* n_selected) {
  GridDependencyTrigger();
  GridDependencyWait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);  // [kSortSlots]
  const int b = blockIdx.x;
  const int len = kv_len[b];
  const int tid = threadIdx.x;
  for (int i = tid; i < kSortSlots; i += kSortThreads) keys[i] = kEmptyKey;
  __syncthreads();
  for (int c0 = 0; c0 < len; c0 += kChunk) {
    // slots [0, k) hold the best so far (or empties); the chunk goes to [kMaxK, kMaxK + kChunk)
    for (int i = tid; i < kChunk; i += kSortThreads) {
      const int t = c0 + i;
      keys[kMaxK + i] = t < len ? SortKey(scores[b * score_stride + t], static_cast<uint32_t>(t)) : kEmptyKey;
    }
    for (int i = k + tid; i < kMaxK; i += kSortThreads) keys[i] = kEmptyKey;
    for (int i = kMaxK + kChunk + tid; i < kSortSlots; i += kSortThreads) keys[i] = kEmptyKey;
    __syncthreads();
    // Bitonic sort, ascending, of the populated prefix rounded up to a power of two: the first chunk has no
    // kept keys in front of it, so it is sorted on its own (in place at kMaxK, then moved to the front).
    const bool first = c0 == 0;
    uint64_t* base = first ? keys + kMaxK : keys;
    const int n_sort = first ? kChunk : kSortSlots;
    for (int size = 2; size <= n_sort; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = tid; i < n_sort / 2; i += kSortThreads) {
          const int lo = 2 * i - (i & (stride - 1));  // index of the pair's lower element
          const int hi = lo + stride;
          const bool ascending = (lo & size) == 0;
          const uint64_t a = base[lo], c = base[hi];
          if ((a > c) == ascending) {
            base[lo] = c;
            base[hi] = a;
          }
        }
        __syncthreads();
      }
    }
    if (first) {  // the best k of the first chunk to the front (k <= kMaxK: source and destination do not overlap)
      for (int i = tid; i < k; i += kSortThreads) keys[i] = keys[kMaxK + i];
      __syncthreads();
    }
  }
  const int kept = len < k ? len : k;
  for (int i = tid; i < k; i += kSortThreads) {
    index[b * k + i] = i < kept ? static_cast<int32_t>(keys[i] & 0xffffffffu) : -1;
  }
  if (tid == 0) n_selected[b] = kept;
}

}  // namespace
}  // namespace b200kv

using namespace b200kv;

extern "C" size_t b200kv_indexer_workspace_bytes(int32_t batch, int64_t max_kv_len) {
  if (batch <= 0 || max_kv_len <= 0) return 0;
  return static_cast<size_t>(batch) * static_cast<size_t>((max_kv_len + 3) & ~3ll) * sizeof(float);
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
  static thread_local int configured_device = -1;
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device != configured_device) {
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(IndexerTopkKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    kSortSlots * 8),
                               "indexer top-k smem opt-in")) {
      return rc;
    }
    configured_device = device;
  }
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
  p.score_stride = (a.max_kv_len + 3) & ~3ll;
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>((a.max_kv_len + kScoreThreads - 1) / kScoreThreads), static_cast<unsigned>(a.batch));
  if (int32_t rc = CheckCuda(LaunchOverlapped(IndexerScoreKernel, grid, dim3(kScoreThreads), 0, s, p), "indexer score launch")) {
    return rc;
  }
  return CheckCuda(LaunchOverlapped(IndexerTopkKernel, dim3(static_cast<unsigned>(a.batch)), dim3(kSortThreads),
                                    static_cast<size_t>(kSortSlots) * 8, s, static_cast<const float*>(p.scores), p.score_stride,
                                    a.kv_len, a.k, a.index_out, a.n_selected_out),
                   "indexer top-k launch");
}
