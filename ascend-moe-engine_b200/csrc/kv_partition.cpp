// Host-side work partition for multi-GPU decode. The reference runs on one device
// (include/moe/core/config.hpp:280) and has no counterpart; these are the two ways the path shards:
//   * batched decode: whole sequences go to ranks (no exchange on the data path);
//   * one long sequence: its block range is cut into contiguous shards, each rank attends over its
//     shard and the partial (m, l, O) triples are merged after one all-gather.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "b200kv.h"

namespace b200kv {
void SetLastError(const char* fmt, ...);
}
using b200kv::SetLastError;

// Longest-processing-time greedy: sequences in order of decreasing length (ties: lower index first)
// each go to the rank with the least tokens so far (ties: lower rank). rank_of_seq[i] receives the rank.
extern "C" int32_t b200kv_partition_sequences(const int32_t* kv_len, int32_t n_seqs, int32_t n_ranks,
                                              int32_t* rank_of_seq, int64_t* tokens_per_rank) {
  if (kv_len == nullptr || rank_of_seq == nullptr) {
    SetLastError("partition_sequences: null kv_len or rank_of_seq");
    return B200KV_ERR_NULLPTR;
  }
  if (n_seqs < 0 || n_ranks <= 0) {
    SetLastError("partition_sequences refused: %d sequences over %d ranks", n_seqs, n_ranks);
    return B200KV_ERR_INVALID;
  }
  std::vector<int32_t> order(static_cast<size_t>(n_seqs));
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return kv_len[a] > kv_len[b]; });
  std::vector<int64_t> load(static_cast<size_t>(n_ranks), 0);
  for (int32_t seq : order) {
    const int32_t rank = static_cast<int32_t>(std::min_element(load.begin(), load.end()) - load.begin());
    rank_of_seq[seq] = rank;
    load[static_cast<size_t>(rank)] += kv_len[seq];
  }
  if (tokens_per_rank != nullptr) std::copy(load.begin(), load.end(), tokens_per_rank);
  return B200KV_OK;
}

// Shard `rank` of `n_ranks` of a sequence of kv_len tokens: contiguous block ranges of near-equal block
// counts (the first blocks % n_ranks shards hold one more block). begin is a multiple of block_size.
extern "C" int32_t b200kv_split_kv_range(int32_t kv_len, int32_t block_size, int32_t n_ranks, int32_t rank,
                                         int32_t* begin, int32_t* len) {
  if (begin == nullptr || len == nullptr) {
    SetLastError("split_kv_range: null output");
    return B200KV_ERR_NULLPTR;
  }
  if (kv_len < 0 || block_size <= 0 || n_ranks <= 0 || rank < 0 || rank >= n_ranks) {
    SetLastError("split_kv_range refused: len %d block %d rank %d of %d", kv_len, block_size, rank, n_ranks);
    return B200KV_ERR_INVALID;
  }
  const int64_t blocks = (static_cast<int64_t>(kv_len) + block_size - 1) / block_size;
  const int64_t base = blocks / n_ranks, extra = blocks % n_ranks;
  const int64_t first_block = rank * base + std::min<int64_t>(rank, extra);
  const int64_t n_blocks = base + (rank < extra ? 1 : 0);
  const int64_t b = first_block * block_size;
  const int64_t e = std::min<int64_t>(kv_len, (first_block + n_blocks) * block_size);
  *begin = static_cast<int32_t>(std::min<int64_t>(b, kv_len));
  *len = static_cast<int32_t>(std::max<int64_t>(0, e - b));
  return B200KV_OK;
}
