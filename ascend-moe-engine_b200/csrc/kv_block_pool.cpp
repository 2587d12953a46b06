// Host bookkeeping for the paged KV pool: a fixed-capacity block allocator with per-sequence block
// tables, plus the reservation arithmetic of the reference arena manager.
//
// Everything is sized at create time and nothing allocates afterwards, the way the reference seals
// its arena before the decode loop (src/memory/static_arena.cpp:301-304, and the zero-allocation
// assertions of src/pipeline/pipeline.cpp:502-503). A call either completes or changes nothing
// (plan, then commit), and Validate() states the failing arithmetic, after the pattern of the
// reference's expert slot pool (src/memory/exclusive_staging.cpp:313-399, 529-572).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <iomanip>
#include <locale>
#include <new>
#include <sstream>
#include <string>

#include "b200kv.h"

namespace b200kv {
void SetLastError(const char* fmt, ...);
}

using b200kv::SetLastError;

struct b200kv_block_pool {
  int32_t num_blocks;
  int32_t block_size;
  int32_t max_seqs;
  int32_t max_blocks_per_seq;
  // Free list: a ring of block ids; [head, head + free_count) modulo num_blocks are free, oldest first.
  int32_t* ring;
  int32_t head;
  int32_t free_count;
  int32_t* table;        // [max_seqs][max_blocks_per_seq], unused entries 0
  int32_t* lens;         // tokens per sequence
  int32_t* used_blocks;  // table entries in use per sequence
  uint8_t* live;
  uint8_t* scratch;      // [num_blocks] ownership marks for Validate
};

extern "C" b200kv_block_pool* b200kv_block_pool_create(int32_t num_blocks, int32_t block_size, int32_t max_seqs,
                                                       int32_t max_blocks_per_seq, const int32_t* free_order) {
  if (num_blocks <= 0 || block_size <= 0 || max_seqs <= 0 || max_blocks_per_seq <= 0 ||
      static_cast<int64_t>(num_blocks) * block_size > INT32_MAX) {
    SetLastError("block pool refused: blocks %d, block_size %d, max_seqs %d, max_blocks_per_seq %d "
                 "(all > 0, blocks*block_size < 2^31 so slots fit int32)",
                 num_blocks, block_size, max_seqs, max_blocks_per_seq);
    return nullptr;
  }
  auto* pool = new (std::nothrow) b200kv_block_pool();
  if (pool == nullptr) return nullptr;
  pool->num_blocks = num_blocks;
  pool->block_size = block_size;
  pool->max_seqs = max_seqs;
  pool->max_blocks_per_seq = max_blocks_per_seq;
  const size_t table_entries = static_cast<size_t>(max_seqs) * max_blocks_per_seq;
  pool->ring = new (std::nothrow) int32_t[num_blocks];
  pool->table = new (std::nothrow) int32_t[table_entries]();
  pool->lens = new (std::nothrow) int32_t[max_seqs]();
  pool->used_blocks = new (std::nothrow) int32_t[max_seqs]();
  pool->live = new (std::nothrow) uint8_t[max_seqs]();
  pool->scratch = new (std::nothrow) uint8_t[num_blocks]();
  if (!pool->ring || !pool->table || !pool->lens || !pool->used_blocks || !pool->live || !pool->scratch) {
    SetLastError("block pool: host allocation failed");
    b200kv_block_pool_destroy(pool);
    return nullptr;
  }
  for (int32_t i = 0; i < num_blocks; ++i) {
    const int32_t id = free_order ? free_order[i] : i;
    if (id < 0 || id >= num_blocks || pool->scratch[id]) {
      SetLastError("block pool: free_order[%d] = %d is out of range or repeated", i, id);
      b200kv_block_pool_destroy(pool);
      return nullptr;
    }
    pool->scratch[id] = 1;
    pool->ring[i] = id;
  }
  std::memset(pool->scratch, 0, static_cast<size_t>(num_blocks));
  pool->head = 0;
  pool->free_count = num_blocks;
  return pool;
}

extern "C" void b200kv_block_pool_destroy(b200kv_block_pool* pool) {
  if (pool == nullptr) return;
  delete[] pool->ring;
  delete[] pool->table;
  delete[] pool->lens;
  delete[] pool->used_blocks;
  delete[] pool->live;
  delete[] pool->scratch;
  delete pool;
}

namespace {
bool SeqInRange(const b200kv_block_pool* pool, int32_t seq, const char* what) {
  if (pool == nullptr) {
    SetLastError("%s: pool is null", what);
    return false;
  }
  if (seq < 0 || seq >= pool->max_seqs) {
    SetLastError("%s: sequence %d outside [0, %d)", what, seq, pool->max_seqs);
    return false;
  }
  return true;
}
}  // namespace

extern "C" int32_t b200kv_block_pool_admit(b200kv_block_pool* pool, int32_t seq) {
  if (!SeqInRange(pool, seq, "admit")) return pool ? B200KV_ERR_INVALID : B200KV_ERR_NULLPTR;
  if (pool->live[seq]) {
    SetLastError("admit: sequence %d is already live with %d tokens", seq, pool->lens[seq]);
    return B200KV_ERR_INVALID;
  }
  pool->live[seq] = 1;
  pool->lens[seq] = 0;
  pool->used_blocks[seq] = 0;
  return B200KV_OK;
}

extern "C" int32_t b200kv_block_pool_grow(b200kv_block_pool* pool, int32_t seq, int32_t n_tokens,
                                          int32_t* slots_out) {
  if (!SeqInRange(pool, seq, "grow")) return pool ? B200KV_ERR_INVALID : B200KV_ERR_NULLPTR;
  if (!pool->live[seq] || n_tokens < 0 || (n_tokens > 0 && slots_out == nullptr)) {
    SetLastError("grow: sequence %d live=%d, n_tokens %d, slots_out %p", seq, static_cast<int>(pool->live[seq]),
                 n_tokens, static_cast<void*>(slots_out));
    return B200KV_ERR_INVALID;
  }
  // Plan: how many blocks the new length needs, refused as a whole when the row or the free list is short.
  const int64_t new_len = static_cast<int64_t>(pool->lens[seq]) + n_tokens;
  const int64_t need = (new_len + pool->block_size - 1) / pool->block_size;
  const int64_t have = pool->used_blocks[seq];
  if (need > pool->max_blocks_per_seq) {
    SetLastError("grow: sequence %d would need %lld blocks for %lld tokens, table row holds %d", seq,
                 static_cast<long long>(need), static_cast<long long>(new_len), pool->max_blocks_per_seq);
    return B200KV_ERR_INVALID;
  }
  if (need - have > pool->free_count) {
    SetLastError("grow: sequence %d needs %lld more blocks, %d free of %d", seq, static_cast<long long>(need - have),
                 pool->free_count, pool->num_blocks);
    return B200KV_ERR_INVALID;
  }
  // Commit.
  int32_t* row = pool->table + static_cast<size_t>(seq) * pool->max_blocks_per_seq;
  for (int64_t i = have; i < need; ++i) {
    row[i] = pool->ring[pool->head];
    pool->head = pool->head + 1 == pool->num_blocks ? 0 : pool->head + 1;
    --pool->free_count;
  }
  pool->used_blocks[seq] = static_cast<int32_t>(need);
  const int32_t old_len = pool->lens[seq];
  for (int32_t k = 0; k < n_tokens; ++k) {
    const int32_t j = old_len + k;
    slots_out[k] = row[j / pool->block_size] * pool->block_size + j % pool->block_size;
  }
  pool->lens[seq] = static_cast<int32_t>(new_len);
  return B200KV_OK;
}

// Takes back the last n_tokens of a sequence and returns the blocks that empties to the FRONT of the free
// list, newest first: undoing the most recent grows in reverse order restores tables, lengths and the free
// list exactly (a step that is abandoned half way leaves no trace).
extern "C" int32_t b200kv_block_pool_ungrow(b200kv_block_pool* pool, int32_t seq, int32_t n_tokens) {
  if (!SeqInRange(pool, seq, "ungrow")) return pool ? B200KV_ERR_INVALID : B200KV_ERR_NULLPTR;
  if (!pool->live[seq] || n_tokens < 0 || n_tokens > pool->lens[seq]) {
    SetLastError("ungrow: sequence %d live=%d holds %d tokens, %d to take back", seq, static_cast<int>(pool->live[seq]),
                 pool->lens[seq], n_tokens);
    return B200KV_ERR_INVALID;
  }
  const int32_t new_len = pool->lens[seq] - n_tokens;
  const int32_t keep = (new_len + pool->block_size - 1) / pool->block_size;
  int32_t* row = pool->table + static_cast<size_t>(seq) * pool->max_blocks_per_seq;
  for (int32_t i = pool->used_blocks[seq] - 1; i >= keep; --i) {
    pool->head = pool->head == 0 ? pool->num_blocks - 1 : pool->head - 1;
    pool->ring[pool->head] = row[i];
    ++pool->free_count;
    row[i] = 0;
  }
  pool->used_blocks[seq] = keep;
  pool->lens[seq] = new_len;
  return B200KV_OK;
}

extern "C" int32_t b200kv_block_pool_release(b200kv_block_pool* pool, int32_t seq) {
  if (!SeqInRange(pool, seq, "release")) return pool ? B200KV_ERR_INVALID : B200KV_ERR_NULLPTR;
  if (!pool->live[seq]) {
    SetLastError("release: sequence %d is not live", seq);
    return B200KV_ERR_INVALID;
  }
  int32_t* row = pool->table + static_cast<size_t>(seq) * pool->max_blocks_per_seq;
  int32_t tail = pool->head + pool->free_count;
  if (tail >= pool->num_blocks) tail -= pool->num_blocks;
  for (int32_t i = 0; i < pool->used_blocks[seq]; ++i) {
    pool->ring[tail] = row[i];
    tail = tail + 1 == pool->num_blocks ? 0 : tail + 1;
    ++pool->free_count;
    row[i] = 0;
  }
  pool->used_blocks[seq] = 0;
  pool->lens[seq] = 0;
  pool->live[seq] = 0;
  return B200KV_OK;
}

extern "C" int32_t b200kv_block_pool_free_count(const b200kv_block_pool* pool) {
  return pool ? pool->free_count : -1;
}

extern "C" int32_t b200kv_block_pool_seq_len(const b200kv_block_pool* pool, int32_t seq) {
  if (!SeqInRange(pool, seq, "seq_len")) return -1;
  return pool->live[seq] ? pool->lens[seq] : -1;
}

extern "C" const int32_t* b200kv_block_pool_table(const b200kv_block_pool* pool) {
  return pool ? pool->table : nullptr;
}

extern "C" const int32_t* b200kv_block_pool_lens(const b200kv_block_pool* pool) { return pool ? pool->lens : nullptr; }

extern "C" int32_t b200kv_block_pool_export_free(const b200kv_block_pool* pool, int32_t* out, int32_t capacity) {
  if (pool == nullptr || out == nullptr) return -1;
  int32_t n = 0;
  int32_t at = pool->head;
  for (; n < pool->free_count && n < capacity; ++n) {
    out[n] = pool->ring[at];
    at = at + 1 == pool->num_blocks ? 0 : at + 1;
  }
  return n;
}

extern "C" int32_t b200kv_block_pool_validate(const b200kv_block_pool* pool) {
  if (pool == nullptr) {
    SetLastError("validate: pool is null");
    return B200KV_ERR_NULLPTR;
  }
  std::memset(pool->scratch, 0, static_cast<size_t>(pool->num_blocks));
  int64_t owned = 0;
  int32_t at = pool->head;
  for (int32_t i = 0; i < pool->free_count; ++i) {
    const int32_t id = pool->ring[at];
    if (id < 0 || id >= pool->num_blocks || pool->scratch[id]) {
      SetLastError("validate: free-list entry %d holds block %d (out of range or listed twice)", i, id);
      return B200KV_ERR_INVALID;
    }
    pool->scratch[id] = 1;
    at = at + 1 == pool->num_blocks ? 0 : at + 1;
  }
  for (int32_t s = 0; s < pool->max_seqs; ++s) {
    const int32_t* row = pool->table + static_cast<size_t>(s) * pool->max_blocks_per_seq;
    if (!pool->live[s]) {
      if (pool->lens[s] != 0 || pool->used_blocks[s] != 0) {
        SetLastError("validate: idle sequence %d keeps %d tokens / %d blocks", s, pool->lens[s], pool->used_blocks[s]);
        return B200KV_ERR_INVALID;
      }
      continue;
    }
    const int64_t need = (static_cast<int64_t>(pool->lens[s]) + pool->block_size - 1) / pool->block_size;
    if (need != pool->used_blocks[s]) {
      SetLastError("validate: sequence %d has %d tokens -> ceil(%d/%d) = %lld blocks, table holds %d", s,
                   pool->lens[s], pool->lens[s], pool->block_size, static_cast<long long>(need), pool->used_blocks[s]);
      return B200KV_ERR_INVALID;
    }
    for (int32_t i = 0; i < pool->used_blocks[s]; ++i) {
      const int32_t id = row[i];
      if (id < 0 || id >= pool->num_blocks || pool->scratch[id]) {
        SetLastError("validate: sequence %d entry %d holds block %d (out of range or owned twice)", s, i, id);
        return B200KV_ERR_INVALID;
      }
      pool->scratch[id] = 1;
      ++owned;
    }
  }
  if (owned + pool->free_count != pool->num_blocks) {
    SetLastError("validate: %lld blocks in tables + %d free != %d total", static_cast<long long>(owned),
                 pool->free_count, pool->num_blocks);
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

extern "C" int32_t b200kv_plan_reservation(int64_t max_context, int64_t block_size, int64_t layers, int64_t max_seqs,
                                           int64_t tokens_per_step, b200kv_reservation* out) {
  if (out == nullptr) {
    SetLastError("plan_reservation: out is null");
    return B200KV_ERR_NULLPTR;
  }
  if (max_context <= 0 || block_size <= 0 || layers <= 0 || max_seqs <= 0 || tokens_per_step <= 0) {
    SetLastError("plan_reservation refused: context %lld, block_size %lld, layers %lld, seqs %lld, tokens/step %lld",
                 static_cast<long long>(max_context), static_cast<long long>(block_size),
                 static_cast<long long>(layers), static_cast<long long>(max_seqs),
                 static_cast<long long>(tokens_per_step));
    return B200KV_ERR_INVALID;
  }
  const int64_t blocks = (max_context + block_size - 1) / block_size;
  out->blocks_per_layer = blocks;
  out->total_blocks = blocks * layers;
  out->latent_bytes = layers * blocks * block_size * B200KV_LATENT_DIM * 2;
  out->rope_bytes = layers * blocks * block_size * B200KV_ROPE_DIM * 2;
  out->block_table_bytes = max_seqs * blocks * 4;
  out->slot_mapping_bytes = tokens_per_step * 4;
  return B200KV_OK;
}

extern "C" double b200kv_utilisation(int64_t active_tokens, int64_t blocks_per_layer, int64_t block_size) {
  const int64_t capacity = blocks_per_layer * block_size;
  return capacity > 0 ? static_cast<double>(active_tokens) / static_cast<double>(capacity) : 0.0;
}

// The "paged_attention" object of the reference's diagnostics file, key for key and with its number
// formatting (std::setprecision(12) in the classic locale; src/diagnostics/inference_stats.cpp:22, 42-47).
extern "C" int64_t b200kv_paged_attention_stats_json(int64_t blocks_per_layer, int64_t layers, int64_t active_tokens,
                                                     int64_t block_size, char* buffer, int64_t capacity) {
  std::ostringstream out;
  out.imbue(std::locale::classic());
  out << std::setprecision(12);
  out << "\"paged_attention\": {\n"
      << "    \"total_blocks_allocated\": " << blocks_per_layer * layers << ",\n"
      << "    \"active_context_tokens\": " << active_tokens << ",\n"
      << "    \"block_size\": " << block_size << ",\n"
      << "    \"kv_cache_utilization\": " << b200kv_utilisation(active_tokens, blocks_per_layer, block_size) << "\n  }";
  const std::string text = out.str();
  if (buffer != nullptr && capacity > 0) {
    const size_t n = text.size() < static_cast<size_t>(capacity - 1) ? text.size() : static_cast<size_t>(capacity - 1);
    std::memcpy(buffer, text.data(), n);
    buffer[n] = '\0';
  }
  return static_cast<int64_t>(text.size());
}
