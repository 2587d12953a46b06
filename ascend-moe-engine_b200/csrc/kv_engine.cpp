// The KV path as the engine drives it, batched: what Dsv4Pipeline::Build and ::DecodeStep do for the paged cache
// and the attention stages (src/pipeline/pipeline.cpp:212-258, 496-537), lifted from one sequence and one token
// per step (src/memory/static_arena_manager.cpp:37-39; src/pipeline/pipeline.cpp:40, 515-519) to max_seqs
// sequences and to prefill chunks of many tokens (apps/moe_runner.cpp:434-439 runs the prompt as P single-token
// steps).
//
//   Build      reserve the KV spans and the step's staging in the static arena, note the attention workspace,
//              ONE commit, the workspace, seal; create the block pool; one pinned staging block for the uploads.
//   step       begin: grow every sequence of the step in the block pool (plan, then commit: a refused growth
//              changes nothing), write the step's table rows, lengths and slots into the pinned block and upload
//              them with ONE copy (the reference's mailbox, :515-519). Then per layer, in the reference's stage
//              order: producer (kv_a_norm + rope + kv_cache_write, stages 6-8), attention (9), MX quantisation of
//              its output (10). end: no allocation happened since begin, as the reference asserts per step
//              (:502-503, 535-536).
// Every device operation is one of the library's own entry points (b200kv_append_fused, b200kv_mla_decode,
// b200kv_mx_quant_e4m3); this file is host logic only and allocates nothing after Build.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "b200kv.h"

namespace b200kv {
void SetLastError(const char* fmt, ...);
int32_t CheckCuda(cudaError_t err, const char* what);
int32_t FaultCheck(const char* entry_point);
}  // namespace b200kv

using b200kv::CheckCuda;
using b200kv::SetLastError;

struct b200kv_engine {
  b200kv_engine_config cfg{};
  b200kv_arena* arena = nullptr;
  b200kv_kv_cache cache{};
  b200kv_block_pool* pool = nullptr;
  int64_t status_handle = -1;
  // Device addresses of the step's spans (resolved once, after Commit).
  int32_t* d_table = nullptr;
  int32_t* d_slots = nullptr;
  int32_t* d_lens = nullptr;
  int32_t* d_status = nullptr;
  // One pinned block that mirrors [table .. lens] of the arena byte for byte: one copy uploads a step.
  unsigned char* staging = nullptr;
  size_t staging_bytes = 0;
  size_t table_off = 0, slots_off = 0, lens_off = 0;
  // The step in flight.
  bool in_step = false;
  int32_t step_seqs = 0;
  int32_t step_tokens = 0;
  int32_t allocations_at_begin = 0;
  int64_t steps = 0;
  int64_t active_tokens = 0;
  std::vector<int32_t> step_seq_ids;   // sized at Build: the step's sequences and by how much each grew
  std::vector<int32_t> step_grown;
};

namespace {

int32_t Refuse(const char* text) {
  SetLastError("%s", text);
  return B200KV_ERR_INVALID;
}

}  // namespace

extern "C" b200kv_engine* b200kv_engine_create(const b200kv_engine_config* config) {
  if (config == nullptr) {
    SetLastError("engine_create: config is null");
    return nullptr;
  }
  const b200kv_engine_config& c = *config;
  if (c.layers <= 0 || c.max_seqs <= 0 || c.num_blocks <= 0 || c.block_size <= 0 || c.block_size % 64 != 0 ||
      c.max_blocks_per_seq <= 0 || c.max_step_tokens < c.max_seqs || !(c.scale > 0.0f) || !(c.eps >= 0.0f) ||
      (c.backend != B200KV_ARENA_DEVICE && c.backend != B200KV_ARENA_HOST_SIM)) {
    SetLastError("engine_create refused: layers %d, sequences %d, blocks %d x %d rows (a multiple of 64), blocks per "
                 "sequence %d, tokens per step %d (at least one per sequence), scale %g, eps %g, backend %d",
                 c.layers, c.max_seqs, c.num_blocks, c.block_size, c.max_blocks_per_seq, c.max_step_tokens,
                 static_cast<double>(c.scale), static_cast<double>(c.eps), c.backend);
    return nullptr;
  }
  auto* e = new (std::nothrow) b200kv_engine();
  if (e == nullptr) return nullptr;
  e->cfg = c;
  auto fail = [&]() {
    b200kv_engine_destroy(e);
    return static_cast<b200kv_engine*>(nullptr);
  };
  e->arena = b200kv_arena_create(c.backend);
  if (e->arena == nullptr) return fail();
  // RESERVE: the KV spans (table, slots, lengths, the two layer-major caches), then the status word.
  if (b200kv_kv_cache_reserve_batched(e->arena, c.num_blocks, c.block_size, c.layers, c.max_seqs, c.max_blocks_per_seq,
                                      c.max_step_tokens, &e->cache) != B200KV_OK) {
    return fail();
  }
  e->status_handle = b200kv_arena_reserve(e->arena, "kv.status", 16, 0);
  if (e->status_handle < 0) return fail();
  // The attention workspace is the only operator workspace of this path (the producer and the quantiser need
  // none): its high-water mark, one commit, the workspace, the latch.
  const size_t workspace = c.backend == B200KV_ARENA_DEVICE ? b200kv_mla_decode_workspace_bytes(c.max_seqs, B200KV_HEADS, 0)
                                                            : 4096;
  if (b200kv_arena_note_workspace(e->arena, workspace) != B200KV_OK || b200kv_arena_commit(e->arena) != B200KV_OK ||
      b200kv_arena_commit_workspace(e->arena) != B200KV_OK) {
    return fail();
  }
  e->d_table = static_cast<int32_t*>(b200kv_arena_address(e->arena, e->cache.block_table_handle));
  e->d_slots = static_cast<int32_t*>(b200kv_arena_address(e->arena, e->cache.slot_mapping_handle));
  e->d_lens = static_cast<int32_t*>(b200kv_arena_address(e->arena, e->cache.seq_lens_handle));
  e->d_status = static_cast<int32_t*>(b200kv_arena_address(e->arena, e->status_handle));
  e->table_off = 0;
  e->slots_off = static_cast<size_t>(b200kv_arena_offset(e->arena, e->cache.slot_mapping_handle) -
                                     b200kv_arena_offset(e->arena, e->cache.block_table_handle));
  e->lens_off = static_cast<size_t>(b200kv_arena_offset(e->arena, e->cache.seq_lens_handle) -
                                    b200kv_arena_offset(e->arena, e->cache.block_table_handle));
  e->staging_bytes = e->lens_off + static_cast<size_t>(c.max_seqs) * 4;
  if (c.backend == B200KV_ARENA_DEVICE) {
    void* pinned = nullptr;
    if (CheckCuda(cudaMallocHost(&pinned, e->staging_bytes), "engine staging (pinned)") != B200KV_OK) return fail();
    e->staging = static_cast<unsigned char*>(pinned);
  } else {
    e->staging = new (std::nothrow) unsigned char[e->staging_bytes];
    if (e->staging == nullptr) return fail();
  }
  std::memset(e->staging, 0, e->staging_bytes);
  e->pool = b200kv_block_pool_create(c.num_blocks, c.block_size, c.max_seqs, c.max_blocks_per_seq, nullptr);
  if (e->pool == nullptr) return fail();
  e->step_seq_ids.resize(static_cast<size_t>(c.max_seqs));
  e->step_grown.resize(static_cast<size_t>(c.max_seqs));
  if (b200kv_arena_seal(e->arena) != B200KV_OK) return fail();
  return e;
}

extern "C" void b200kv_engine_destroy(b200kv_engine* e) {
  if (e == nullptr) return;
  if (e->pool != nullptr) b200kv_block_pool_destroy(e->pool);
  if (e->staging != nullptr) {
    if (e->cfg.backend == B200KV_ARENA_DEVICE) cudaFreeHost(e->staging); else delete[] e->staging;
  }
  if (e->arena != nullptr) b200kv_arena_destroy(e->arena);
  delete e;
}

extern "C" const b200kv_arena* b200kv_engine_arena(const b200kv_engine* e) { return e ? e->arena : nullptr; }
extern "C" const b200kv_kv_cache* b200kv_engine_cache(const b200kv_engine* e) { return e ? &e->cache : nullptr; }
extern "C" const b200kv_block_pool* b200kv_engine_block_pool(const b200kv_engine* e) { return e ? e->pool : nullptr; }
extern "C" b200kv_status_word* b200kv_engine_status(const b200kv_engine* e) { return e ? e->d_status : nullptr; }

extern "C" int32_t b200kv_engine_admit(b200kv_engine* e, int32_t seq) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (e->in_step) return Refuse("engine_admit: a step is in flight");
  return b200kv_block_pool_admit(e->pool, seq);
}

extern "C" int32_t b200kv_engine_release(b200kv_engine* e, int32_t seq) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (e->in_step) return Refuse("engine_release: a step is in flight");
  const int32_t len = b200kv_block_pool_seq_len(e->pool, seq);
  const int32_t rc = b200kv_block_pool_release(e->pool, seq);
  if (rc == B200KV_OK && len > 0) e->active_tokens -= len;
  return rc;
}

extern "C" int32_t b200kv_engine_begin_step(b200kv_engine* e, const int32_t* seqs, const int32_t* new_tokens,
                                            int32_t n_seqs, void* stream) {
  if (e == nullptr || seqs == nullptr) {
    SetLastError("engine_begin_step: engine and seqs must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (e->in_step) return Refuse("engine_begin_step: the previous step has not ended");
  if (n_seqs <= 0 || n_seqs > e->cfg.max_seqs) {
    SetLastError("engine_begin_step: %d sequences outside [1, %d]", n_seqs, e->cfg.max_seqs);
    return B200KV_ERR_INVALID;
  }
  // PLAN: the whole step must fit (tokens per step, blocks per sequence, free blocks) before anything changes.
  int64_t total_new = 0, blocks_needed = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int32_t n = new_tokens != nullptr ? new_tokens[i] : 1;
    const int32_t len = b200kv_block_pool_seq_len(e->pool, seqs[i]);
    if (n < 1 || len < 0) {
      SetLastError("engine_begin_step: sequence %d (entry %d) is not admitted, or grows by %d tokens", seqs[i], i, n);
      return B200KV_ERR_INVALID;
    }
    for (int32_t j = 0; j < i; ++j) {
      if (seqs[j] == seqs[i]) {
        SetLastError("engine_begin_step: sequence %d appears twice in the step", seqs[i]);
        return B200KV_ERR_INVALID;
      }
    }
    const int64_t bs = e->cfg.block_size;
    const int64_t have = (len + bs - 1) / bs, want = (static_cast<int64_t>(len) + n + bs - 1) / bs;
    if (want > e->cfg.max_blocks_per_seq) {
      SetLastError("engine_begin_step: sequence %d would need %lld blocks, its table row holds %d", seqs[i],
                   static_cast<long long>(want), e->cfg.max_blocks_per_seq);
      return B200KV_ERR_INVALID;
    }
    blocks_needed += want - have;
    total_new += n;
  }
  if (total_new > e->cfg.max_step_tokens || blocks_needed > b200kv_block_pool_free_count(e->pool)) {
    SetLastError("engine_begin_step: the step appends %lld tokens (at most %d) and needs %lld free blocks (%d free)",
                 static_cast<long long>(total_new), e->cfg.max_step_tokens, static_cast<long long>(blocks_needed),
                 b200kv_block_pool_free_count(e->pool));
    return B200KV_ERR_INVALID;
  }
  // COMMIT: grow, and mirror the step into the pinned block: table rows in step order, lengths, slots.
  int32_t* s_table = reinterpret_cast<int32_t*>(e->staging + e->table_off);
  int32_t* s_slots = reinterpret_cast<int32_t*>(e->staging + e->slots_off);
  int32_t* s_lens = reinterpret_cast<int32_t*>(e->staging + e->lens_off);
  const int32_t* table = b200kv_block_pool_table(e->pool);
  int32_t at = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int32_t n = new_tokens != nullptr ? new_tokens[i] : 1;
    if (int32_t rc = b200kv_block_pool_grow(e->pool, seqs[i], n, s_slots + at)) return rc;  // cannot fail after the plan
    at += n;
    std::memcpy(s_table + static_cast<size_t>(i) * e->cfg.max_blocks_per_seq,
                table + static_cast<size_t>(seqs[i]) * e->cfg.max_blocks_per_seq,
                static_cast<size_t>(e->cfg.max_blocks_per_seq) * 4);
    s_lens[i] = b200kv_block_pool_seq_len(e->pool, seqs[i]);
    e->step_seq_ids[static_cast<size_t>(i)] = seqs[i];
    e->step_grown[static_cast<size_t>(i)] = n;
  }
  for (int32_t i = at; i < e->cfg.max_step_tokens; ++i) s_slots[i] = -1;  // padding rows write nothing
  e->allocations_at_begin = b200kv_arena_allocations(e->arena);
  e->step_seqs = n_seqs;
  e->step_tokens = at;
  // ONE upload per step: the table rows, the slots and the lengths lie in the arena in this order. An upload
  // that fails takes the step's growth back: the call changed nothing.
  int32_t rc = b200kv::FaultCheck("b200kv_engine_step_upload");
  if (rc == B200KV_OK) {
    if (e->cfg.backend == B200KV_ARENA_DEVICE) {
      rc = CheckCuda(cudaMemcpyAsync(e->d_table, e->staging, e->staging_bytes, cudaMemcpyHostToDevice,
                                     static_cast<cudaStream_t>(stream)),
                     "engine step upload");
    } else {
      std::memcpy(e->d_table, e->staging, e->staging_bytes);
    }
  }
  if (rc != B200KV_OK) {
    for (int32_t i = n_seqs - 1; i >= 0; --i) b200kv_block_pool_ungrow(e->pool, seqs[i], e->step_grown[static_cast<size_t>(i)]);
    return rc;
  }
  e->in_step = true;
  e->active_tokens += at;
  return B200KV_OK;
}

extern "C" int32_t b200kv_engine_abort_step(b200kv_engine* e) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (!e->in_step) return Refuse("engine_abort_step: no step in flight");
  // The step's growth is taken back newest first, which restores tables, lengths and the free list exactly.
  // Rows the step's launches already wrote lie beyond every sequence's length and mean nothing.
  for (int32_t i = e->step_seqs - 1; i >= 0; --i) {
    if (int32_t rc = b200kv_block_pool_ungrow(e->pool, e->step_seq_ids[static_cast<size_t>(i)], e->step_grown[static_cast<size_t>(i)])) {
      return rc;
    }
  }
  e->active_tokens -= e->step_tokens;
  e->in_step = false;
  return b200kv_block_pool_validate(e->pool);
}

extern "C" int32_t b200kv_engine_layer_append(b200kv_engine* e, int32_t layer, const void* kv_a, int64_t kv_a_stride,
                                              const void* gamma, const void* cos, int64_t cos_stride, const void* sin,
                                              int64_t sin_stride, void* q_rope, int64_t q_token_stride,
                                              int64_t q_head_stride, void* stream) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (!e->in_step) return Refuse("engine_layer_append: no step in flight");
  b200kv_producer_args a{};
  if (int32_t rc = b200kv_kv_cache_layer_view(e->arena, &e->cache, layer, &a.pool)) return rc;
  a.kv_a = kv_a;
  a.kv_a_stride = kv_a_stride;
  a.gamma = gamma;
  a.eps = e->cfg.eps;
  a.cos = cos;
  a.cos_stride = cos_stride;
  a.sin = sin;
  a.sin_stride = sin_stride;
  a.slot_mapping = e->d_slots;
  a.n_tokens = e->step_tokens;
  a.q_rope = q_rope;
  a.q_token_stride = q_token_stride;
  a.q_head_stride = q_head_stride;
  a.heads = q_rope != nullptr ? B200KV_HEADS : 0;
  return b200kv_append_fused(&a, stream, e->d_status);
}

extern "C" int32_t b200kv_engine_layer_attend(b200kv_engine* e, int32_t layer, const void* q, int64_t q_seq_stride,
                                              int64_t q_head_stride, void* out, void* out_fp8, void* out_scales,
                                              void* stream) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (!e->in_step) return Refuse("engine_layer_attend: no step in flight");
  if (e->step_tokens != e->step_seqs) {
    return Refuse("engine_layer_attend: decode attention takes one new token per sequence (this step is a prefill chunk)");
  }
  b200kv_decode_args a{};
  if (int32_t rc = b200kv_kv_cache_layer_view(e->arena, &e->cache, layer, &a.pool)) return rc;
  a.q = q;
  a.q_seq_stride = q_seq_stride;
  a.q_head_stride = q_head_stride;
  a.block_table = e->d_table;
  a.max_blocks = e->cfg.max_blocks_per_seq;
  a.kv_len = e->d_lens;
  a.batch = e->step_seqs;
  a.heads = B200KV_HEADS;
  a.block_size = e->cfg.block_size;
  a.scale = e->cfg.scale;
  a.out = out;
  a.workspace = b200kv_arena_workspace(e->arena);
  a.workspace_bytes = static_cast<size_t>(b200kv_arena_workspace_bytes(e->arena));
  a.variant = B200KV_DECODE_AUTO;
  // The step's table and lengths were uploaded before the first layer; from the second layer on the kernel
  // before this one on the stream is the producer, which does not write them.
  a.flags = B200KV_DECODE_STABLE_TABLES;
  // Stage 10, the attention output [sequences, 64 x 512] as FP8 E4M3 with one E8M0 scale per 32 values, rides in
  // the attention call: the kernel that writes `out` quantises what it writes.
  a.out_fp8 = out_fp8;
  a.out_scale = out_fp8 != nullptr ? out_scales : nullptr;
  if (out_fp8 != nullptr && out_scales == nullptr) return Refuse("engine_layer_attend: out_fp8 without out_scales");
  if (int32_t rc = b200kv_arena_workspace_fits(e->arena, b200kv_mla_decode_workspace_bytes(a.batch, a.heads, 0))) return rc;
  return b200kv_mla_decode(&a, stream, e->d_status);
}

extern "C" int32_t b200kv_engine_end_step(b200kv_engine* e) {
  if (e == nullptr) return B200KV_ERR_NULLPTR;
  if (!e->in_step) return Refuse("engine_end_step: no step in flight");
  e->in_step = false;
  ++e->steps;
  if (b200kv_arena_allocations(e->arena) != e->allocations_at_begin) {
    SetLastError("the step allocated device memory: %d allocations at its start, %d at its end",
                 e->allocations_at_begin, b200kv_arena_allocations(e->arena));
    return B200KV_ERR_INVALID;
  }
  return b200kv_block_pool_validate(e->pool);
}

extern "C" int64_t b200kv_engine_stats_json(const b200kv_engine* e, char* buffer, int64_t capacity) {
  if (e == nullptr) return -1;
  return b200kv_paged_attention_stats_json(e->cfg.num_blocks, e->cfg.layers, e->active_tokens, e->cfg.block_size, buffer,
                                           capacity);
}
