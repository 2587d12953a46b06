// Three-phase static arena for the KV reservation, and the KV cache carved out of it.
//
// Mirrors the contract of the reference's StaticMemoryArena (src/memory/static_arena.cpp:88-124,
// 275-304): RESERVE names and sizes spans with a bump cursor, COMMIT makes exactly one device
// allocation, zero-fills it and resolves every span to base + offset, SEAL latches so that nothing
// can allocate inside the decode loop. Every refusal of the reference is a refusal here, reported as
// a status code plus text instead of an exception (no exceptions cross the C ABI).
//
// The KV cache on top follows src/memory/static_arena_manager.cpp:298-300, 315-318 (span names, layer
// major layout, two co-indexed caches) and src/pipeline/pipeline.cpp:391-395 (per-layer base).
#include <cuda_runtime.h>

#include <climits>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "b200kv.h"

namespace b200kv {
void SetLastError(const char* fmt, ...);
int32_t CheckCuda(cudaError_t err, const char* what);
}  // namespace b200kv

using b200kv::CheckCuda;
using b200kv::SetLastError;

namespace {

constexpr size_t kArenaAlign = 512;       // default span alignment (include/moe/core/config.hpp:237)
constexpr size_t kHostSimAlign = 4096;    // the simulated backend serves page-aligned blocks

size_t AlignUp(size_t value, size_t align) { return (value + align - 1) & ~(align - 1); }

struct Span {
  std::string name;
  size_t offset;
  size_t bytes;
  size_t align;
};

}  // namespace

struct b200kv_arena {
  int32_t backend = B200KV_ARENA_DEVICE;
  std::vector<Span> spans;
  size_t cursor = 0;
  void* base = nullptr;
  size_t bytes = 0;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
  uint64_t workspace_high_water = 0;
  bool workspace_committed = false;
  bool sealed = false;
  int32_t allocations = 0;
};

namespace {

void* BackendAlloc(b200kv_arena* arena, size_t bytes) {
  void* p = nullptr;
  if (arena->backend == B200KV_ARENA_HOST_SIM) {
    p = std::aligned_alloc(kHostSimAlign, AlignUp(bytes, kHostSimAlign));
    if (p == nullptr) SetLastError("arena: host allocation of %zu bytes failed", bytes);
    else std::memset(p, 0, bytes);
  } else {
    if (CheckCuda(cudaMalloc(&p, bytes), "arena cudaMalloc") != B200KV_OK) return nullptr;
    if (CheckCuda(cudaMemset(p, 0, bytes), "arena cudaMemset") != B200KV_OK) {
      cudaFree(p);
      return nullptr;
    }
  }
  if (p != nullptr) ++arena->allocations;
  return p;
}

void BackendFree(b200kv_arena* arena, void* p) {
  if (p == nullptr) return;
  if (arena->backend == B200KV_ARENA_HOST_SIM) std::free(p); else cudaFree(p);
}

int32_t Refuse(const char* text) {
  SetLastError("%s", text);
  return B200KV_ERR_INVALID;
}

}  // namespace

extern "C" b200kv_arena* b200kv_arena_create(int32_t backend) {
  if (backend != B200KV_ARENA_DEVICE && backend != B200KV_ARENA_HOST_SIM) {
    SetLastError("arena: unknown backend %d", backend);
    return nullptr;
  }
  auto* arena = new b200kv_arena();
  arena->backend = backend;
  return arena;
}

extern "C" void b200kv_arena_destroy(b200kv_arena* arena) {
  if (arena == nullptr) return;
  BackendFree(arena, arena->workspace);
  BackendFree(arena, arena->base);
  delete arena;
}

extern "C" int64_t b200kv_arena_reserve(b200kv_arena* arena, const char* name, size_t bytes, size_t align) {
  if (arena == nullptr || name == nullptr) {
    SetLastError("arena reserve: null arena or name");
    return -B200KV_ERR_NULLPTR;
  }
  if (align == 0) align = kArenaAlign;
  if (arena->sealed) return -Refuse("reserve refused: the arena has been sealed for the decode loop");
  if (arena->base != nullptr) return -Refuse("reserve refused: the arena was committed and its size can no longer change");
  if (bytes == 0) return -Refuse("a reservation must not be empty");
  if ((align & (align - 1)) != 0) return -Refuse("a reservation's alignment must be a power of two");
  Span span{name, AlignUp(arena->cursor, align), bytes, align};
  arena->cursor = span.offset + bytes;
  arena->spans.push_back(span);
  return static_cast<int64_t>(arena->spans.size() - 1);
}

extern "C" int32_t b200kv_arena_commit(b200kv_arena* arena) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  if (arena->sealed) return Refuse("the arena is sealed; Commit refused");
  if (arena->base != nullptr) return Refuse("commit refused: the arena has been committed before");
  if (arena->spans.empty()) return Refuse("commit refused: the arena holds no reservation");
  arena->bytes = AlignUp(arena->cursor, kArenaAlign);
  arena->base = BackendAlloc(arena, arena->bytes);  // ONE allocation, zero-filled
  if (arena->base == nullptr) return B200KV_ERR_RUNTIME;
  return b200kv_arena_validate(arena);
}

extern "C" void* b200kv_arena_address(const b200kv_arena* arena, int64_t handle) {
  if (arena == nullptr || arena->base == nullptr) {
    SetLastError("Address needs the arena to be committed first");
    return nullptr;
  }
  if (handle < 0 || handle >= static_cast<int64_t>(arena->spans.size())) {
    SetLastError("arena handle %lld out of range", static_cast<long long>(handle));
    return nullptr;
  }
  return static_cast<uint8_t*>(arena->base) + arena->spans[static_cast<size_t>(handle)].offset;
}

extern "C" int64_t b200kv_arena_offset(const b200kv_arena* arena, int64_t handle) {
  if (arena == nullptr || handle < 0 || handle >= static_cast<int64_t>(arena->spans.size())) return -1;
  return static_cast<int64_t>(arena->spans[static_cast<size_t>(handle)].offset);
}

extern "C" size_t b200kv_arena_reserved_bytes(const b200kv_arena* arena) { return arena ? arena->cursor : 0; }
extern "C" size_t b200kv_arena_bytes(const b200kv_arena* arena) { return arena ? arena->bytes : 0; }
extern "C" int32_t b200kv_arena_allocations(const b200kv_arena* arena) { return arena ? arena->allocations : -1; }

extern "C" int32_t b200kv_arena_note_workspace(b200kv_arena* arena, uint64_t bytes) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  if (arena->sealed) return Refuse("the arena is sealed; NoteWorkspace refused");
  if (bytes > arena->workspace_high_water) arena->workspace_high_water = bytes;
  return B200KV_OK;
}

extern "C" int32_t b200kv_arena_commit_workspace(b200kv_arena* arena) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  if (arena->sealed) return Refuse("the arena is sealed; CommitWorkspace refused");
  if (arena->workspace_committed) return Refuse("the workspace is already committed");
  arena->workspace_committed = true;
  arena->workspace_bytes = arena->workspace_high_water;
  if (arena->workspace_bytes == 0) return B200KV_OK;  // every planned operator asked for none
  arena->workspace = BackendAlloc(arena, static_cast<size_t>(arena->workspace_bytes));
  return arena->workspace != nullptr ? B200KV_OK : B200KV_ERR_RUNTIME;
}

extern "C" void* b200kv_arena_workspace(const b200kv_arena* arena) { return arena ? arena->workspace : nullptr; }
extern "C" uint64_t b200kv_arena_workspace_bytes(const b200kv_arena* arena) {
  return arena ? arena->workspace_bytes : 0;
}

extern "C" int32_t b200kv_arena_workspace_fits(const b200kv_arena* arena, uint64_t bytes) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  if (bytes > arena->workspace_bytes) {
    SetLastError("a plan needs %llu workspace bytes but only %llu were reserved at init; rebuild, never grow the "
                 "workspace inside a step",
                 static_cast<unsigned long long>(bytes), static_cast<unsigned long long>(arena->workspace_bytes));
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

extern "C" int32_t b200kv_arena_seal(b200kv_arena* arena) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  if (arena->base == nullptr) return Refuse("Seal needs the arena to be committed first");
  arena->sealed = true;
  return B200KV_OK;
}

extern "C" int32_t b200kv_arena_sealed(const b200kv_arena* arena) { return arena && arena->sealed ? 1 : 0; }

extern "C" int32_t b200kv_arena_validate(const b200kv_arena* arena) {
  if (arena == nullptr) return B200KV_ERR_NULLPTR;
  size_t previous_end = 0;
  const char* previous = "<start>";
  for (const Span& span : arena->spans) {
    if (span.offset % span.align != 0) {
      SetLastError("reservation %s sits at %zu, not aligned to %zu", span.name.c_str(), span.offset, span.align);
      return B200KV_ERR_INVALID;
    }
    if (span.offset < previous_end) {
      SetLastError("reservation %s at %zu overlaps %s which ends at %zu", span.name.c_str(), span.offset, previous,
                   previous_end);
      return B200KV_ERR_INVALID;
    }
    if (arena->base != nullptr && span.offset + span.bytes > arena->bytes) {
      SetLastError("reservation %s ends at %zu beyond the %zu-byte arena", span.name.c_str(),
                   span.offset + span.bytes, arena->bytes);
      return B200KV_ERR_INVALID;
    }
    previous_end = span.offset + span.bytes;
    previous = span.name.c_str();
  }
  if (arena->base != nullptr && reinterpret_cast<uintptr_t>(arena->base) % kArenaAlign != 0) {
    SetLastError("the committed arena base is not %zu-byte aligned", kArenaAlign);
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

// ---- the KV cache carved from the arena -----------------------------------------------------------

extern "C" int32_t b200kv_kv_cache_reserve(b200kv_arena* arena, int64_t max_context, int64_t block_size,
                                           int64_t layers, int64_t max_seqs, int64_t tokens_per_step,
                                           b200kv_kv_cache* out) {
  if (arena == nullptr || out == nullptr) {
    SetLastError("kv_cache_reserve: null arena or out");
    return B200KV_ERR_NULLPTR;
  }
  if (block_size <= 0 || max_context < block_size) {
    SetLastError("kv_cache_reserve: max context %lld is below one block of %lld", static_cast<long long>(max_context),
                 static_cast<long long>(block_size));
    return B200KV_ERR_INVALID;
  }
  b200kv_reservation plan;
  if (int32_t rc = b200kv_plan_reservation(max_context, block_size, layers, max_seqs, tokens_per_step, &plan)) return rc;
  std::memset(out, 0, sizeof(*out));
  out->geometry = plan;
  out->layers = layers;
  out->block_size = block_size;
  out->max_seqs = max_seqs;
  // Activation-side spans first, cache spans after, in the reference's order and under its names.
  out->block_table_handle = b200kv_arena_reserve(arena, "kv.block_table", static_cast<size_t>(plan.block_table_bytes), 0);
  out->slot_mapping_handle = b200kv_arena_reserve(arena, "kv.slot_mapping", static_cast<size_t>(plan.slot_mapping_bytes), 0);
  out->latent_handle = b200kv_arena_reserve(arena, "kv.latent_cache", static_cast<size_t>(plan.latent_bytes), 0);
  out->rope_handle = b200kv_arena_reserve(arena, "kv.rope_cache", static_cast<size_t>(plan.rope_bytes), 0);
  if (out->block_table_handle < 0 || out->slot_mapping_handle < 0 || out->latent_handle < 0 || out->rope_handle < 0) {
    return B200KV_ERR_INVALID;
  }
  out->max_blocks_per_seq = plan.blocks_per_layer;
  out->seq_lens_handle = -1;
  return B200KV_OK;
}

extern "C" int32_t b200kv_kv_cache_reserve_batched(b200kv_arena* arena, int64_t num_blocks, int64_t block_size,
                                                   int64_t layers, int64_t max_seqs, int64_t max_blocks_per_seq,
                                                   int64_t tokens_per_step, b200kv_kv_cache* out) {
  if (arena == nullptr || out == nullptr) {
    SetLastError("kv_cache_reserve_batched: null arena or out");
    return B200KV_ERR_NULLPTR;
  }
  if (num_blocks <= 0 || block_size <= 0 || layers <= 0 || max_seqs <= 0 || max_blocks_per_seq <= 0 ||
      tokens_per_step <= 0 || num_blocks * block_size > INT32_MAX) {
    SetLastError("kv_cache_reserve_batched refused: blocks %lld x %lld rows, layers %lld, sequences %lld, blocks per "
                 "sequence %lld, tokens per step %lld",
                 static_cast<long long>(num_blocks), static_cast<long long>(block_size), static_cast<long long>(layers),
                 static_cast<long long>(max_seqs), static_cast<long long>(max_blocks_per_seq),
                 static_cast<long long>(tokens_per_step));
    return B200KV_ERR_INVALID;
  }
  std::memset(out, 0, sizeof(*out));
  b200kv_reservation& plan = out->geometry;
  plan.blocks_per_layer = num_blocks;
  plan.total_blocks = num_blocks * layers;
  plan.latent_bytes = layers * num_blocks * block_size * B200KV_LATENT_DIM * 2;
  plan.rope_bytes = layers * num_blocks * block_size * B200KV_ROPE_DIM * 2;
  plan.block_table_bytes = max_seqs * max_blocks_per_seq * 4;
  plan.slot_mapping_bytes = tokens_per_step * 4;
  out->layers = layers;
  out->block_size = block_size;
  out->max_seqs = max_seqs;
  out->max_blocks_per_seq = max_blocks_per_seq;
  // The reference's four spans under its names and in its order, and the lengths beside the table.
  out->block_table_handle = b200kv_arena_reserve(arena, "kv.block_table", static_cast<size_t>(plan.block_table_bytes), 0);
  out->slot_mapping_handle = b200kv_arena_reserve(arena, "kv.slot_mapping", static_cast<size_t>(plan.slot_mapping_bytes), 0);
  out->seq_lens_handle = b200kv_arena_reserve(arena, "kv.seq_lens", static_cast<size_t>(max_seqs) * 4, 0);
  out->latent_handle = b200kv_arena_reserve(arena, "kv.latent_cache", static_cast<size_t>(plan.latent_bytes), 0);
  out->rope_handle = b200kv_arena_reserve(arena, "kv.rope_cache", static_cast<size_t>(plan.rope_bytes), 0);
  if (out->block_table_handle < 0 || out->slot_mapping_handle < 0 || out->seq_lens_handle < 0 || out->latent_handle < 0 ||
      out->rope_handle < 0) {
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

extern "C" int32_t b200kv_kv_cache_layer_view(const b200kv_arena* arena, const b200kv_kv_cache* cache, int64_t layer,
                                              b200kv_pool_view* out) {
  if (arena == nullptr || cache == nullptr || out == nullptr) {
    SetLastError("kv_cache_layer_view: null argument");
    return B200KV_ERR_NULLPTR;
  }
  if (layer < 0 || layer >= cache->layers) {
    SetLastError("kv_cache_layer_view: layer %lld outside [0, %lld)", static_cast<long long>(layer),
                 static_cast<long long>(cache->layers));
    return B200KV_ERR_INVALID;
  }
  auto* latent = static_cast<uint8_t*>(b200kv_arena_address(arena, cache->latent_handle));
  auto* rope = static_cast<uint8_t*>(b200kv_arena_address(arena, cache->rope_handle));
  if (latent == nullptr || rope == nullptr) return B200KV_ERR_INVALID;
  const int64_t rows = cache->geometry.blocks_per_layer * cache->block_size;
  // Per-layer base = span + layer * blocks * block_size * width * 2 bytes.
  out->latent = latent + layer * rows * B200KV_LATENT_DIM * 2;
  out->rope = rope + layer * rows * B200KV_ROPE_DIM * 2;
  out->latent_row_stride = B200KV_LATENT_DIM;
  out->rope_row_stride = B200KV_ROPE_DIM;
  out->pool_rows = rows;
  return B200KV_OK;
}
