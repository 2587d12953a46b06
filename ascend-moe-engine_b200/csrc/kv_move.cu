// Scatter-append and block-table gather of MLA latent rows (bf16) on sm_100a.
//
// Both are pure byte movement bounded by HBM bandwidth: a row is latent_dim*2 + rope_dim*2 bytes
// (1,152 B at 512+64), moved as 16-byte chunks. A warp owns four rows at a time (288 chunks at the
// model geometry, nine per lane), issues all its loads before its first store so that nine 16-byte
// requests per lane are in flight, and touches each byte exactly once: algorithmic traffic is
// row_bytes read + row_bytes written (+ 4 B of index per row).
#include "common.cuh"

namespace b200kv {
namespace {

constexpr int kRowsPerWarp = 4;
constexpr int kWarpsPerCta = 8;

struct RowPair {
  const char* src_latent;
  const char* src_rope;
  char* dst_latent;
  char* dst_rope;
};

// Copies up to four rows; `valid` (lanes 0..3) says which of the warp's rows exist. Pointers of row r
// are broadcast from lane r. kChunks > 0 fixes chunks-per-row at compile time.
template <int kLatentChunks, int kRopeChunks>
__device__ __forceinline__ void CopyFourRows(const RowPair& mine, bool valid, int latent_chunks, int rope_chunks) {
  const int lane = threadIdx.x & 31;
  const int lc = kLatentChunks > 0 ? kLatentChunks : latent_chunks;
  const int rc = kRopeChunks > 0 ? kRopeChunks : rope_chunks;
  const int per_row = lc + rc;
  const int total = per_row * kRowsPerWarp;

  unsigned long long sl[kRowsPerWarp], sr[kRowsPerWarp], dl[kRowsPerWarp], dr[kRowsPerWarp];
  unsigned ok_mask = __ballot_sync(0xffffffffu, valid && lane < kRowsPerWarp);
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    sl[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine.src_latent), r);
    sr[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine.src_rope), r);
    dl[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine.dst_latent), r);
    dr[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine.dst_rope), r);
  }

  constexpr int kMaxItems = (kLatentChunks > 0) ? ((kLatentChunks + kRopeChunks) * kRowsPerWarp + 31) / 32 : 12;
  int4 regs[kMaxItems];
  for (int base = 0; base < total; base += 32 * kMaxItems) {
#pragma unroll
    for (int i = 0; i < kMaxItems; ++i) {
      const int idx = base + lane + 32 * i;
      if (idx < total) {
        const int r = idx / per_row;
        const int c = idx - r * per_row;
        if ((ok_mask >> r) & 1u) {
          // Selecting by comparison keeps the pointer arrays in registers.
          unsigned long long sl_r = sl[0], sr_r = sr[0];
#pragma unroll
          for (int q = 1; q < kRowsPerWarp; ++q) {
            if (r == q) {
              sl_r = sl[q];
              sr_r = sr[q];
            }
          }
          const char* src = c < lc ? reinterpret_cast<const char*>(sl_r) + 16 * c
                                   : reinterpret_cast<const char*>(sr_r) + 16 * (c - lc);
          regs[i] = LoadStream16(src);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kMaxItems; ++i) {
      const int idx = base + lane + 32 * i;
      if (idx < total) {
        const int r = idx / per_row;
        const int c = idx - r * per_row;
        if ((ok_mask >> r) & 1u) {
          unsigned long long dl_r = dl[0], dr_r = dr[0];
#pragma unroll
          for (int q = 1; q < kRowsPerWarp; ++q) {
            if (r == q) {
              dl_r = dl[q];
              dr_r = dr[q];
            }
          }
          char* dst = c < lc ? reinterpret_cast<char*>(dl_r) + 16 * c : reinterpret_cast<char*>(dr_r) + 16 * (c - lc);
          StoreStream16(dst, regs[i]);
        }
      }
    }
  }
}

template <int kLatentChunks, int kRopeChunks>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    AppendKernel(b200kv_pool_view pool, const char* latent_src, int64_t src_latent_stride_b, const char* rope_src,
                 int64_t src_rope_stride_b, const int32_t* __restrict__ slot_mapping, int64_t n_tokens,
                 int latent_chunks, int rope_chunks, int32_t* status) {
  GridDependencyTrigger();
  GridDependencyWait();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t groups = (n_tokens + kRowsPerWarp - 1) / kRowsPerWarp;
  const int lc = kLatentChunks > 0 ? kLatentChunks : latent_chunks;
  const int rc = kRopeChunks > 0 ? kRopeChunks : rope_chunks;
  const int per_row = lc + rc;
  const int total = per_row * kRowsPerWarp;
  constexpr int kMaxItems = (kLatentChunks > 0) ? ((kLatentChunks + kRopeChunks) * kRowsPerWarp + 31) / 32 : 12;
  for (int64_t g = warp; g < groups; g += n_warps) {
    const int64_t t0 = g * kRowsPerWarp;
    // Where a row comes from depends on its token index only, where it goes on its slot: the slot loads
    // (lanes 0..3) and all the row loads leave together, one round trip to memory instead of two.
    int64_t slot = -1;
    if (lane < kRowsPerWarp && t0 + lane < n_tokens) slot = slot_mapping[t0 + lane];
    int4 regs[kMaxItems];
    for (int base = 0; base < total; base += 32 * kMaxItems) {
#pragma unroll
      for (int i = 0; i < kMaxItems; ++i) {
        const int idx = base + lane + 32 * i;
        const int r = idx / per_row;
        const int c = idx - r * per_row;
        if (idx < total && t0 + r < n_tokens) {
          const char* src = c < lc ? latent_src + (t0 + r) * src_latent_stride_b + 16 * c
                                   : rope_src + (t0 + r) * src_rope_stride_b + 16 * (c - lc);
          regs[i] = LoadStream16(src);
        }
      }
      // Destinations: a negative slot is padding, one past the pool is recorded and skipped.
      bool valid = false;
      char* my_latent = nullptr;
      char* my_rope = nullptr;
      if (lane < kRowsPerWarp && t0 + lane < n_tokens) {
        if (slot >= pool.pool_rows) {
          if (base == 0) RecordError(status, B200KV_DEV_BAD_SLOT, static_cast<int32_t>(t0 + lane), static_cast<int32_t>(slot));
        } else if (slot >= 0) {
          valid = true;
          my_latent = static_cast<char*>(pool.latent) + slot * pool.latent_row_stride * 2;
          my_rope = static_cast<char*>(pool.rope) + slot * pool.rope_row_stride * 2;
        }
      }
      const unsigned ok_mask = __ballot_sync(0xffffffffu, valid);
      unsigned long long dl[kRowsPerWarp], dr[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        dl[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_latent), r);
        dr[r] = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_rope), r);
      }
#pragma unroll
      for (int i = 0; i < kMaxItems; ++i) {
        const int idx = base + lane + 32 * i;
        const int r = idx / per_row;
        const int c = idx - r * per_row;
        if (idx < total && ((ok_mask >> r) & 1u)) {
          // Selecting by comparison keeps the pointer arrays in registers.
          unsigned long long dl_r = dl[0], dr_r = dr[0];
#pragma unroll
          for (int q = 1; q < kRowsPerWarp; ++q) {
            if (r == q) {
              dl_r = dl[q];
              dr_r = dr[q];
            }
          }
          char* dst = c < lc ? reinterpret_cast<char*>(dl_r) + 16 * c : reinterpret_cast<char*>(dr_r) + 16 * (c - lc);
          StoreStream16(dst, regs[i]);
        }
      }
    }
  }
}

// 64 registers (four CTAs per SM) cost the gather nothing and double its resident warps; the append
// spills at that bound and is faster left alone.
template <int kLatentChunks, int kRopeChunks>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 4)
    GatherKernel(b200kv_pool_view pool, const int32_t* __restrict__ block_table, int64_t max_blocks,
                 const int32_t* __restrict__ kv_len, int32_t batch, int32_t block_size, char* out_latent,
                 int64_t out_latent_stride_b, char* out_rope, int64_t out_rope_stride_b,
                 const int64_t* __restrict__ out_row_offsets, int64_t total_rows, int latent_chunks, int rope_chunks,
                 int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t groups = (total_rows + kRowsPerWarp - 1) / kRowsPerWarp;
  for (int64_t g = warp; g < groups; g += n_warps) {
    RowPair mine{};
    bool valid = false;
    if (lane < kRowsPerWarp) {
      const int64_t row = g * kRowsPerWarp + lane;
      if (row < total_rows) {
        // Last sequence whose first output row is <= row.
        int lo = 0, hi = batch - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (out_row_offsets[mid] <= row) lo = mid; else hi = mid - 1;
        }
        const int64_t j = row - out_row_offsets[lo];
        if (j >= 0 && j < kv_len[lo]) {
          // The lengths live on the device, so only the kernel can see a length that runs past the table's row.
          const int64_t column = j / block_size;
          const int64_t block = column < max_blocks ? block_table[static_cast<int64_t>(lo) * max_blocks + column] : -1;
          const int64_t src_row = block * block_size + j % block_size;
          if (block < 0 || src_row >= pool.pool_rows) {
            RecordError(status, B200KV_DEV_BAD_BLOCK, lo, static_cast<int32_t>(j / block_size),
                        static_cast<int32_t>(block));
          } else {
            valid = true;
            mine.src_latent = static_cast<const char*>(pool.latent) + src_row * pool.latent_row_stride * 2;
            mine.src_rope = static_cast<const char*>(pool.rope) + src_row * pool.rope_row_stride * 2;
            mine.dst_latent = out_latent + row * out_latent_stride_b;
            mine.dst_rope = out_rope + row * out_rope_stride_b;
          }
        }
      }
    }
    CopyFourRows<kLatentChunks, kRopeChunks>(mine, valid, latent_chunks, rope_chunks);
  }
}

// Physical pool row of every selected token: rows[b][j] = table[b][t / bs] * bs + t % bs for t = index[b][j],
// j < n_selected[b]; the rest of a row of `rows` is filled with -1.
__global__ void __launch_bounds__(256)
    ResolveRowsKernel(const int32_t* __restrict__ block_table, int64_t max_blocks, int32_t block_size,
                      const int32_t* __restrict__ token_index, int64_t max_selected, const int32_t* __restrict__ n_selected,
                      int32_t batch, int64_t pool_rows, int32_t* __restrict__ rows, int32_t* status) {
  GridDependencyTrigger();
  GridDependencyWait();
  const int64_t total = static_cast<int64_t>(batch) * max_selected;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / max_selected, j = i % max_selected;
    int32_t row = -1;
    if (j < n_selected[b]) {
      const int64_t t = token_index[i];
      const int64_t column = t / block_size;
      const int64_t block = (t >= 0 && column < max_blocks) ? block_table[b * max_blocks + column] : -1;
      const int64_t r = block * block_size + t % block_size;
      if (t < 0 || block < 0 || r >= pool_rows) {
        RecordError(status, B200KV_DEV_BAD_BLOCK, static_cast<int32_t>(b), static_cast<int32_t>(j), static_cast<int32_t>(t));
      } else {
        row = static_cast<int32_t>(r);
      }
    }
    rows[i] = row;
  }
}

int GridFor(int64_t rows) {
  const int64_t groups = (rows + kRowsPerWarp - 1) / kRowsPerWarp;
  const int64_t ctas = (groups + kWarpsPerCta - 1) / kWarpsPerCta;
  // Eight resident CTAs of 256 threads per SM; the grid-stride loop covers the rest.
  const int64_t cap = static_cast<int64_t>(CurrentDeviceSmCount()) * 8;
  return static_cast<int>(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int32_t CheckPool(const b200kv_pool_view* pool) {
  if (pool == nullptr || pool->latent == nullptr || pool->rope == nullptr) {
    SetLastError("pool view or one of its base pointers is null");
    return B200KV_ERR_NULLPTR;
  }
  if (!Aligned16(pool->latent) || !Aligned16(pool->rope) || pool->latent_row_stride % 8 != 0 ||
      pool->rope_row_stride % 8 != 0 || pool->latent_row_stride < B200KV_LATENT_DIM ||
      pool->rope_row_stride < B200KV_ROPE_DIM || pool->pool_rows <= 0) {
    SetLastError("pool view refused: bases must be 16-byte aligned, row strides multiples of 8 elements and >= "
                 "the row width, pool_rows > 0 (latent stride %lld, rope stride %lld, rows %lld)",
                 static_cast<long long>(pool->latent_row_stride), static_cast<long long>(pool->rope_row_stride),
                 static_cast<long long>(pool->pool_rows));
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

}  // namespace

int32_t ValidatePoolView(const b200kv_pool_view* pool) { return CheckPool(pool); }

}  // namespace b200kv

namespace b200kv {
bool GatherTmaSupports(const b200kv_pool_view& pool, int64_t batch, int64_t block_size, int64_t out_latent_stride,
                       int64_t out_rope_stride, int64_t total_rows);
int32_t LaunchGatherTma(const b200kv_pool_view& pool, const int32_t* block_table, int64_t max_blocks, const int32_t* kv_len,
                        int32_t batch, int32_t block_size, void* out_latent, int64_t out_latent_stride, void* out_rope,
                        int64_t out_rope_stride, const int64_t* out_row_offsets, int64_t total_rows, cudaStream_t stream,
                        int32_t* status);
}  // namespace b200kv

using namespace b200kv;

extern "C" int32_t b200kv_append(const b200kv_pool_view* pool, const void* latent_src, int64_t src_latent_stride,
                                 const void* rope_src, int64_t src_rope_stride, const int32_t* slot_mapping,
                                 int64_t n_tokens, void* stream, b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_append")) return rc;
  if (int32_t rc = CheckPool(pool)) return rc;
  if (n_tokens == 0) return B200KV_OK;
  if (latent_src == nullptr || rope_src == nullptr || slot_mapping == nullptr) {
    SetLastError("append: latent_src, rope_src and slot_mapping must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (n_tokens < 0 || !Aligned16(latent_src) || !Aligned16(rope_src) || src_latent_stride % 8 != 0 ||
      src_rope_stride % 8 != 0 || src_latent_stride < B200KV_LATENT_DIM || src_rope_stride < B200KV_ROPE_DIM) {
    SetLastError("append refused: n_tokens %lld, source strides %lld/%lld (multiples of 8, >= row width), "
                 "sources 16-byte aligned",
                 static_cast<long long>(n_tokens), static_cast<long long>(src_latent_stride),
                 static_cast<long long>(src_rope_stride));
    return B200KV_ERR_INVALID;
  }
  return CheckCuda(
      LaunchOverlapped(AppendKernel<B200KV_LATENT_DIM / 8, B200KV_ROPE_DIM / 8>, dim3(GridFor(n_tokens)),
                       dim3(kWarpsPerCta * 32), 0, static_cast<cudaStream_t>(stream), *pool,
                       static_cast<const char*>(latent_src), src_latent_stride * 2, static_cast<const char*>(rope_src),
                       src_rope_stride * 2, slot_mapping, n_tokens, B200KV_LATENT_DIM / 8, B200KV_ROPE_DIM / 8, status),
      "append launch");
}

extern "C" int32_t b200kv_gather(const b200kv_pool_view* pool, const int32_t* block_table, int64_t max_blocks,
                                 const int32_t* kv_len, int64_t batch, int64_t block_size, void* out_latent,
                                 int64_t out_latent_stride, void* out_rope, int64_t out_rope_stride,
                                 const int64_t* out_row_offsets, int64_t total_rows, void* stream,
                                 b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_gather")) return rc;
  if (int32_t rc = CheckPool(pool)) return rc;
  if (batch == 0 || total_rows == 0) return B200KV_OK;
  if (block_table == nullptr || kv_len == nullptr || out_latent == nullptr || out_rope == nullptr ||
      out_row_offsets == nullptr) {
    SetLastError("gather: block_table, kv_len, outputs and out_row_offsets must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (batch < 0 || batch > INT32_MAX || total_rows < 0 || block_size <= 0 || max_blocks <= 0 ||
      pool->pool_rows % block_size != 0 || !Aligned16(out_latent) || !Aligned16(out_rope) ||
      out_latent_stride % 8 != 0 || out_rope_stride % 8 != 0 || out_latent_stride < B200KV_LATENT_DIM ||
      out_rope_stride < B200KV_ROPE_DIM) {
    SetLastError("gather refused: batch %lld, rows %lld, block_size %lld, max_blocks %lld, out strides %lld/%lld",
                 static_cast<long long>(batch), static_cast<long long>(total_rows),
                 static_cast<long long>(block_size), static_cast<long long>(max_blocks),
                 static_cast<long long>(out_latent_stride), static_cast<long long>(out_rope_stride));
    return B200KV_ERR_INVALID;
  }
  // Blocks of a multiple of 64 tokens go through shared memory by TMA, 64 rows at a time (kv_gather_tma.cu); other
  // geometries row by row through registers.
  if (GatherTmaSupports(*pool, batch, block_size, out_latent_stride, out_rope_stride, total_rows)) {
    return LaunchGatherTma(*pool, block_table, max_blocks, kv_len, static_cast<int32_t>(batch), static_cast<int32_t>(block_size),
                           out_latent, out_latent_stride, out_rope, out_rope_stride, out_row_offsets, total_rows,
                           static_cast<cudaStream_t>(stream), status);
  }
  GatherKernel<B200KV_LATENT_DIM / 8, B200KV_ROPE_DIM / 8>
      <<<GridFor(total_rows), kWarpsPerCta * 32, 0, static_cast<cudaStream_t>(stream)>>>(
          *pool, block_table, max_blocks, kv_len, static_cast<int32_t>(batch), static_cast<int32_t>(block_size),
          static_cast<char*>(out_latent), out_latent_stride * 2, static_cast<char*>(out_rope), out_rope_stride * 2,
          out_row_offsets, total_rows, B200KV_LATENT_DIM / 8, B200KV_ROPE_DIM / 8, status);
  return CheckCuda(cudaGetLastError(), "gather launch");
}

extern "C" int32_t b200kv_resolve_rows(const int32_t* block_table, int64_t max_blocks, int64_t block_size,
                                       const int32_t* token_index, int64_t max_selected, const int32_t* n_selected,
                                       int64_t batch, int64_t pool_rows, int32_t* rows, void* stream,
                                       b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_resolve_rows")) return rc;
  if (batch == 0 || max_selected == 0) return B200KV_OK;
  if (block_table == nullptr || token_index == nullptr || n_selected == nullptr || rows == nullptr) {
    SetLastError("resolve_rows: block_table, token_index, n_selected and rows must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (batch < 0 || batch > INT32_MAX || max_selected < 0 || block_size <= 0 || block_size > INT32_MAX || max_blocks <= 0 ||
      pool_rows <= 0 || pool_rows > INT32_MAX) {
    SetLastError("resolve_rows refused: batch %lld, max_selected %lld, block_size %lld, max_blocks %lld, pool_rows %lld",
                 static_cast<long long>(batch), static_cast<long long>(max_selected), static_cast<long long>(block_size),
                 static_cast<long long>(max_blocks), static_cast<long long>(pool_rows));
    return B200KV_ERR_INVALID;
  }
  const int64_t total = batch * max_selected;
  const int64_t want = (total + 255) / 256;
  const int grid = static_cast<int>(want > 1184 ? 1184 : want);
  return CheckCuda(LaunchOverlapped(ResolveRowsKernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                    block_table, max_blocks, static_cast<int32_t>(block_size), token_index, max_selected,
                                    n_selected, static_cast<int32_t>(batch), pool_rows, rows, status),
                   "resolve_rows launch");
}
