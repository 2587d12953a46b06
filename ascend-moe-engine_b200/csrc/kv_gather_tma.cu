// Block-table gather with the blocks staged through shared memory by TMA: for every sequence, its logical rows
// 0 .. kv_len - 1 (pool row block_table[b][j / bs] * bs + j % bs) copied to the contiguous outputs out_latent
// [total_rows][512] and out_rope [total_rows][64] at out_row_offsets[b] + j. The reference has no such function
// of its own; the addressing is what its attention operator applies through block_table and block_size
// (src/pipeline/pipeline.cpp:241-244; restated in
// third_party/ops_transformer/attention/quant_lightning_indexer/op_kernel/arch35/quant_lightning_indexer_service_cube.h:243-268).
//
// A tile is 64 consecutive tokens of a sequence, which a block of the pool holds in 64 consecutive rows (block
// sizes that are multiples of 64). Three tiled TMA loads bring it into a stage of shared memory as plain rows
// (latent columns 0-255 and 256-511, the 64 rope columns; no swizzle, nothing computes on them), and three
// tiled TMA stores write the stage to the outputs, whose rows are consecutive whatever the block table says. No
// thread touches the data. A sequence's last tile holds 1 .. 64 rows; a store's box is fixed, so such a tile goes
// out in boxes of 32, 16, 8, 4, 2 and 1 rows (one tensor map of the outputs per box height), each from its offset
// in the stage. One thread per CTA drives three stages: the loads of tile i + 2 are issued before the stores
// of tile i, and a stage is reused once the bulk group of its stores has finished reading it. Persistent CTAs,
// one per SM (three stages of 72 KB), tiles dealt out round-robin over the flat list of all sequences' tiles:
// the warp first lays the sequences' running tile counts into shared memory (a scan over the lengths), and the
// driving thread finds the sequence of its k-th tile by bisection there. (A first version walked the sequences
// one by one in that thread: 0.6 us a sequence, 164 us for 256 short sequences.)
// Bit-exact by construction (bytes are copied); bound by HBM: 1,152 bytes read and written per row.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200kv {

int32_t EncodePlainBf16Map(const void* base, int64_t stride_bytes, int64_t rows, int32_t width, int32_t box_cols,
                           int32_t box_rows, CUtensorMap* out);

namespace {

constexpr int kTileRows = 64;
constexpr int kHalfLatent = 256;                                  // elements per latent box (512 bytes a row)
constexpr int kLatentBoxBytes = kTileRows * kHalfLatent * 2;      // 32 KB
constexpr int kRopeBoxBytes = kTileRows * B200KV_ROPE_DIM * 2;    // 8 KB
constexpr int kStageBytes = 2 * kLatentBoxBytes + kRopeBoxBytes;  // 72 KB
constexpr int kStages = 3;
constexpr int kHeights = 7;  // store boxes of 64, 32, 16, 8, 4, 2, 1 rows
constexpr int kMaxBatch = 2048;  // sequences whose running tile counts fit beside the stages
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 128 + (kMaxBatch + 1) * 4;

struct GatherMaps {
  CUtensorMap src_latent, src_rope;                  // the pool, boxes of 64 rows
  CUtensorMap dst_latent[kHeights], dst_rope[kHeights];  // the outputs, boxes of 64 >> h rows
};

struct GatherParams {
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  int32_t batch;
  int32_t block_size;
  int64_t pool_rows;
  const int64_t* out_row_offsets;
  int32_t* status;
};

__global__ void __launch_bounds__(32, 1) GatherTmaKernel(const __grid_constant__ GatherMaps maps, GatherParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = ptx::SmemAddr(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (stage0 - raw) + kStages * kStageBytes);
  int* first_tile = reinterpret_cast<int*>(full + kStages);  // [batch + 1]: tiles of the sequences before b
  GridDependencyTrigger();
  GridDependencyWait();
  {
    const int lane = threadIdx.x;
    int running = 0;
    for (int c = 0; c < p.batch; c += 32) {
      const int i = c + lane;
      const int len = i < p.batch ? p.kv_len[i] : 0;
      int incl = len > 0 ? (len + kTileRows - 1) / kTileRows : 0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
      }
      if (i < p.batch) first_tile[i + 1] = running + incl;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) first_tile[0] = 0;
    __syncwarp();
  }
  if (threadIdx.x != 0) return;  // one thread drives the copies; the rest of the warp has nothing more to do
  for (int s = 0; s < kStages; ++s) ptx::MbarInit(ptx::SmemAddr(&full[s]), 1);
  ptx::FenceBarrierInit();
  ptx::PrefetchTensorMap(&maps.src_latent);
  ptx::PrefetchTensorMap(&maps.src_rope);

  // This CTA's tiles: number cta, cta + G, ... of the flat list (sequence after sequence). The list is walked
  // twice in step, once for the loads (running kStages - 1 tiles ahead) and once for the stores.
  struct Walk {
    int flat;  // the next tile of this CTA in the flat list
    int b;     // a sequence at or before that tile's (the bisection starts there: tiles only move forward)
  };
  const int G = gridDim.x, cta = blockIdx.x;
  const int total_tiles = first_tile[p.batch];
  auto start = [&](Walk* w) {
    w->flat = cta;
    w->b = 0;
  };
  // This CTA's next tile; false at the end.
  auto next = [&](Walk* w, int* seq, int* tile, int* rows) -> bool {
    if (w->flat >= total_tiles) return false;
    int lo = w->b, hi = p.batch - 1;  // the last sequence whose first tile is at or before flat
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (first_tile[mid] <= w->flat) lo = mid; else hi = mid - 1;
    }
    w->b = lo;
    *seq = lo;
    *tile = w->flat - first_tile[lo];
    *rows = min(kTileRows, p.kv_len[lo] - *tile * kTileRows);
    w->flat += G;
    return true;
  };
  bool good[kStages];  // whether the tile in a stage came through a usable table entry: a bad one is not stored
  auto issue_load = [&](int seq, int tile, int i) {
    const int s = i % kStages;
    const int64_t tok = static_cast<int64_t>(tile) * kTileRows;
    const int64_t column = tok / p.block_size;
    const int64_t block = column < p.max_blocks ? p.block_table[static_cast<int64_t>(seq) * p.max_blocks + column] : -1;
    int64_t row = block * p.block_size + tok % p.block_size;
    good[s] = !(block < 0 || row + kTileRows > p.pool_rows);
    if (!good[s]) {
      RecordError(p.status, B200KV_DEV_BAD_BLOCK, seq, static_cast<int32_t>(column), static_cast<int32_t>(block));
      row = 0;  // the pipeline keeps its shape on addressable memory; nothing of this tile is written out
    }
    const uint32_t dst = stage0 + s * kStageBytes, bar = ptx::SmemAddr(&full[s]);
    ptx::MbarArriveExpectTx(bar, kStageBytes);
    ptx::TmaLoad2D(dst, &maps.src_latent, 0, static_cast<int32_t>(row), bar);
    ptx::TmaLoad2D(dst + kLatentBoxBytes, &maps.src_latent, kHalfLatent, static_cast<int32_t>(row), bar);
    ptx::TmaLoad2D(dst + 2 * kLatentBoxBytes, &maps.src_rope, 0, static_cast<int32_t>(row), bar);
  };

  Walk ahead, here;
  start(&ahead);
  start(&here);
  int seq, tile, rows, issued = 0;
  for (; issued < kStages - 1 && next(&ahead, &seq, &tile, &rows); ++issued) issue_load(seq, tile, issued);
  bool ok = true;
  for (int i = 0; ok && next(&here, &seq, &tile, &rows); ++i) {
    // The stage that tile i + 2 will use was read by the stores of tile i - 1: all but the latest group done.
    int seq2, tile2, rows2;
    if (next(&ahead, &seq2, &tile2, &rows2)) {
      ptx::BulkWaitGroupRead<0>();
      issue_load(seq2, tile2, issued);
      ++issued;
    }
    const int s = i % kStages;
    const uint32_t bar = ptx::SmemAddr(&full[s]);
    const uint64_t t0 = ptx::GlobalTimerNs();
    for (uint32_t spins = 0; !ptx::MbarTryWait(bar, (i / kStages) & 1); ++spins) {
      if ((spins & 255u) == 255u && ptx::GlobalTimerNs() - t0 > 1000000000ull) {
        RecordError(p.status, B200KV_DEV_TIMEOUT, 70, cta, i);
        ok = false;
        break;
      }
    }
    if (!ok) break;
    const uint32_t src = stage0 + s * kStageBytes;
    const int32_t out_row = static_cast<int32_t>(p.out_row_offsets[seq] + static_cast<int64_t>(tile) * kTileRows);
    int done = 0;
#pragma unroll
    for (int h = 0; h < kHeights; ++h) {
      const int height = kTileRows >> h;
      if (good[s] && rows - done >= height) {
        ptx::TmaStore2D(&maps.dst_latent[h], 0, out_row + done, src + done * (kHalfLatent * 2));
        ptx::TmaStore2D(&maps.dst_latent[h], kHalfLatent, out_row + done, src + kLatentBoxBytes + done * (kHalfLatent * 2));
        ptx::TmaStore2D(&maps.dst_rope[h], 0, out_row + done, src + 2 * kLatentBoxBytes + done * (B200KV_ROPE_DIM * 2));
        done += height;
      }
    }
    ptx::BulkCommitGroup();
  }
  // Nothing of this CTA's may still be reading shared memory, or on its way into it, when the CTA leaves.
  ptx::BulkWaitGroupRead<0>();
  if (!ok) {
    for (int i = max(0, issued - kStages); i < issued; ++i) {
      const uint64_t t0 = ptx::GlobalTimerNs();
      while (!ptx::MbarTryWait(ptx::SmemAddr(&full[i % kStages]), (i / kStages) & 1)) {
        if (ptx::GlobalTimerNs() - t0 > 200000000ull) break;
      }
    }
  }
}

}  // namespace

bool GatherTmaSupports(const b200kv_pool_view& pool, int64_t batch, int64_t block_size, int64_t out_latent_stride,
                       int64_t out_rope_stride, int64_t total_rows) {
  return batch <= kMaxBatch && block_size % kTileRows == 0 && pool.pool_rows <= INT32_MAX && total_rows <= INT32_MAX && pool.pool_rows >= kTileRows &&
         out_latent_stride % 8 == 0 && out_rope_stride % 8 == 0 && pool.latent_row_stride % 8 == 0 && pool.rope_row_stride % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(pool.latent) & 15u) == 0 && (reinterpret_cast<uintptr_t>(pool.rope) & 15u) == 0;
}

int32_t LaunchGatherTma(const b200kv_pool_view& pool, const int32_t* block_table, int64_t max_blocks, const int32_t* kv_len,
                        int32_t batch, int32_t block_size, void* out_latent, int64_t out_latent_stride, void* out_rope,
                        int64_t out_rope_stride, const int64_t* out_row_offsets, int64_t total_rows, cudaStream_t stream,
                        int32_t* status) {
  GatherMaps maps;
  if (int32_t rc = EncodePlainBf16Map(pool.latent, pool.latent_row_stride * 2, pool.pool_rows, B200KV_LATENT_DIM, kHalfLatent,
                                      kTileRows, &maps.src_latent)) return rc;
  if (int32_t rc = EncodePlainBf16Map(pool.rope, pool.rope_row_stride * 2, pool.pool_rows, B200KV_ROPE_DIM, B200KV_ROPE_DIM,
                                      kTileRows, &maps.src_rope)) return rc;
  for (int h = 0; h < kHeights; ++h) {
    if (int32_t rc = EncodePlainBf16Map(out_latent, out_latent_stride * 2, total_rows, B200KV_LATENT_DIM, kHalfLatent,
                                        kTileRows >> h, &maps.dst_latent[h])) return rc;
    if (int32_t rc = EncodePlainBf16Map(out_rope, out_rope_stride * 2, total_rows, B200KV_ROPE_DIM, B200KV_ROPE_DIM,
                                        kTileRows >> h, &maps.dst_rope[h])) return rc;
  }
  static thread_local int configured_device = -1;
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device != configured_device) {
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(GatherTmaKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                               "gather (TMA) smem opt-in")) return rc;
    configured_device = device;
  }
  GatherParams p{};
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.kv_len = kv_len;
  p.batch = batch;
  p.block_size = block_size;
  p.pool_rows = pool.pool_rows;
  p.out_row_offsets = out_row_offsets;
  p.status = status;
  const int64_t tiles = (total_rows + kTileRows - 1) / kTileRows + batch;  // an upper bound
  const int32_t sms = CurrentDeviceSmCount();
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  return CheckCuda(LaunchOverlapped(GatherTmaKernel, dim3(grid), dim3(32), kSmemBytes, stream, maps, p), "gather (TMA) launch");
}

}  // namespace b200kv
