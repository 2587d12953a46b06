// Split-KV absorbed-MLA decode attention on tcgen05 tensor cores (sm_100a), 64 heads x (512+64).
//
// Work partition. A sequence of L tokens is ceil(L/64) tiles. The tiles of all sequences form one flat
// list, which is cut into G contiguous runs by cost (CostCut below: a tile costs 2, entering another sequence
// in mid-run 3 more), one run per CTA. A CTA therefore walks a few "segments" (a tile range inside one
// sequence). A segment that covers its whole sequence writes the result directly; otherwise it writes an
// un-normalised partial (m, l, O) to the workspace and the finalize kernel merges the parts with a
// log-sum-exp reduction. Only the first and the last segment of a CTA can be partial, so the workspace holds
// two partial slots per CTA.
//
// Per tile of 64 tokens (one KV stage of 73,728 bytes: nine 64-column slabs, TMA-loaded, 128-byte
// swizzled, never multicast):
//   S[64 heads x 64 tok]  = Q[64 x 576] . K_tile^T            36 MMAs M=64  N=64 K=16 (K-major A, B)
//   P = exp2(S*scale*log2e - m)  (softmax warps, fp32 -> bf16, written over the stage's rope slab,
//                                 which QK has finished with)
//   O^T[512 x 64 heads]  += V_tile^T[512 x 64] . P^T[64 x 64]  16 MMAs M=128 N=64 K=16 (MN-major A)
// V is the first 512 columns of the same shared-memory tile that served as K: a tile is read from HBM
// once. O^T lives in TMEM (4 accumulators of 128 lanes x 64 columns), S double-buffered beside it.
// Measured on B200: one tcgen05.mma costs max(N/2, operand bytes/128, about 32) cycles whatever M is, so
// the tile is 64 tokens (N = 64 costs the same as N = 32) and PV runs transposed to use M = 128.
//
// Warp roles (224 threads): warps 0-3 softmax + epilogue (TMEM lanes 32w..32w+31); warp 4 TMA producer, its
// lanes sharing out a tile's loads (one thread issues a cp.async.bulk.tensor only every 170 cycles or so);
// warp 5 issues every QK and owns the TMEM allocation, warp 6 issues every PV: two independent instruction
// streams into the tensor pipe. Shared memory holds Q (72 KB) and two KV stages, each filled and given back
// in four slab groups.
//
// Every wait is bounded: when a wait runs out the kernel records B200KV_DEV_TIMEOUT in the status
// word, raises a CTA-wide abort flag, waits (bounded) for its own TMA loads, frees TMEM and returns.
#include <cuda.h>
#include <cuda_fp8.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kv_peer.cuh"
#include "sm100_ptx.cuh"

namespace b200kv {

namespace {

constexpr int kHeads = 64;
constexpr int kLatent = B200KV_LATENT_DIM;
constexpr int kRope = B200KV_ROPE_DIM;
constexpr int kTile = 64;      // tokens per tile / KV stage
constexpr int kStages = 2;
constexpr int kGroups = 4;                              // slab groups of a stage: slabs 2c, 2c+1 (and 8 with the last)
constexpr int kSlabBytes = kTile * 128;                 // one 64-column slab of a tile: kTile rows x 128 B
constexpr int kStageBytes = 9 * kSlabBytes;             // 73,728
constexpr int kQSlabBytes = kHeads * 128;               // 8,192
constexpr int kQBytes = 9 * kQSlabBytes;                // 73,728
constexpr int kSoftmaxThreads = 128;
constexpr int kSoftmaxWarps = kSoftmaxThreads / 32;     // one lane of each arrives on the barriers they signal
constexpr int kThreads = 224;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemColS = 256;                     // S buffers at columns 256 and 256 + kTile
constexpr float kRescaleThreshold = 8.0f;               // log2 units: rescale O only when max grows by > 2^8

// Shared memory carve-up (offsets from a 1024-byte aligned base).
constexpr int kOffQ = 0;
constexpr int kOffKv = kOffQ + kQBytes;
constexpr int kOffMisc = kOffKv + kStages * kStageBytes;
constexpr int kMiscBytes = 4096;
constexpr int kSmemBytes = kOffMisc + kMiscBytes + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");

struct Misc {
  // A stage is filled, consumed and given back in four groups of slabs (0-1, 2-3, 4-5, 6-8): QK starts on a
  // tile's first group while the rest is landing, and PV, which runs one 128-column accumulator after the other,
  // gives the first group back after a quarter of its work, so the reload of a stage overlaps the PV that is
  // still reading its other slabs.
  uint64_t kv_full[kStages][kGroups];
  uint64_t kv_empty[kStages][kGroups];
  uint64_t s_full[2];
  uint64_t s_empty[2];
  uint64_t p_full[kStages];
  uint64_t q_full[kGroups];  // Q lands in the same four slab groups as a stage: QK starts on the first
  uint64_t q_empty;
  uint64_t o_full;
  uint64_t o_empty;
  uint64_t drain[2];
  uint32_t tmem_base;
  int32_t abort_flag;
  int32_t start_seq;
  int32_t start_tile;
  int32_t n_tiles;
  float factor[kHeads];
  float inv_l[kHeads];
  // Fused append: the sequence's new row (512 latent + 64 rope bf16) on its way from the caller's buffer to
  // the pool, and the barrier its bulk load completes on.
  alignas(16) unsigned char new_row[(kLatent + kRope) * 2];
  uint64_t new_row_full;
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc does not fit its reservation");

struct TcParams {
  const __nv_bfloat16* q;
  int64_t q_seq_stride;
  int64_t q_head_stride;
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  const int32_t* kv_begin;
  int64_t pool_rows;
  // Fused append (null = none): the new rows, and the pool once more as plain pointers to write them through.
  const char* new_latent;
  const char* new_rope;
  int64_t new_latent_bytes;  // row strides in bytes
  int64_t new_rope_bytes;
  char* pool_latent;
  char* pool_rope;
  int64_t pool_latent_bytes;
  int64_t pool_rope_bytes;
  int32_t batch;
  int32_t block_size;
  int32_t stable_tables;  // lengths and block table may be read before the stream dependency wait
  int32_t force_ws;       // every segment leaves a partial in the workspace, one that covers its sequence too
  const int32_t* row_index;  // [B][row_index_stride]: the pool rows to attend over, in place of the block table; or null
  int64_t row_index_stride;
  float scale_log2;  // scale * log2(e)
  __nv_bfloat16* out;
  uint8_t* out_q;      // [B][64][512] FP8 E4M3 of out, MX block 32 along a head's row; or null
  uint8_t* out_scale;  // [B][64][16] E8M0
  float* lse;
  float* user_o;  // caller's partial buffers (shard mode) or null
  float* user_m;
  float* user_l;
  // Partials, one slot per (CTA, first / later segment): [2G slots][16 head quads][512 dv][4 heads] fp32, and
  // (m, l) as [2G][64]. A thread of the epilogue owns one dv (a TMEM lane) and reads its heads as consecutive
  // registers: four heads make a 16-byte store, and the 32 lanes of a warp (32 consecutive dv) write 512
  // contiguous bytes per instruction. The merge kernel reads the same lines the same way, lanes along dv,
  // which is also the order of the output rows: nothing has to be turned round.
  float* ws_o;
  int32_t n_slots;  // 2G
  float* ws_m;  // [2G][64]
  float* ws_l;
  int32_t* status;
};

__device__ __forceinline__ int TilesOf(int len) { return (len + kTile - 1) / kTile; }

__device__ __forceinline__ bool Aborting(const Misc* misc) {
  return *reinterpret_cast<const volatile int32_t*>(&misc->abort_flag) != 0;
}

__device__ __noinline__ void RaiseTimeout(Misc* misc, int32_t* status, int site, uint32_t parity) {
  *reinterpret_cast<volatile int32_t*>(&misc->abort_flag) = 1;
  RecordError(status, B200KV_DEV_TIMEOUT, site, static_cast<int32_t>(blockIdx.x), static_cast<int32_t>(parity));
}

// Bounded mbarrier wait. Returns false when the CTA is aborting or this wait ran out (about one
// second), after recording where.
__device__ __noinline__ bool BoundedWait(uint32_t bar, uint32_t parity, Misc* misc, int32_t* status, int site) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    if (ptx::MbarTryWait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (Aborting(misc)) return false;
      const uint64_t now = ptx::GlobalTimerNs();
      if (start == 0) start = now;
      if (now - start > 1000000000ull) {
        RaiseTimeout(misc, status, site, parity);
        return false;
      }
    }
  }
}

// The same with a non-blocking probe in a tight loop. mbarrier.try_wait parks the thread and, measured here, a
// parked thread resumes some 500 cycles after the phase completes; the producer's waits sit on the path that
// refills a stage, so it spins instead (one thread: the issue slots it takes are few).
__device__ __noinline__ bool BoundedSpin(uint32_t bar, uint32_t parity, Misc* misc, int32_t* status, int site) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    if (ptx::MbarTestWait(bar, parity)) return true;
    if ((it & 1023u) == 1023u) {
      if (Aborting(misc)) return false;
      const uint64_t now = ptx::GlobalTimerNs();
      if (start == 0) start = now;
      if (now - start > 1000000000ull) {
        RaiseTimeout(misc, status, site, parity);
        return false;
      }
    }
  }
}

// ---- work partition -----------------------------------------------------------------------------------
// The tiles of all sequences form one flat list (sequence after sequence, empty ones contribute nothing).
// Cutting that list into G equal runs of tiles leaves the CTAs uneven: a CTA whose run crosses from one
// sequence into the next reloads Q and drains its accumulators in mid-run, which costs it about as much
// as one and a half tiles. So the list is cut by cost instead: a tile costs 2, entering a new sequence
// costs 3 more. Tile x of the sequence with ordinal s (among the non-empty ones) sits at cost position
// 2x + 3s; with C = 2T + 3(S - 1) the total, CTA c takes the tiles whose position lies in
// [ceil(c*C/G), ceil((c+1)*C/G)). Both kernels derive everything from these two functions.
struct CostCut {
  long long cost_total;  // C, at least 2 when there is any tile
  long long n_ctas;      // G
  // Non-negative quotient; the 32-bit division is several times shorter and covers every realistic size.
  __device__ static long long Div(long long a, long long b) {
    if (((a | b) >> 32) == 0) return static_cast<long long>(static_cast<uint32_t>(a) / static_cast<uint32_t>(b));
    return a / b;
  }
  static constexpr long long kTileCost = 2;   // one tile of 64 tokens
  static constexpr long long kCrossCost = 3;  // entering another sequence in mid-run
  __device__ static long long Pos(long long x, long long s) { return kTileCost * x + kCrossCost * s; }
  __device__ static long long Total(long long tiles, long long nonempty) {
    return kTileCost * tiles + kCrossCost * (nonempty > 0 ? nonempty - 1 : 0);
  }
  __device__ long long CtaOf(long long x, long long s) const { return Div(Pos(x, s) * n_ctas, cost_total); }
  __device__ long long FirstPos(long long c) const { return Div(c * cost_total + n_ctas - 1, n_ctas); }
  // First tile of a sequence (first tile `first`, ordinal s) at or after cost position k.
  __device__ long long FirstTileAt(long long k, long long first, long long s) const {
    static_assert(kTileCost == 2, "the ceiling below divides by the tile cost with a shift");
    const long long x = (k - kCrossCost * s + 1) >> 1;  // ceil((k - cross * s) / 2), also right for negative values
    return x > first ? x : first;
  }
};

// Walks the segments of this CTA's tile range. All roles run the same iterator.
struct SegmentWalker {
  const int32_t* kv_len;
  int batch;
  int seq;
  int tile;       // first tile of the segment inside `seq`
  int remaining;  // tiles left for this CTA
  __device__ SegmentWalker(const int32_t* lens, int batch_, int seq_, int tile_, int remaining_)
      : kv_len(lens), batch(batch_), seq(seq_), tile(tile_), remaining(remaining_) {}
  // Fills the current segment; returns false when the CTA's range is exhausted.
  __device__ bool Next(int* seq_out, int* tile_lo, int* tile_hi, int* seq_tiles, int* seq_len) {
    while (remaining > 0 && seq < batch) {
      const int len = kv_len[seq];
      const int tiles = TilesOf(len);
      if (tile < tiles) {
        const int take = min(remaining, tiles - tile);
        *seq_out = seq;
        *tile_lo = tile;
        *tile_hi = tile + take;
        *seq_tiles = tiles;
        *seq_len = len;
        remaining -= take;
        tile += take;
        if (tile == tiles) {
          tile = 0;
          ++seq;
        }
        return true;
      }
      tile = 0;
      ++seq;
    }
    return false;
  }
};

// A 64-bit shared-memory descriptor whose start address is advanced by adding to the low word.
__device__ __forceinline__ uint64_t DescAt(uint64_t base_desc, uint32_t byte_offset) {
  return base_desc + static_cast<uint64_t>(byte_offset >> 4);
}

// The QK k-steps of kSlabs 64-column slabs (four each) starting at slab kFirstSlab; called by the whole MMA warp.
template <int kFirstSlab, int kSlabs>
__device__ __forceinline__ void IssueQkGroup(uint64_t q_desc, uint64_t kdesc, uint32_t d) {
  constexpr uint32_t kIdescQk = ptx::InstrDescBf16(64, kTile, 0, 0);
#pragma unroll
  for (int i = 0; i < 4 * kSlabs; ++i) {
    const int c = kFirstSlab + (i >> 2), kk = i & 3;
    const uint64_t a = DescAt(q_desc, c * kQSlabBytes + kk * 32);
    const uint64_t b = DescAt(kdesc, c * kSlabBytes + kk * 32);
    if (ptx::ElectOne()) ptx::MmaF16SS(d, a, b, kIdescQk, (kFirstSlab + i) > 0 ? 1u : 0u);
  }
}

// kGathered: the tiles are runs of 64 entries of a list of pool rows (TcParams::row_index) instead of runs of 64
// tokens of a block; a separate instantiation, so that the dense kernel's code is not touched by it.
template <bool kGathered>
__global__ void __launch_bounds__(kThreads, 1)
    MlaDecodeTcKernel(const __grid_constant__ CUtensorMap latent_map, const __grid_constant__ CUtensorMap rope_map,
                      const __grid_constant__ CUtensorMap q_map, TcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = ptx::SmemAddr(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* smem = smem_dyn + (base - raw);
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t q_addr = base + kOffQ;
  const uint32_t kv_addr = base + kOffKv;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int n_ctas = gridDim.x;

  auto bar = [&](const uint64_t* b) { return ptx::SmemAddr(b); };

  // ---- setup ----------------------------------------------------------------------------------
  // The finalize kernel may be scheduled as SMs free up. It reads the lengths before it waits for this kernel, so
  // unless the caller vouches for them (B200KV_DECODE_STABLE_TABLES) it is let go only once this kernel's own
  // wait for the preceding kernel has returned (below).
  if (p.stable_tables != 0) GridDependencyTrigger();

  // One tile's nine TMA loads (eight latent slabs, one rope slab) into stage g % kStages.
  // A tile is dead in L2 once it has been loaded.
  const uint64_t drop_policy = ptx::L2PolicyEvictFirst();
  // Pool row at which tile t of a sequence starts, through the block table; -1 (after recording it) when the
  // table entry is missing or points outside the pool.
  auto tile_row_checked = [&](int seq, int begin, int t) -> int64_t {
    const int tok = begin + t * kTile;
    const int64_t table_col = tok / p.block_size;
    const int64_t block =
        table_col < p.max_blocks ? p.block_table[static_cast<int64_t>(seq) * p.max_blocks + table_col] : -1;
    int64_t row = block * p.block_size + tok % p.block_size;
    if (block < 0 || row + kTile > p.pool_rows) {
      RecordError(p.status, B200KV_DEV_BAD_BLOCK, seq, tok / p.block_size, static_cast<int32_t>(block));
      row = -1;
    }
    return row;
  };
  // For loads: a bad entry reads row 0 instead, which keeps the pipeline moving on addressable memory (the
  // status word tells the host that the result is void). Nothing is ever written through a bad entry.
  auto tile_row = [&](int seq, int begin, int t) -> int64_t {
    const int64_t row = tile_row_checked(seq, begin, t);
    return row < 0 ? 0 : row;
  };
  // Group c of a tile into stage g % kStages: slabs 2c and 2c + 1, and the rope slab with the last group.
  auto issue_group = [&](int64_t row, int g, int c) {
    const int stage = g % kStages;
    const uint32_t dst = kv_addr + stage * kStageBytes;
    const uint32_t full = bar(&misc->kv_full[stage][c]);
    ptx::MbarArriveExpectTx(full, (c == kGroups - 1 ? 3 : 2) * kSlabBytes);
    ptx::TmaLoad2DHint(dst + 2 * c * kSlabBytes, &latent_map, 128 * c, static_cast<int32_t>(row), full, drop_policy);
    ptx::TmaLoad2DHint(dst + (2 * c + 1) * kSlabBytes, &latent_map, 128 * c + 64, static_cast<int32_t>(row), full, drop_policy);
    if (c == kGroups - 1) ptx::TmaLoad2DHint(dst + 8 * kSlabBytes, &rope_map, 0, static_cast<int32_t>(row), full, drop_policy);
  };
  // The producer warp spreads a tile's TMA instructions over its lanes: one thread needs some 170 cycles per
  // cp.async.bulk.tensor, so nine loads and nine prefetches issued by one thread take a whole tile period.
  // Lane s < 9 owns slab s (its group: slabs 0-1, 2-3, 4-5, 6-8) and lanes 0, 2, 4, 6 announce their group's bytes;
  // the barrier counts one arrival, so a phase cannot complete before its announcement, whichever lane's
  // instruction comes first. (Bringing the next tile into L2 with TMA prefetches from further lanes, which paid
  // while one thread issued everything, now only takes TMA slots from the loads: 43.0 us per launch with, 42.4
  // without.)
  const int my_group = lane < 6 ? (lane >> 1) : 3;
  auto issue_slab = [&](int64_t row, int g) {  // lanes 0 .. 8
    const int stage = g % kStages;
    const uint32_t dst = kv_addr + stage * kStageBytes + lane * kSlabBytes;
    const uint32_t full = bar(&misc->kv_full[stage][my_group]);
    if (lane < 8 && (lane & 1) == 0) ptx::MbarArriveExpectTx(full, (my_group == kGroups - 1 ? 3 : 2) * kSlabBytes);
    if (lane < 8) {
      ptx::TmaLoad2DHint(dst, &latent_map, 64 * lane, static_cast<int32_t>(row), full, drop_policy);
    } else {
      ptx::TmaLoad2DHint(dst, &rope_map, 0, static_cast<int32_t>(row), full, drop_policy);
    }
  };
  // A tile of gathered rows (row_index in place of the block table): entries 64 t .. 64 t + 63 of the sequence's
  // row list. The producer warp copies them with 16-byte asynchronous copies, doing the 128-byte swizzle in the
  // address arithmetic: chunk c of tile row r goes to r * 128 + ((c ^ (r % 8)) * 16) of its slab, which is where
  // a swizzled TMA load would have put it. An instruction of the warp moves four rows' 128 bytes of one slab
  // (lane = row within the four x chunk), 144 instructions a tile. (The gathering form of the TMA load, four
  // rows of one slab per instruction, was measured first: the TMA unit spends some 90 cycles on an instruction
  // whatever its size, so 144 of them a tile made a tile five microseconds long.) The copies of a group arrive
  // on the group's barrier, which in this mode counts the warp's 32 lanes instead of one announcement of bytes;
  // they write through the generic proxy, so the warps that issue MMAs fence after their wait. The warp takes
  // the tile group by group as PV gives the stage back. Entries past the sequence's length are not read (their
  // rows load as row 0 and the softmax masks them); an entry inside it that is not a row of the pool is recorded
  // and reads row 0.
  // The row numbers of a tile are read a tile ahead (gathered_rows fills `rid` for the tile the next call of
  // issue_gathered copies), so their latency lies under the previous tile's copies instead of in front of
  // this tile's.
  const int g_sub = lane >> 3;          // row within each run of four
  const uint32_t g_chunk = lane & 7;    // 16-byte chunk of the slab's 128-byte row
  int rid[kTile / 4];
  auto gathered_rows = [&](int seq, int seq_len, int t) {
#pragma unroll
    for (int q = 0; q < kTile / 4; ++q) {
      const int j = t * kTile + 4 * q + g_sub;
      int row = 0;
      if (j < seq_len && j < p.row_index_stride) row = p.row_index[static_cast<int64_t>(seq) * p.row_index_stride + j];
      rid[q] = row;
    }
  };
  auto issue_gathered = [&](int seq, int g) -> bool {
    const int stage = g % kStages;
#pragma unroll
    for (int q = 0; q < kTile / 4; ++q) {
      if (rid[q] < 0 || rid[q] >= p.pool_rows) {
        if (g_chunk == 0) RecordError(p.status, B200KV_DEV_BAD_BLOCK, seq, 4 * q + g_sub, rid[q]);
        rid[q] = 0;
      }
    }
    const char* latent_lane = p.pool_latent + g_chunk * 16;
    const uint32_t dst_lane = kv_addr + stage * kStageBytes + g_sub * 128;
    bool ok = true;
#pragma unroll 1
    for (int c = 0; c < kGroups && ok; ++c) {
      if (g >= kStages) {
        ok = __all_sync(0xffffffffu, BoundedSpin(bar(&misc->kv_empty[stage][c]), ((g / kStages) & 1) ^ 1, misc, p.status, 10));
        if (!ok) break;
      }
#pragma unroll 1
      for (int k = 0; k < 2; ++k) {
        const int slab = 2 * c + k;
#pragma unroll
        for (int q = 0; q < kTile / 4; ++q) {
          // row r = 4 q + g_sub, so r % 8 = 4 (q % 2) + g_sub
          ptx::CpAsync16(dst_lane + slab * kSlabBytes + q * 512 + ((g_chunk ^ (4 * (q & 1) + g_sub)) << 4),
                         latent_lane + rid[q] * p.pool_latent_bytes + slab * 128);
        }
      }
      if (c == kGroups - 1) {
#pragma unroll
        for (int q = 0; q < kTile / 4; ++q) {
          ptx::CpAsync16(dst_lane + 8 * kSlabBytes + q * 512 + ((g_chunk ^ (4 * (q & 1) + g_sub)) << 4),
                         p.pool_rope + rid[q] * p.pool_rope_bytes + g_chunk * 16);
        }
      }
      ptx::CpAsyncArriveOn(bar(&misc->kv_full[stage][c]));
    }
    return ok;
  };
  // Fused append, first half: the new row of `seq` starts towards shared memory.
  auto new_row_fetch = [&](int seq) {
    const uint32_t full = bar(&misc->new_row_full);
    ptx::MbarArriveExpectTx(full, (kLatent + kRope) * 2);
    ptx::BulkLoad(ptx::SmemAddr(misc->new_row), p.new_latent + seq * p.new_latent_bytes, kLatent * 2, full);
    ptx::BulkLoad(ptx::SmemAddr(misc->new_row) + kLatent * 2, p.new_rope + seq * p.new_rope_bytes, kRope * 2, full);
  };
  // Second half, just before the load of the tile that holds the row: shared memory -> pool row with plain
  // stores (72 x 16 bytes, one thread), made visible to the TMA load that follows. `parity` counts this CTA's
  // appends.
  auto new_row_store = [&](int64_t row, uint32_t parity) -> bool {
    if (!BoundedWait(bar(&misc->new_row_full), parity, misc, p.status, 12)) return false;
    if (row < 0) return true;  // bad table entry: the fetched row is consumed (parities stay in step), not stored
    const int4* src = reinterpret_cast<const int4*>(misc->new_row);
    int4* latent_dst = reinterpret_cast<int4*>(p.pool_latent + row * p.pool_latent_bytes);
    int4* rope_dst = reinterpret_cast<int4*>(p.pool_rope + row * p.pool_rope_bytes);
#pragma unroll 8
    for (int i = 0; i < kLatent / 8; ++i) latent_dst[i] = src[i];
#pragma unroll
    for (int i = 0; i < kRope / 8; ++i) rope_dst[i] = src[kLatent / 8 + i];
    __threadfence();
    ptx::FenceProxyAsync();
    return true;
  };
  // Q of one sequence: nine 64-column slabs of 64 head rows.
  auto issue_q = [&](int seq) {  // lanes 0 .. 8, one slab each, completing on its group's barrier
    const uint32_t qbar = bar(&misc->q_full[my_group]);
    if (lane < 8 && (lane & 1) == 0) ptx::MbarArriveExpectTx(qbar, (my_group == kGroups - 1 ? 3 : 2) * kQSlabBytes);
    ptx::TmaLoad3D(q_addr + lane * kQSlabBytes, &q_map, 64 * lane, 0, seq, qbar);
  };

  int pre_issued = 0;  // tiles the producer put in flight before the CTA-wide setup barrier
  if (warp == 4) {
    // The producer warp initialises the barriers, finds this CTA's slice of the flat tile list and
    // puts Q and the first tiles in flight at once: the other warps' setup (TMEM allocation, the
    // barrier below) then overlaps the first loads' latency instead of preceding it.
    // The lengths are the head of a chain of dependent loads (lengths, block table, tiles): when the caller
    // vouches for them their load goes out first and the barrier set-up runs under its latency.
    int early_len = 0;
    if (p.stable_tables != 0 && lane < p.batch) early_len = p.kv_len[lane];
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) {
        for (int k = 0; k < kGroups; ++k) {
          ptx::MbarInit(bar(&misc->kv_full[s][k]), kGathered ? 32 : 1);  // gathered: one arrival a lane
          ptx::MbarInit(bar(&misc->kv_empty[s][k]), 1);
        }
        ptx::MbarInit(bar(&misc->p_full[s]), kSoftmaxWarps);
      }
      for (int s = 0; s < 2; ++s) {
        ptx::MbarInit(bar(&misc->s_full[s]), 1);
        ptx::MbarInit(bar(&misc->s_empty[s]), kSoftmaxWarps);
      }
      ptx::MbarInit(bar(&misc->new_row_full), 1);
      for (int k = 0; k < kGroups; ++k) ptx::MbarInit(bar(&misc->q_full[k]), 1);
      ptx::MbarInit(bar(&misc->q_empty), 1);
      ptx::MbarInit(bar(&misc->o_full), 1);
      ptx::MbarInit(bar(&misc->o_empty), kSoftmaxWarps);
      ptx::MbarInit(bar(&misc->drain[0]), 1);
      ptx::MbarInit(bar(&misc->drain[1]), 1);
      misc->abort_flag = 0;
      ptx::FenceBarrierInit();
      ptx::PrefetchTensorMap(&latent_map);
      ptx::PrefetchTensorMap(&rope_map);
      ptx::PrefetchTensorMap(&q_map);
    }
    __syncwarp();
    // Up to here nothing read memory that an earlier kernel in the stream may still be writing, so under
    // a programmatic dependent launch the lines above overlap that kernel's tail. From here on the
    // lengths, the block table, Q and the pool are read.
    if (p.stable_tables == 0) GridDependencyWait();
    // This CTA's run of the flat tile list (see CostCut): totals first, then the tile at which the run
    // starts and the tile at which the next CTA's run starts.
    // Per-lane and per-chunk quantities are 32-bit (a sequence has at most 2^25 tiles, a chunk of 32 at most
    // 2^30); only the running totals are 64-bit. This warp's instruction count is on every launch's critical
    // path, so the scans are kept short.
    long long total = 0, nonempty = 0;
    const int first_tiles =  // the first chunk's lengths, kept
        lane < p.batch ? TilesOf(p.stable_tables != 0 ? early_len : p.kv_len[lane]) : 0;
    for (int b0 = 0; b0 < p.batch; b0 += 32) {
      int t = b0 == 0 ? first_tiles : (b0 + lane < p.batch ? TilesOf(p.kv_len[b0 + lane]) : 0);
      int ne = t > 0 ? 1 : 0;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        t += __shfl_xor_sync(0xffffffffu, t, off);
        ne += __shfl_xor_sync(0xffffffffu, ne, off);
      }
      total += t;
      nonempty += ne;
    }
    const CostCut cut{CostCut::Total(total, nonempty), n_ctas};
    // One pass over the sequences finds both the first tile at or after this CTA's first cost position
    // (flat index `lo`, its sequence, that sequence's first flat index and tile count) and the first tile
    // at or after the next CTA's (`hi`); either is `total` when no tile is left.
    int start_seq = p.batch, start_seq_tiles = 0;
    long long start_first = 0;
    long long lo = total, hi = total;
    if (total > 0) {
      const long long k_lo = cut.FirstPos(cta), k_hi = cut.FirstPos(cta + 1);
      bool have_lo = false, have_hi = false;
      long long before = 0, before_s = 0;
      for (int b0 = 0; b0 < p.batch && !have_hi; b0 += 32) {
        const int mine = b0 == 0 ? first_tiles : (b0 + lane < p.batch ? TilesOf(p.kv_len[b0 + lane]) : 0);
        int incl = mine, incl_s = mine > 0 ? 1 : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, off);
          const int up_s = __shfl_up_sync(0xffffffffu, incl_s, off);
          if (lane >= off) {
            incl += up;
            incl_s += up_s;
          }
        }
        const long long s = before_s + incl_s - 1;                      // ordinal of this lane's sequence, if not empty
        const long long last_pos = CostCut::Pos(before + incl - 1, s);     // cost position of its last tile
        const unsigned hit_lo = __ballot_sync(0xffffffffu, mine > 0 && last_pos >= k_lo);
        const unsigned hit_hi = __ballot_sync(0xffffffffu, mine > 0 && last_pos >= k_hi);
        if (!have_lo && hit_lo != 0) {
          const int src = __ffs(hit_lo) - 1;
          start_first = before + __shfl_sync(0xffffffffu, incl - mine, src);
          start_seq = b0 + src;
          start_seq_tiles = __shfl_sync(0xffffffffu, mine, src);
          lo = cut.FirstTileAt(k_lo, start_first, before_s + __shfl_sync(0xffffffffu, incl_s, src) - 1);
          have_lo = true;
        }
        if (hit_hi != 0) {
          const int src = __ffs(hit_hi) - 1;
          const long long first = before + __shfl_sync(0xffffffffu, incl - mine, src);
          hi = cut.FirstTileAt(k_hi, first, before_s + __shfl_sync(0xffffffffu, incl_s, src) - 1);
          have_hi = true;
        }
        before += __shfl_sync(0xffffffffu, incl, 31);
        before_s += __shfl_sync(0xffffffffu, incl_s, 31);
      }
    }
    const int start_tile = static_cast<int>(lo - start_first);
    if (lane == 0) {
      misc->start_seq = start_seq;
      misc->start_tile = start_tile;
      misc->n_tiles = static_cast<int>(hi - lo);
    }
    // Everything below is the same in every lane (the values above came out of shuffles); lanes 0 .. 8 issue.
    if (hi > lo && start_seq < p.batch) {
      const int begin = p.kv_begin ? p.kv_begin[start_seq] : 0;
      // A tile that a fused append still has to write into is left to the main loop.
      const int t_end = min(start_seq_tiles - (p.new_latent != nullptr ? 1 : 0), start_tile + static_cast<int>(hi - lo));
      static_assert(kStages == 2, "the first tiles' rows are looked up before the dependency wait, two of them");
      // (Gathered rows: every tile goes out from the main loop, which reads the row numbers after the wait.)
      const int n_first = kGathered ? 0 : max(0, min(kStages, t_end - start_tile));
      const int64_t row0 = n_first > 0 ? tile_row(start_seq, begin, start_tile) : 0;
      const int64_t row1 = n_first > 1 ? tile_row(start_seq, begin, start_tile + 1) : 0;
      if (p.stable_tables != 0) GridDependencyWait();  // Q and the pool are the preceding kernels' to write
      // Group by group, Q's slabs and the first tile's together: QK starts when the first group of both has
      // landed, a quarter of the way into the 144 KB, not at its end.
      for (int c = 0; c < kGroups; ++c) {
        if (lane < 9 && my_group == c) {
          issue_q(start_seq);
          if (n_first > 0) issue_slab(row0, 0);
        }
      }
      if (lane < 9 && n_first > 1) issue_slab(row1, 1);
      pre_issued = n_first;
    } else if (p.stable_tables != 0) {
      GridDependencyWait();
    }
    __syncwarp();
  }
  if (warp == 5) {
    ptx::TmemAlloc(ptx::SmemAddr(&misc->tmem_base), kTmemCols);
    ptx::TmemRelinquish();
  }
  GridDependencyWait();  // every thread, before it reads anything of the caller's
  if (p.stable_tables == 0) GridDependencyTrigger();
  ptx::TcFenceBeforeSync();
  __syncthreads();
  ptx::TcFenceAfterSync();

  const uint32_t tmem = misc->tmem_base;
  const int start_seq = misc->start_seq;
  const int start_tile = misc->start_tile;
  const int my_tiles = misc->n_tiles;

  if (warp == 4) {
    // ======================= TMA producer =======================================================
    // All lanes walk the segments together; what a lane issues depends on its number (see issue_slab).
    {
      SegmentWalker walk(p.kv_len, p.batch, start_seq, start_tile, my_tiles);
      int seq, t_lo, t_hi, seq_tiles, seq_len;
      int g = 0;  // tiles issued
      bool ok = true;
      int seg = 0;
      uint32_t n_appended = 0;
      bool fetch_pending = false;  // a new row's bulk load is in flight towards shared memory
      bool rows_ahead = false;     // gathered rows: `rid` already holds the row numbers of the tile to come
      const bool loader = lane < 9;
      while (ok && walk.Next(&seq, &t_lo, &t_hi, &seq_tiles, &seq_len)) {
        // Q of this segment's sequence, once the previous segment's last QK has finished reading the
        // buffer (the first segment's Q went out before the setup barrier).
        if (seg > 0) {
          ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->q_empty), (seg - 1) & 1, misc, p.status, 11));
          if (!ok) break;
          if (loader) issue_q(seq);
        }
        ++seg;
        const int begin = p.kv_begin ? p.kv_begin[seq] : 0;
        const bool appends = p.new_latent != nullptr && t_hi == seq_tiles;  // this segment holds the sequence's end
        if (appends) {
          if (lane == 0) new_row_fetch(seq);
          fetch_pending = true;
        }
        for (int t = t_lo; t < t_hi; ++t, ++g) {
          if (g < pre_issued) continue;
          if constexpr (kGathered) {
            if (!rows_ahead) gathered_rows(seq, seq_len, t);  // the CTA's first tile
            ok = issue_gathered(seq, g);
            if (!ok) break;
            // The next tile's row numbers start on their way now: the next tile of this segment, or the first of
            // the next segment (whose sequence and length the walker's copy below looks up).
            rows_ahead = false;
            if (t + 1 < t_hi) {
              gathered_rows(seq, seq_len, t + 1);
              rows_ahead = true;
            } else {
              SegmentWalker peek = walk;
              int seq2, lo2, hi2, tiles2, len2;
              if (peek.Next(&seq2, &lo2, &hi2, &tiles2, &len2)) {
                gathered_rows(seq2, len2, lo2);
                rows_ahead = true;
              }
            }
            continue;
          }
          const int64_t checked_row = tile_row_checked(seq, begin, t);
          const int64_t row = checked_row < 0 ? 0 : checked_row;
          if (appends && t == seq_tiles - 1) {
            // The tile that receives the new row: one lane writes the row and then issues the tile's loads itself,
            // so that its stores, its fences and its loads are one thread's program order.
            if (lane == 0) {
              ok = new_row_store(checked_row < 0 ? -1 : checked_row + (seq_len - 1 - t * kTile), n_appended & 1);
              for (int c = 0; c < kGroups && ok; ++c) {
                if (g >= kStages) {
                  ok = BoundedSpin(bar(&misc->kv_empty[g % kStages][c]), ((g / kStages) & 1) ^ 1, misc, p.status, 10);
                }
                if (ok) issue_group(row, g, c);
              }
            }
            ++n_appended;
            fetch_pending = false;
          } else if (g < kStages) {
            if (loader) issue_slab(row, g);
          } else {
            // The warp polls together and a lane issues its slab inside the loop, the moment its group has been
            // given back: PV releases a stage group by group, and lanes that left a spin loop of their own would
            // wait for each other at the loop's end before any of them issued.
            const uint32_t empty = bar(&misc->kv_empty[g % kStages][my_group]);
            const uint32_t parity = ((g / kStages) & 1) ^ 1;
            bool done = !loader;
            uint64_t start = 0;
            for (uint32_t it = 0;; ++it) {
              if (!done && ptx::MbarTestWait(empty, parity)) {
                issue_slab(row, g);
                done = true;
              }
              if (__all_sync(0xffffffffu, done)) break;
              if ((it & 1023u) == 1023u) {
                const uint64_t now = ptx::GlobalTimerNs();
                if (start == 0) start = now;
                if (Aborting(misc) || now - start > 1000000000ull) {
                  if (!Aborting(misc) && lane == 0) RaiseTimeout(misc, p.status, 10, parity);
                  ok = false;
                  break;
                }
              }
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
      }
      if (lane == 0 && !ok && fetch_pending) {
        const uint64_t t0 = ptx::GlobalTimerNs();
        while (!ptx::MbarTryWait(bar(&misc->new_row_full), n_appended & 1)) {
          if (ptx::GlobalTimerNs() - t0 > 200000000ull) break;
        }
      }
      if (lane == 0 && !ok) {
        // Aborting: let the loads this warp issued land before the CTA exits. A stage whose load
        // was issued at count i (the last one for that stage) completes phase (i / kStages) & 1.
        for (int s = 0; s < kStages; ++s) {
          int last = -1;
          for (int i = g - 1; i >= 0 && i >= g - kStages; --i) {
            if (i % kStages == s) {
              last = i;
              break;
            }
          }
          if (last < 0) continue;
          const uint32_t parity = (last / kStages) & 1;
          const uint64_t t0 = ptx::GlobalTimerNs();
          for (int k = 0; k < kGroups; ++k) {
            while (!ptx::MbarTryWait(bar(&misc->kv_full[s][k]), parity)) {
              if (ptx::GlobalTimerNs() - t0 > 200000000ull) break;
            }
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == 5 || warp == 6) {
    // ======================= MMA issuers =========================================================
    // Warp 5 issues every QK, warp 6 every PV: two independent instruction streams into the tensor
    // pipe, so a PV whose P has just become ready never queues behind a 36-instruction QK burst, and
    // each warp waits with plain blocking waits. A whole warp runs its loop in lockstep and each
    // tcgen05 instruction sits under elect.sync: measured on B200, that form issues an M=64 N=64 MMA
    // every 34 cycles against 46-58 for a single-thread or lane-predicated loop. elect.sync picks the
    // same lane every time, so a warp's commits track the MMAs that warp issued.
    {
      constexpr uint32_t kIdescPv = ptx::InstrDescBf16(128, kHeads, 1, 0);
      const bool is_qk = warp == 5;
      // Descriptor templates; the start address is advanced by adding to the low word.
      const uint64_t q_desc = ptx::SmemDescSw128(q_addr, 16, 1024);            // K-major, 8-row groups 1024 B apart
      const uint64_t k_desc0 = ptx::SmemDescSw128(kv_addr, 16, 1024);          // K-major B (tile rows = N)
      const uint64_t v_desc0 = ptx::SmemDescSw128(kv_addr, kSlabBytes, 1024);  // MN-major A: next 64 dv at +slab
      SegmentWalker walk(p.kv_len, p.batch, start_seq, start_tile, my_tiles);
      int seq, t_lo, t_hi, seq_tiles, seq_len;
      int g0 = 0;   // global index of the segment's first tile
      int seg = 0;  // segment counter
      bool ok = true;
      // Values that steer this loop come from memory; broadcasting them from lane 0 is what tells the
      // compiler they are warp-uniform, which keeps the descriptor arithmetic on the uniform datapath.
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
      // Gathered rows were written by plain asynchronous copies (generic proxy); the MMAs read through the async
      // proxy, so the issuing warp puts a proxy fence between its wait and its instructions.

      while (ok) {
        const int have = walk.Next(&seq, &t_lo, &t_hi, &seq_tiles, &seq_len) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, have, 0) == 0) break;
        const int n = __shfl_sync(0xffffffffu, t_hi - t_lo, 0);
        if (is_qk) {
          for (int i = 0; i < n && ok; ++i) {
            const int g = __shfl_sync(0xffffffffu, g0 + i, 0);
            const int stage = g % kStages;
            const int buf = g & 1;
            const uint32_t kv_parity = (g / kStages) & 1;
            ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->kv_full[stage][0]), kv_parity, misc, p.status, 24));
            if (ok && g >= 2) {
              ok = __all_sync(0xffffffffu,
                              BoundedWait(bar(&misc->s_empty[buf]), ((g >> 1) & 1) ^ 1, misc, p.status, 25));
            }
            // A segment's first tile also waits, group by group, for the sequence's Q.
            const bool first_of_segment = i == 0;
            if (ok && first_of_segment) {
              ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->q_full[0]), seg & 1, misc, p.status, 22));
            }
            if (!ok) break;
            ptx::TcFenceAfterSync();
            if constexpr (kGathered) ptx::FenceProxyAsyncShared();
            const uint64_t kdesc = DescAt(k_desc0, stage * kStageBytes);
            const uint32_t d = tmem_u + kTmemColS + kTile * buf;
            // Twelve k-steps per slab group, each group as soon as its slabs have landed (compile-time
            // offsets; a runtime offset costs the uniform-datapath issue rate).
            IssueQkGroup<0, 2>(q_desc, kdesc, d);
            ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->kv_full[stage][1]), kv_parity, misc, p.status, 26));
            if (ok && first_of_segment) {
              ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->q_full[1]), seg & 1, misc, p.status, 22));
            }
            if (!ok) break;
            ptx::TcFenceAfterSync();
            if constexpr (kGathered) ptx::FenceProxyAsyncShared();
            IssueQkGroup<2, 2>(q_desc, kdesc, d);
            ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->kv_full[stage][2]), kv_parity, misc, p.status, 27));
            if (ok && first_of_segment) {
              ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->q_full[2]), seg & 1, misc, p.status, 22));
            }
            if (!ok) break;
            ptx::TcFenceAfterSync();
            if constexpr (kGathered) ptx::FenceProxyAsyncShared();
            IssueQkGroup<4, 2>(q_desc, kdesc, d);
            ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->kv_full[stage][3]), kv_parity, misc, p.status, 28));
            if (ok && first_of_segment) {
              ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->q_full[3]), seg & 1, misc, p.status, 22));
            }
            if (!ok) break;
            ptx::TcFenceAfterSync();
            if constexpr (kGathered) ptx::FenceProxyAsyncShared();
            IssueQkGroup<6, 3>(q_desc, kdesc, d);
            if (ptx::ElectOne()) {
              ptx::TcCommit(bar(&misc->s_full[buf]));
              if (i == n - 1) ptx::TcCommit(bar(&misc->q_empty));  // Q buffer free for the next segment
            }
          }
        } else {
          if (seg > 0) {
            // The previous segment's accumulators must have been drained by the epilogue.
            ok = __all_sync(0xffffffffu, BoundedWait(bar(&misc->o_empty), (seg - 1) & 1, misc, p.status, 23));
          }
          for (int i = 0; i < n && ok; ++i) {
            const int g = __shfl_sync(0xffffffffu, g0 + i, 0);
            const int stage = g % kStages;
            ok = __all_sync(0xffffffffu,
                            BoundedWait(bar(&misc->p_full[stage]), (g / kStages) & 1, misc, p.status, 21));
            if (!ok) break;
            ptx::TcFenceAfterSync();
            if constexpr (kGathered) ptx::FenceProxyAsyncShared();
            const uint32_t stage_off = stage * kStageBytes;
            const uint64_t pdesc = DescAt(k_desc0, stage_off + 8 * kSlabBytes);  // K-major: row = head, 32 B per k-step
            const uint64_t vdesc = DescAt(v_desc0, stage_off);
            const int first_pv = __shfl_sync(0xffffffffu, i == 0 ? 1 : 0, 0);
#pragma unroll
            for (int tm = 0; tm < 4; ++tm) {  // accumulator by accumulator: slabs 2tm, 2tm + 1 are done with after it
#pragma unroll
              for (int ks = 0; ks < kTile / 16; ++ks) {
                const uint64_t a = DescAt(vdesc, 2 * tm * kSlabBytes + ks * 2048);
                const uint64_t b = DescAt(pdesc, ks * 32);
                const uint32_t acc = (first_pv != 0 && ks == 0) ? 0u : 1u;
                if (ptx::ElectOne()) ptx::MmaF16SS(tmem_u + 64 * tm, a, b, kIdescPv, acc);
              }
              if (ptx::ElectOne()) ptx::TcCommit(bar(&misc->kv_empty[stage][tm]));
            }
          }
          if (ok && ptx::ElectOne()) ptx::TcCommit(bar(&misc->o_full));
        }
        g0 += n;
        ++seg;
      }
      // Nothing of this warp's tensor work may be in flight when TMEM is freed.
      if (ptx::ElectOne()) {
        const uint32_t drain = bar(&misc->drain[is_qk ? 0 : 1]);
        ptx::TcCommit(drain);
        const uint64_t t0 = ptx::GlobalTimerNs();
        while (!ptx::MbarTryWait(drain, 0)) {
          if (ptx::GlobalTimerNs() - t0 > 200000000ull) break;
        }
      }
      __syncwarp();
    }
  } else {
    // ======================= softmax + epilogue warps ============================================
    const int tid = threadIdx.x;                 // 0..127
    const bool row_ok = lane < 16;               // M=64 accumulators use lanes 0..15 of each 32-lane quarter
    const int head = warp * 16 + (lane & 15);    // the row this lane writes (m, l) for in the epilogue
    // In the softmax a thread holds 16 scores of each of two rows: quad q = lane / 4 has rows q and q + 8 of
    // this warp's sixteen, thread lane % 4 of the quad the token pairs 8i + 2(lane % 4), i = 0..7.
    const int quad_row = lane >> 2;
    const int quad_col = (lane & 3) * 2;
    const int head0 = warp * 16 + quad_row;      // and head0 + 8
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    SegmentWalker walk(p.kv_len, p.batch, start_seq, start_tile, my_tiles);
    int seq, t_lo, t_hi, seq_tiles, seq_len;
    int g = 0;
    int seg = 0;
    bool ok = true;
    bool first_segment_of_cta = true;

    while (ok && walk.Next(&seq, &t_lo, &t_hi, &seq_tiles, &seq_len)) {
      float m_run[2] = {-INFINITY, -INFINITY};  // reference maxima of the two rows, log2 domain (s * scale * log2e)
      float l_run[2] = {0.0f, 0.0f};
      const int n = t_hi - t_lo;
      for (int i = 0; i < n && ok; ++i, ++g) {
        const int buf = g & 1;
        const int stage = g % kStages;
        const int tok0 = (t_lo + i) * kTile;
        const int valid = min(kTile, seq_len - tok0);
        ok = BoundedWait(bar(&misc->s_full[buf]), (g >> 1) & 1, misc, p.status, 30);
        if (!ok) break;
        ptx::TcFenceAfterSync();
        static_assert(kTile == 64, "one 16x256b.x8 load covers the 64 columns of a tile");
        uint32_t sr[32];
        ptx::TmemLd16x256bX8(tmem + lane_base + kTmemColS + kTile * buf, sr);
        ptx::TmemWaitLd();
        ptx::TcFenceBeforeSync();
        __syncwarp();
        if (lane == 0) ptx::MbarArrive(bar(&misc->s_empty[buf]));  // one arrival per warp

        // x[r][2k + e] = score of row head0 + 8r, token 8k + quad_col + e.
        float x[2][16];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          x[0][2 * k] = __uint_as_float(sr[4 * k]);
          x[0][2 * k + 1] = __uint_as_float(sr[4 * k + 1]);
          x[1][2 * k] = __uint_as_float(sr[4 * k + 2]);
          x[1][2 * k + 1] = __uint_as_float(sr[4 * k + 3]);
        }
        if (valid < kTile) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (8 * (j >> 1) + quad_col + (j & 1) >= valid) {  // masked out of the maximum and of P
              x[0][j] = -INFINITY;
              x[1][j] = -INFINITY;
            }
          }
        }
        // Raw maxima first (the scale is positive), then one FFMA + one EX2 per element.
        float raw_max[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {  // a tree, not a chain: one warp per scheduler pays every dependent latency
          float t[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = fmaxf(x[r][2 * j], x[r][2 * j + 1]);
          raw_max[r] = fmaxf(fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3])), fmaxf(fmaxf(t[4], t[5]), fmaxf(t[6], t[7])));
        }
        bool rescale = false;
        float neg_m[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          raw_max[r] = fmaxf(raw_max[r], __shfl_xor_sync(0xffffffffu, raw_max[r], 1));
          raw_max[r] = fmaxf(raw_max[r], __shfl_xor_sync(0xffffffffu, raw_max[r], 2));
          const float tile_max = raw_max[r] * p.scale_log2;
          // The reference maximum moves only when the tile's exceeds it by the threshold (always on a segment's
          // first tile, where m_run is -inf and nothing has been accumulated). No branch: a factor of
          // exp2(0) = 1 costs one more EX2, a divergent branch costs more.
          const bool moves = tile_max > m_run[r] + kRescaleThreshold;
          const float m_new = moves ? tile_max : m_run[r];
          const float factor = i == 0 ? 1.0f : ptx::Ex2Approx(m_run[r] - m_new);
          m_run[r] = m_new;
          rescale |= moves && i > 0;
          if ((lane & 3) == 0) misc->factor[head0 + 8 * r] = factor;
          l_run[r] *= factor;
          neg_m[r] = -m_run[r];
        }
        uint32_t packed[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float part[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float p0 = ptx::Ex2Approx(fmaf(x[r][2 * k], p.scale_log2, neg_m[r]));
            const float p1 = ptx::Ex2Approx(fmaf(x[r][2 * k + 1], p.scale_log2, neg_m[r]));
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            packed[r][k] = *reinterpret_cast<const uint32_t*>(&pb);
            part[k] = p0 + p1;  // the denominator (and lse) keep the unrounded fp32 weights
          }
          float sum = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          l_run[r] += sum;
        }

        const bool any_rescale = ptx::NamedBarrierOr(1, kSoftmaxThreads, rescale);
        if (any_rescale) {
          // Rare path: scale the accumulated O^T columns (heads) by their factors. PV of the previous
          // tile must have drained first; its commit is the arrival on that tile's kv_empty.
          const int gp = g - 1;
          ok = BoundedWait(bar(&misc->kv_empty[gp % kStages][kGroups - 1]), (gp / kStages) & 1, misc, p.status, 31);
          if (!ok) break;
          ptx::TcFenceAfterSync();
#pragma unroll 1
          for (int tm = 0; tm < 4; ++tm) {
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
              uint32_t o[32];
              const uint32_t addr = tmem + lane_base + 64 * tm + 32 * half;
              ptx::TmemLd32(addr, o);
              ptx::TmemWaitLd();
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * misc->factor[32 * half + j]);
              ptx::TmemSt32(addr, o);
            }
          }
          ptx::TmemWaitSt();
          ptx::TcFenceBeforeSync();
        }
        unsigned char* stage_ptr = smem + kOffKv + stage * kStageBytes;
        {
          // P over the stage's rope slab, which QK has finished with: row = head, 64 bf16 = 8 chunks of 16
          // bytes, chunks swizzled by the row index as the 128-byte pattern prescribes. This thread's pair of
          // tokens of chunk k is 4 bytes at quad_col * 2; a quad completes the chunk, and the eight quads of a
          // warp land in eight different chunk positions, so a store instruction touches each bank once.
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            // Row base (128-byte aligned) + quad_col * 2 < 16 leaves bits 4-6 free, so the swizzled chunk offset
            // (k ^ quad_row) << 4 is one XOR with a constant on a value prepared once.
            const uint32_t prow = ptx::SmemAddr(stage_ptr + 8 * kSlabBytes + (head0 + 8 * r) * 128 + quad_col * 2) ^
                                  static_cast<uint32_t>(quad_row << 4);
#pragma unroll
            for (int k = 0; k < 8; ++k) ptx::StShared32(prow ^ static_cast<uint32_t>(k << 4), packed[r][k]);
          }
        }
        if (valid < kTile) {
          // Rows past the sequence end hold whatever the pool held; zero them so 0 * NaN cannot reach O.
          const int rows = kTile - valid;
          for (int idx = tid; idx < rows * 8 * 8; idx += kSoftmaxThreads) {
            const int chunk = idx & 7;
            const int slab = (idx >> 3) & 7;
            const int r = valid + (idx >> 6);
            *reinterpret_cast<int4*>(stage_ptr + slab * kSlabBytes + r * 128 + chunk * 16) = make_int4(0, 0, 0, 0);
          }
        }
        ptx::FenceProxyAsyncShared();
        if (any_rescale) ptx::NamedBarrier(2, kSoftmaxThreads);  // factors are read before the next tile rewrites them
        __syncwarp();
        if (lane == 0) ptx::MbarArrive(bar(&misc->p_full[stage]));
      }
      if (!ok) break;

      // ---- epilogue of the segment ----
      ok = BoundedWait(bar(&misc->o_full), seg & 1, misc, p.status, 32);
      if (!ok) break;
      ptx::TcFenceAfterSync();
      const bool whole = (t_lo == 0 && t_hi == seq_tiles);
      const bool to_ws = !whole || p.force_ws != 0;
      const bool to_user_partial = !to_ws && p.user_o != nullptr;
      const int slot = cta * 2 + (first_segment_of_cta ? 0 : 1);
      // Lane j < 16 writes row j of this warp's sixteen: its (m, l) sit in quad j % 8, entry j / 8.
      const int from = 4 * (lane & 7);
      const float m_lo = __shfl_sync(0xffffffffu, m_run[0], from), m_hi = __shfl_sync(0xffffffffu, m_run[1], from);
      const float l_lo = __shfl_sync(0xffffffffu, l_run[0], from), l_hi = __shfl_sync(0xffffffffu, l_run[1], from);
      const float l_row = (lane & 8) ? l_hi : l_lo;
      const float m_nat = ((lane & 8) ? m_hi : m_lo) * 0.6931471805599453f;
      if (row_ok) {
        misc->inv_l[head] = l_row > 0.0f ? 1.0f / l_row : 0.0f;
        if (to_ws) {
          p.ws_m[slot * kHeads + head] = m_nat;
          p.ws_l[slot * kHeads + head] = l_row;
        } else if (to_user_partial) {
          p.user_m[static_cast<int64_t>(seq) * kHeads + head] = m_nat;
          p.user_l[static_cast<int64_t>(seq) * kHeads + head] = l_row;
        } else if (p.lse != nullptr) {
          p.lse[static_cast<int64_t>(seq) * kHeads + head] = m_nat + logf(l_row);
        }
      }
      ptx::NamedBarrier(1, kSoftmaxThreads);
      if (to_ws) {
        // The usual case (a sequence cut over several CTAs). Both halves of an accumulator are read before the
        // one wait; store j of a warp is the 512 contiguous bytes of head quad j, dv 32 w .. 32 w + 31.
        uint4* slot_base = reinterpret_cast<uint4*>(p.ws_o) + static_cast<int64_t>(slot) * (kLatent * kHeads / 4);
#pragma unroll 1
        for (int tm = 0; tm < 4; ++tm) {
          const int dv = 128 * tm + warp * 32 + lane;
          uint32_t lo[32], hi[32];
          ptx::TmemLd32(tmem + lane_base + 64 * tm, lo);
          ptx::TmemLd32(tmem + lane_base + 64 * tm + 32, hi);
          ptx::TmemWaitLd();
          uint4* dst = slot_base + dv;
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[j * kLatent] = make_uint4(lo[4 * j], lo[4 * j + 1], lo[4 * j + 2], lo[4 * j + 3]);
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[(8 + j) * kLatent] = make_uint4(hi[4 * j], hi[4 * j + 1], hi[4 * j + 2], hi[4 * j + 3]);
        }
      } else {
#pragma unroll 1
        for (int tm = 0; tm < 4; ++tm) {
          const int dv = 128 * tm + warp * 32 + lane;
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            uint32_t o[32];
            ptx::TmemLd32(tmem + lane_base + 64 * tm + 32 * half, o);
            ptx::TmemWaitLd();
            if (to_user_partial) {
              float* dst = p.user_o + (static_cast<int64_t>(seq) * kHeads + 32 * half) * kLatent + dv;
#pragma unroll
              for (int j = 0; j < 32; ++j) dst[j * kLatent] = __uint_as_float(o[j]);
            } else {
              __nv_bfloat16* dst = p.out + (static_cast<int64_t>(seq) * kHeads + 32 * half) * kLatent + dv;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                dst[j * kLatent] = __float2bfloat16_rn(__uint_as_float(o[j]) * misc->inv_l[32 * half + j]);
              }
            }
          }
        }
      }
      ptx::TcFenceBeforeSync();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(bar(&misc->o_empty));
      first_segment_of_cta = false;
      ++seg;
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------
  ptx::TcFenceBeforeSync();
  __syncthreads();
  if (warp == 5) {
    ptx::TcFenceAfterSync();
    ptx::TmemDealloc(tmem, kTmemCols);
  }
}

// Merges the partial segments of every sequence that straddles CTAs, and writes the result of empty
// sequences. A CTA takes one sequence, one quad of heads and a range of the 512 output columns; a thread owns
// one column (dv) of the four heads, as the decode kernel's epilogue left them: 16 bytes per part, a warp's
// loads 512 contiguous bytes, and its output stores runs of 32 consecutive values of a row.
//
// Where a sequence's parts lie follows from the lengths alone (the decode kernel's cut of the tile list,
// CostCut), so that arithmetic runs before the wait for the decode kernel. Then, per chunk of parts, the data
// loads of the chunk's first parts are issued, one warp per part group works out the weights of its eight parts
// for the quad's four heads (lane = part x head; the maxima and sums are shuffles) and leaves them in shared
// memory, and every thread accumulates weight x data.
// kGroups = 1: 128 threads, 256 columns per CTA in two passes, every thread walks all parts (batches, where a
// sequence has a handful of parts: 32 CTAs per sequence). kGroups = 8: 256 threads, 32 columns per CTA, a
// chunk is 256 parts of which each warp takes 32 consecutive ones, summed through shared memory at the end
// (a few long sequences with a hundred parts each: 256 CTAs per sequence, one chunk, one round of weights).
// The kernel needs a few hundred bytes of shared memory, so its CTAs fit beside a resident decode CTA.
//
// kPeer (with kGroups = 8): the sequence is a KV-range shard of a longer one that other GPUs hold the rest of.
// The CTA's merged columns are not written out but pushed, as tagged words, into every rank's exchange buffer
// over peer memory, and the same threads then wait (bounded) for the other ranks' words of their columns,
// merge them and write the final rows: the exchange protocol of kv_peer.cu without a kernel, and a pass over
// the partial, in between. A thread waits only for words that other GPUs' kernels write.
template <int kGroups, bool kPeer = false, bool kQuant = false>
__global__ void __launch_bounds__(kGroups == 1 ? 128 : 256, kGroups == 1 ? 7 : 2)
    MlaFinalizeKernel(TcParams p, int32_t n_ctas, PeerRing ring) {
  static_assert(!kPeer || kGroups == 8, "the peer form is built on the few-sequences variant");
  constexpr int kThreadsF = kGroups == 1 ? 128 : 256;
  constexpr int kGroupThreads = kThreadsF / kGroups;   // 128 or 32: columns a group covers per pass
  constexpr int kPasses = kGroups == 1 ? 2 : 1;
  constexpr int kDv = kGroupThreads * kPasses;         // 256 or 32 output columns per CTA
  constexpr int kGroupParts = kGroups == 1 ? 8 : 32;   // parts of a chunk that one group takes
  constexpr int kChunk = kGroupParts * kGroups;        // parts per chunk: 8, or 256 (a long sequence's in one go)
  constexpr int kRounds = kGroupParts / 8;             // a warp works out the weights of 8 parts x 4 heads at a time
  constexpr int kSub = kGroups == 1 ? 4 : 8;           // parts whose data a thread has in flight
  constexpr int kDvChunks = kLatent / kDv;             // 2 or 16
  constexpr int kQuads = kHeads / 4;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int b = blockIdx.x / (kQuads * kDvChunks);
  const int hq = (blockIdx.x / kDvChunks) % kQuads;    // heads 4 hq .. 4 hq + 3
  const int dv0 = (blockIdx.x % kDvChunks) * kDv;
  const int group = tid / kGroupThreads;
  const int tl = tid % kGroupThreads;

  __shared__ long long shared_meta[8];
  __shared__ int s_slot[kChunk];
  __shared__ __align__(16) float s_w[kChunk][4];
  __shared__ float s_gmax[kGroups][4], s_gsum[kGroups][4];
  __shared__ __align__(16) float s_carry[4];
  __shared__ float s_big[4], s_sum[4];
  __shared__ __align__(16) float4 s_red[kGroups > 1 ? kGroups * kGroupThreads : 1];

  if (tid < 32) {
    long long before = 0, total = 0, before_s = 0, nonempty = 0;
    for (int i = lane; i < p.batch; i += 32) {
      const long long t = TilesOf(p.kv_len[i]);
      total += t;
      nonempty += t > 0 ? 1 : 0;
      if (i < b) {
        before += t;
        before_s += t > 0 ? 1 : 0;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      total += __shfl_xor_sync(0xffffffffu, total, off);
      nonempty += __shfl_xor_sync(0xffffffffu, nonempty, off);
      before += __shfl_xor_sync(0xffffffffu, before, off);
      before_s += __shfl_xor_sync(0xffffffffu, before_s, off);
    }
    if (lane == 0) {
      const long long tiles = TilesOf(p.kv_len[b]);
      const CostCut c{CostCut::Total(total, nonempty), n_ctas};
      shared_meta[0] = total;
      shared_meta[1] = nonempty;
      shared_meta[2] = before;
      shared_meta[3] = before_s;
      shared_meta[4] = tiles;
      // c_prev is the CTA that took the tile before this sequence: if it is c_first, this sequence is not that
      // CTA's first segment and its part sits in the CTA's second slot.
      shared_meta[5] = tiles > 0 ? c.CtaOf(before, before_s) : 0;
      shared_meta[6] = tiles > 0 ? c.CtaOf(before + tiles - 1, before_s) : -1;
      shared_meta[7] = before > 0 && tiles > 0 ? c.CtaOf(before - 1, before_s - 1) : -1;
    }
    if (lane < 4) {
      s_big[lane] = -INFINITY;
      s_sum[lane] = 0.0f;
    }
  }
  __syncthreads();
  const long long total = shared_meta[0], nonempty = shared_meta[1], before = shared_meta[2], before_s = shared_meta[3];
  const long long mine = shared_meta[4];
  const int cf = static_cast<int>(shared_meta[5]), cl = static_cast<int>(shared_meta[6]), cp = static_cast<int>(shared_meta[7]);
  const bool want_partial = p.user_o != nullptr;
  // The output's MX quantisation (the reference's next stage, attn_quant: src/pipeline/pipeline.cpp:250-258) as
  // this kernel's epilogue: the 32 lanes of a warp hold 32 consecutive columns of one head's row, which is one
  // block; they agree on its maximum with shuffles and each writes its byte. The value quantised is the bf16
  // the kernel writes to `out`, so the bytes equal those of the stand-alone quantiser run on `out`. (kQuant: an
  // instantiation of its own; the kernel without it is unchanged.)
  auto write_quantised = [&](int64_t out_row, int dv, __nv_bfloat16 y) {  // every lane of the warp calls
    const float x = __bfloat162float(y);
    // One warp reduction over the bit images of |x|: they order like the values, and a NaN's image is above
    // infinity's, so the maximum also tells whether the block holds one.
    const uint32_t top = __reduce_max_sync(0xffffffffu, __float_as_uint(x) & 0x7fffffffu);
    const int nan = top > 0x7f800000u ? 1 : 0;
    const float amax = __uint_as_float(top);
    const MxScale block = MxScaleOf(amax, nan != 0);
    const uint32_t code = nan != 0 ? (((__float_as_uint(x) >> 24) & 0x80u) | 0x7fu)
                                   : static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(x, block.inv), __NV_SATFINITE, __NV_E4M3));
    p.out_q[out_row * kLatent + dv] = static_cast<uint8_t>(code);
    if (lane == 0) p.out_scale[out_row * (kLatent / 32) + dv / 32] = static_cast<uint8_t>(block.code);
  };
  const CostCut cut{CostCut::Total(total, nonempty), n_ctas};
  // Slot of CTA c's part of this sequence, or -1: the CTA holds a part if its first tile inside the sequence
  // lies before the next CTA's run. When every CTA's share of the cost is at least 5 units it holds at least
  // one tile (consecutive tiles are at most 5 units apart), so every CTA from the first to the last holds a
  // part and no division is needed.
  const bool dense = cut.cost_total >= (CostCut::kTileCost + CostCut::kCrossCost) * cut.n_ctas;
  auto slot_of = [&](int c) {
    if (c > cl) return -1;
    if (!dense) {
      const long long x = cut.FirstTileAt(cut.FirstPos(c), before, before_s);
      if (x >= before + mine || CostCut::Pos(x, before_s) >= cut.FirstPos(c + 1)) return -1;
    }
    return c * 2 + (c > cp ? 0 : 1);
  };
  // All of the above came from the lengths, which were stable before the decode kernel ran; the partials
  // below are what that kernel wrote, so they wait for its completion.
  GridDependencyTrigger();
  GridDependencyWait();
  if (!kPeer && mine > 0 && cf == cl) {  // written directly by the decode kernel
    if (kQuant && group == 0) {  // ... whose rows this CTA's columns are read back from and quantised
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int q = 0; q < kPasses; ++q) {
          const int64_t out_row = static_cast<int64_t>(b) * kHeads + 4 * hq + i;
          const int dv = dv0 + tl + kGroupThreads * q;
          write_quantised(out_row, dv, p.out[out_row * kLatent + dv]);
        }
      }
    }
    return;
  }

  float acc[kPasses][4];
#pragma unroll
  for (int q = 0; q < kPasses; ++q) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[q][i] = 0.0f;
  }
  // float4 index of this thread's column of the quad in pass q of slot s: (s * 16 + hq) * 512 + dv
  const float4* ws4 = reinterpret_cast<const float4*>(p.ws_o);
  const int dv_first = dv0 + tl;

  for (int c0 = cf; c0 <= cl && mine > 0; c0 += kChunk) {
    if (c0 != cf) __syncthreads();  // the previous chunk's weights and slots have been used
    if (tid < kChunk) s_slot[tid] = slot_of(c0 + tid);
    __syncthreads();
    // This thread's parts of the chunk: kGroupParts consecutive ones per group, kSub at a time.
    float4 data[kSub][kPasses];
    auto load_sub = [&](int sub) {
#pragma unroll
      for (int k = 0; k < kSub; ++k) {
        const int slot = s_slot[group * kGroupParts + sub * kSub + k];
#pragma unroll
        for (int q = 0; q < kPasses; ++q) {
          data[k][q] = slot >= 0 ? ws4[(static_cast<int64_t>(slot) * kQuads + hq) * kLatent + dv_first + kGroupThreads * q]
                                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
      }
    };
    load_sub(0);
    // ---- weights of the chunk: warp g of the first kGroups warps takes its group's parts, eight at a time,
    // lane = (part, head) ----
    float m_mine[kRounds], l_mine[kRounds];
    if (warp < kGroups) {
      float gmax = -INFINITY;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        const int slot = s_slot[warp * kGroupParts + 8 * r + (lane >> 2)];
        m_mine[r] = -INFINITY;
        l_mine[r] = 0.0f;
        if (slot >= 0) {
          l_mine[r] = p.ws_l[slot * kHeads + 4 * hq + (lane & 3)];
          m_mine[r] = p.ws_m[slot * kHeads + 4 * hq + (lane & 3)];
        }
      }
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        if (!(l_mine[r] > 0.0f)) m_mine[r] = -INFINITY;
        gmax = fmaxf(gmax, m_mine[r]);
      }
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, off));
      if (lane < 4) s_gmax[warp][lane] = gmax;
    }
    if constexpr (kGroups > 1) __syncthreads(); else __syncwarp();
    if (warp < kGroups) {
      const int i = lane & 3;
      const float old_big = s_big[i];
      float new_big = old_big;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) new_big = fmaxf(new_big, s_gmax[g][i]);
      float gsum = 0.0f;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        const float w = (l_mine[r] > 0.0f && new_big != -INFINITY) ? expf(m_mine[r] - new_big) : 0.0f;
        s_w[warp * kGroupParts + 8 * r + (lane >> 2)][i] = w;
        gsum = fmaf(l_mine[r], w, gsum);
      }
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, off);
      if (lane < 4) s_gsum[warp][lane] = gsum;
      if constexpr (kGroups > 1) {
        // every warp has read s_big before warp 0 replaces it
        asm volatile("bar.sync 1, %0;" ::"r"(kGroups * 32) : "memory");
      } else {
        __syncwarp();
      }
      if (warp == 0 && lane < 4) {
        // Rescale what earlier chunks accumulated (only sequences cut over more parts than a chunk holds).
        const float carry = (old_big == -INFINITY || new_big == -INFINITY) ? 0.0f : expf(old_big - new_big);
        float sum = s_sum[i] * carry;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) sum += s_gsum[g][i];
        s_sum[i] = sum;
        s_big[i] = new_big;
        s_carry[i] = carry;
      }
    }
    __syncthreads();
    // ---- data of the chunk ----
    if (c0 != cf) {
      const float4 cr = *reinterpret_cast<const float4*>(s_carry);
#pragma unroll
      for (int q = 0; q < kPasses; ++q) {
        acc[q][0] *= cr.x;
        acc[q][1] *= cr.y;
        acc[q][2] *= cr.z;
        acc[q][3] *= cr.w;
      }
    }
#pragma unroll 1
    for (int sub = 0; sub < kGroupParts / kSub; ++sub) {
      if (sub > 0) {
        if (s_slot[group * kGroupParts + sub * kSub] < 0 && dense) break;  // dense: parts are consecutive, the rest is absent
        load_sub(sub);
      }
#pragma unroll
      for (int k = 0; k < kSub; ++k) {
        // An absent part has weight zero and zero data; a present one with l = 0 may hold anything (0 x NaN is
        // not 0), so its data is dropped with its weight.
        const float4 w = *reinterpret_cast<const float4*>(s_w[group * kGroupParts + sub * kSub + k]);
#pragma unroll
        for (int q = 0; q < kPasses; ++q) {
          acc[q][0] = fmaf(w.x != 0.0f ? data[k][q].x : 0.0f, w.x, acc[q][0]);
          acc[q][1] = fmaf(w.y != 0.0f ? data[k][q].y : 0.0f, w.y, acc[q][1]);
          acc[q][2] = fmaf(w.z != 0.0f ? data[k][q].z : 0.0f, w.z, acc[q][2]);
          acc[q][3] = fmaf(w.w != 0.0f ? data[k][q].w : 0.0f, w.w, acc[q][3]);
        }
      }
    }
  }
  if constexpr (kGroups > 1) {
    s_red[group * kGroupThreads + tl] = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
    __syncthreads();
    if (group != 0) return;
#pragma unroll
    for (int g = 1; g < kGroups; ++g) {
      const float4 v = s_red[g * kGroupThreads + tl];
      acc[0][0] += v.x;
      acc[0][1] += v.y;
      acc[0][2] += v.z;
      acc[0][3] += v.w;
    }
  }
  if constexpr (kPeer) {
    // ---- across the GPUs: push this rank's merged columns, wait for the others', merge, write ----
    const int64_t row_first = static_cast<int64_t>(b) * kHeads + 4 * hq;
    const PeerLayout lay = PeerLayoutOf(ring.world, ring.rows);
    unsigned char* own = ring.peer[ring.rank];
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(own + lay.epoch_offset) + 1u;
    const uint64_t tag = static_cast<uint64_t>(epoch) << 32;
    const size_t half = (epoch & 1u) * lay.inbox_bytes;
    const bool owns_ml = dv0 == 0 && lane < 4;  // lane i of the first column range also carries (m, l) of head i
    for (int dst = 0; dst < ring.world; ++dst) {
      uint64_t* inbox = reinterpret_cast<uint64_t*>(ring.peer[dst] + half) +
                        (static_cast<size_t>(ring.rank) * ring.rows + row_first) * kPeerRowWords;
#pragma unroll
      for (int i = 0; i < 4; ++i) PeerStoreWord(inbox + i * kPeerRowWords + dv_first, tag | __float_as_uint(acc[0][i]));
      if (owns_ml) {
        PeerStoreWord(inbox + lane * kPeerRowWords + kLatent, tag | __float_as_uint(s_big[lane]));
        PeerStoreWord(inbox + lane * kPeerRowWords + kLatent + 1, tag | __float_as_uint(s_sum[lane]));
      }
    }
    const uint64_t* inbox = reinterpret_cast<const uint64_t*>(own + half);
    const uint64_t start = PeerTimerNs();
    float big[4], total_l[4], merged[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      big[i] = -INFINITY;
      total_l[i] = 0.0f;
      merged[i] = 0.0f;
    }
    bool ok = true;
    for (int src = 0; src < ring.world && ok; ++src) {
      const uint64_t* words = inbox + (static_cast<size_t>(src) * ring.rows + row_first) * kPeerRowWords;
      uint64_t w[12];
      for (uint32_t spins = 0;; ++spins) {
        bool here = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i] = PeerLoadWord(words + i * kPeerRowWords + dv_first);
          w[4 + i] = PeerLoadWord(words + i * kPeerRowWords + kLatent);
          w[8 + i] = PeerLoadWord(words + i * kPeerRowWords + kLatent + 1);
        }
#pragma unroll
        for (int i = 0; i < 12; ++i) here = here && (w[i] >> 32) == epoch;
        if (__all_sync(0xffffffffu, here)) break;
        if ((spins & 63u) == 63u && PeerTimerNs() - start > 1000000000ull) {
          if (lane == 0) RecordError(p.status, B200KV_DEV_TIMEOUT, 51, src, static_cast<int32_t>(epoch));
          ok = false;
          break;
        }
      }
      if (!ok) break;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float m = __uint_as_float(static_cast<uint32_t>(w[4 + i]));
        const float l = __uint_as_float(static_cast<uint32_t>(w[8 + i]));
        if (!(l > 0.0f)) continue;  // an empty shard
        const float new_big = fmaxf(big[i], m);
        const float carry = big[i] == -INFINITY ? 0.0f : expf(big[i] - new_big);
        const float weight = expf(m - new_big);
        big[i] = new_big;
        total_l[i] = total_l[i] * carry + l * weight;
        merged[i] = fmaf(merged[i], carry, __uint_as_float(static_cast<uint32_t>(w[i])) * weight);
      }
    }
    ok = __all_sync(0xffffffffu, ok);  // (one warp is left here; the quantiser below shuffles across all of it)
    if (ok) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float inv = total_l[i] > 0.0f ? 1.0f / total_l[i] : 0.0f;
        const __nv_bfloat16 y = __float2bfloat16_rn(merged[i] * inv);
        p.out[(row_first + i) * kLatent + dv_first] = y;
        if constexpr (kQuant) write_quantised(row_first + i, dv_first, y);
      }
      if (owns_ml && p.lse != nullptr) {
        float lse_value = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i == lane && total_l[i] > 0.0f) lse_value = big[i] + logf(total_l[i]);
        }
        p.lse[row_first + lane] = lse_value;
      }
    }
    // The epoch is complete for this rank when every CTA is done with the inbox half; a launch whose wait ran
    // out completes it too, so that the ranks that did arrive are not held up in the next one by this one.
    __syncwarp();
    if (lane == 0) {
      uint32_t* done = reinterpret_cast<uint32_t*>(own + lay.done_offset);
      __threadfence();
      if (atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0;
        *reinterpret_cast<volatile uint32_t*>(own + lay.epoch_offset) = epoch;
      }
    }
    return;
  }
  const int64_t row0 = static_cast<int64_t>(b) * kHeads + 4 * hq;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float sum = s_sum[i];
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
#pragma unroll
    for (int q = 0; q < kPasses; ++q) {
      const int64_t at = (row0 + i) * kLatent + dv_first + kGroupThreads * q;
      if (want_partial) {
        p.user_o[at] = acc[q][i];
      } else {
        const __nv_bfloat16 y = __float2bfloat16_rn(acc[q][i] * inv);
        p.out[at] = y;
        if constexpr (kQuant) write_quantised(row0 + i, dv_first + kGroupThreads * q, y);
      }
    }
  }
  if (dv0 == 0 && tid < 4) {
    const float sum = s_sum[tid];
    if (want_partial) {
      p.user_m[row0 + tid] = s_big[tid];
      p.user_l[row0 + tid] = sum;
    } else if (p.lse != nullptr) {
      p.lse[row0 + tid] = sum > 0.0f ? s_big[tid] + logf(sum) : -INFINITY;
    }
  }
}

// ---- tensor maps ----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn ResolveEncodeTiled() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  int64_t stride;
  int64_t rows;
  int32_t width;
  int32_t box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && stride == o.stride && rows == o.rows && width == o.width && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h ^= static_cast<size_t>(k.stride) * 0x9E3779B97F4A7C15ull;
    h ^= static_cast<size_t>(k.rows) * 0xC2B2AE3D27D4EB4Full;
    return h ^ static_cast<size_t>(k.width) ^ (static_cast<size_t>(k.box_rows) << 20);
  }
};

// Row-major [rows][width] bf16 view with row stride `stride` elements; box = 64 columns x box_rows rows (a tile
// of 64 consecutive rows, or a single row for the loads that gather four rows each), 128-byte swizzle. Maps are
// cached: a decode step reuses the same 2 x layers views every token.
int32_t GetRowMap(const void* base, int64_t stride, int64_t rows, int32_t width, int32_t box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, stride, rows, width, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return B200KV_OK;
    }
  }
  EncodeTiledFn encode = ResolveEncodeTiled();
  if (encode == nullptr) {
    SetLastError("cuTensorMapEncodeTiled could not be resolved from the CUDA driver");
    return B200KV_ERR_RUNTIME;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    SetLastError("cuTensorMapEncodeTiled failed with CUresult %d (base %p, stride %lld, rows %lld, width %d)",
                 static_cast<int>(rc), base, static_cast<long long>(stride), static_cast<long long>(rows), width);
    return B200KV_ERR_RUNTIME;
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
  }
  *out = map;
  return B200KV_OK;
}

// Query view [batch][64 heads][576] bf16 with element strides (q_seq_stride, q_head_stride, 1);
// box = 64 columns x 64 heads of one sequence, 128-byte swizzle.
struct QKey {
  const void* base;
  int64_t head_stride;
  int64_t seq_stride;  // the effective one: a batch of one has none of its own
  int32_t batch;
  bool operator==(const QKey& o) const {
    return base == o.base && head_stride == o.head_stride && seq_stride == o.seq_stride && batch == o.batch;
  }
};
struct QKeyHash {
  size_t operator()(const QKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h ^= static_cast<size_t>(k.head_stride) * 0x9E3779B97F4A7C15ull;
    h ^= static_cast<size_t>(k.seq_stride) * 0xC2B2AE3D27D4EB4Full;
    return h ^ (static_cast<size_t>(k.batch) * 0x165667B19E3779F9ull);
  }
};

int32_t GetQMap(const void* base, int64_t head_stride, int64_t seq_stride, int32_t batch, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<QKey, CUtensorMap, QKeyHash> cache;
  // A batch of one has no meaningful sequence stride; any multiple of 16 bytes that covers a sequence will do.
  const int64_t seq_stride_eff = batch > 1 ? seq_stride : static_cast<int64_t>(kHeads) * head_stride;
  const QKey key{base, head_stride, seq_stride_eff, batch};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return B200KV_OK;
    }
  }
  EncodeTiledFn encode = ResolveEncodeTiled();
  if (encode == nullptr) {
    SetLastError("cuTensorMapEncodeTiled could not be resolved from the CUDA driver");
    return B200KV_ERR_RUNTIME;
  }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kLatent + kRope), kHeads, static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_stride) * 2, static_cast<cuuint64_t>(seq_stride_eff) * 2};
  const cuuint32_t box[3] = {64, kHeads, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUtensorMap map;
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    SetLastError("cuTensorMapEncodeTiled (query) failed with CUresult %d (base %p, strides %lld/%lld, batch %d)",
                 static_cast<int>(rc), base, static_cast<long long>(head_stride), static_cast<long long>(seq_stride),
                 batch);
    return B200KV_ERR_RUNTIME;
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
  }
  *out = map;
  return B200KV_OK;
}

}  // namespace

// Row-major [rows][128] one-byte view (FP8 vectors of 128) with a row stride of `stride_bytes`; box = the whole
// 128-byte row x box_rows rows, 128-byte swizzle. For the indexer's tensor-core kernel; encoded per call.
int32_t EncodeByteRowMap(const void* base, int64_t stride_bytes, int64_t rows, int32_t box_rows, CUtensorMap* out) {
  EncodeTiledFn encode = ResolveEncodeTiled();
  if (encode == nullptr) {
    SetLastError("cuTensorMapEncodeTiled could not be resolved from the CUDA driver");
    return B200KV_ERR_RUNTIME;
  }
  const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride_bytes)};
  const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    SetLastError("cuTensorMapEncodeTiled (byte rows) failed with CUresult %d (base %p, stride %lld, rows %lld)",
                 static_cast<int>(rc), base, static_cast<long long>(stride_bytes), static_cast<long long>(rows));
    return B200KV_ERR_RUNTIME;
  }
  return B200KV_OK;
}

// Row-major [rows][width] bf16 view, row stride `stride_bytes`; box = box_cols x box_rows, no swizzle (the box
// lands in shared memory as plain rows of box_cols elements). For kernels that only move rows.
int32_t EncodePlainBf16Map(const void* base, int64_t stride_bytes, int64_t rows, int32_t width, int32_t box_cols,
                           int32_t box_rows, CUtensorMap* out) {
  EncodeTiledFn encode = ResolveEncodeTiled();
  if (encode == nullptr) {
    SetLastError("cuTensorMapEncodeTiled could not be resolved from the CUDA driver");
    return B200KV_ERR_RUNTIME;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    SetLastError("cuTensorMapEncodeTiled (plain rows) failed with CUresult %d (base %p, stride %lld, rows %lld, box %d x %d)",
                 static_cast<int>(rc), base, static_cast<long long>(stride_bytes), static_cast<long long>(rows), box_cols, box_rows);
    return B200KV_ERR_RUNTIME;
  }
  return B200KV_OK;
}

size_t TcWorkspaceBytes(int32_t n_ctas) {
  return static_cast<size_t>(n_ctas) * 2 * kHeads * (kLatent + 2) * sizeof(float);
}

bool TcSupports(const b200kv_decode_args& a) {
  if (a.row_index != nullptr && (a.kv_begin != nullptr || a.new_latent != nullptr || a.row_index_stride < 1)) return false;
  return a.heads == kHeads && (a.row_index != nullptr || a.block_size % kTile == 0) && a.q_head_stride % 8 == 0 &&
         a.q_seq_stride % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 && a.pool.pool_rows <= INT32_MAX &&
         a.pool.latent_row_stride * 2 < (1ll << 40);
}

bool TcPeerSupports(const b200kv_decode_args& a) { return a.batch < 16; }

// ring != nullptr: the call's sequences are KV-range shards and the merge kernel finishes them across the GPUs
// (TcPeerSupports says for which batches that form exists).
int32_t LaunchMlaDecodeTc(const b200kv_decode_args& a, int32_t n_ctas, cudaStream_t stream, int32_t* status,
                          const PeerRing* ring) {
  if (a.new_latent != nullptr || a.new_rope != nullptr) {
    if (a.new_latent == nullptr || a.new_rope == nullptr) {
      SetLastError("decode: a fused append needs both new_latent and new_rope");
      return B200KV_ERR_NULLPTR;
    }
    if (a.kv_begin != nullptr || a.new_latent_stride < kLatent || a.new_latent_stride % 8 != 0 ||
        a.new_rope_stride < kRope || a.new_rope_stride % 8 != 0 ||
        ((reinterpret_cast<uintptr_t>(a.new_latent) | reinterpret_cast<uintptr_t>(a.new_rope)) & 15u) != 0) {
      SetLastError("decode: the fused append works without kv_begin, from 16-byte aligned rows whose strides are "
                   "multiples of 8 elements (strides %lld / %lld)",
                   static_cast<long long>(a.new_latent_stride), static_cast<long long>(a.new_rope_stride));
      return B200KV_ERR_INVALID;
    }
  }
  static thread_local int configured_device = -1;
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device != configured_device) {
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(MlaDecodeTcKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    kSmemBytes),
                               "tcgen05 decode smem opt-in")) {
      return rc;
    }
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(MlaDecodeTcKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    kSmemBytes),
                               "tcgen05 decode (gathered rows) smem opt-in")) {
      return rc;
    }
    configured_device = device;
  }
  CUtensorMap latent_map, rope_map;
  const int32_t box_rows = kTile;
  if (int32_t rc = GetRowMap(a.pool.latent, a.pool.latent_row_stride, a.pool.pool_rows, kLatent, box_rows, &latent_map)) return rc;
  if (int32_t rc = GetRowMap(a.pool.rope, a.pool.rope_row_stride, a.pool.pool_rows, kRope, box_rows, &rope_map)) return rc;

  CUtensorMap q_map;
  if (int32_t rc = GetQMap(a.q, a.q_head_stride, a.q_seq_stride, a.batch, &q_map)) return rc;

  TcParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.q_seq_stride = a.q_seq_stride;
  p.q_head_stride = a.q_head_stride;
  p.block_table = a.block_table;
  p.max_blocks = a.max_blocks;
  p.kv_len = a.kv_len;
  p.kv_begin = a.kv_begin;
  p.pool_rows = a.pool.pool_rows;
  p.stable_tables = (a.flags & B200KV_DECODE_STABLE_TABLES) != 0 ? 1 : 0;
  p.force_ws = ring != nullptr ? 1 : 0;
  p.row_index = a.row_index;
  p.row_index_stride = a.row_index_stride;
  p.new_latent = static_cast<const char*>(a.new_latent);
  p.new_rope = static_cast<const char*>(a.new_rope);
  p.new_latent_bytes = a.new_latent_stride * 2;
  p.new_rope_bytes = a.new_rope_stride * 2;
  p.pool_latent = static_cast<char*>(a.pool.latent);
  p.pool_rope = static_cast<char*>(a.pool.rope);
  p.pool_latent_bytes = a.pool.latent_row_stride * 2;
  p.pool_rope_bytes = a.pool.rope_row_stride * 2;
  p.batch = a.batch;
  p.block_size = a.block_size;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.out_q = static_cast<uint8_t*>(a.out_fp8);
  p.out_scale = static_cast<uint8_t*>(a.out_scale);
  p.lse = a.lse;
  p.user_o = a.partial_o;
  p.user_m = a.partial_m;
  p.user_l = a.partial_l;
  float* ws = static_cast<float*>(a.workspace);
  const size_t slots = static_cast<size_t>(n_ctas) * 2;
  p.ws_o = ws;
  p.n_slots = static_cast<int32_t>(slots);
  p.ws_m = ws + slots * kHeads * kLatent;
  p.ws_l = p.ws_m + slots * kHeads;
  p.status = status;

  if (int32_t rc = CheckCuda(a.row_index != nullptr
                                 ? LaunchOverlapped(MlaDecodeTcKernel<true>, dim3(n_ctas), dim3(kThreads), kSmemBytes,
                                                    stream, latent_map, rope_map, q_map, p)
                                 : LaunchOverlapped(MlaDecodeTcKernel<false>, dim3(n_ctas), dim3(kThreads), kSmemBytes,
                                                    stream, latent_map, rope_map, q_map, p),
                             "tcgen05 decode launch")) {
    return rc;
  }
  // One or two long sequences: 256 CTAs per sequence, the parts shared out among a CTA's eight warps, so that
  // the merge still fills the GPU. Batches: 32 CTAs per sequence, every thread walking the sequence's parts.
  const bool quant = p.out_q != nullptr;
  const dim3 grid_few(static_cast<unsigned>(a.batch) * 16 * (kLatent / 32)), grid_many(static_cast<unsigned>(a.batch) * 16 * (kLatent / 256));
  cudaError_t launched;
  const char* what = "decode finalize launch";
  // (The 256-CTA form runs two CTAs per SM: one sequence is one wave, two are two, and from three on the
  // 32-CTA form, whose threads walk a sequence's parts eight at a time, is the shorter one. The exchange across
  // GPUs exists in the 256-CTA form only.)
  if (a.batch < 3 || ring != nullptr) {
    if (ring != nullptr) {
      what = "decode finalize + peer merge launch";
      launched = quant ? LaunchOverlapped(MlaFinalizeKernel<8, true, true>, grid_few, dim3(256), 0, stream, p, n_ctas, *ring)
                       : LaunchOverlapped(MlaFinalizeKernel<8, true, false>, grid_few, dim3(256), 0, stream, p, n_ctas, *ring);
    } else {
      launched = quant ? LaunchOverlapped(MlaFinalizeKernel<8, false, true>, grid_few, dim3(256), 0, stream, p, n_ctas, PeerRing{})
                       : LaunchOverlapped(MlaFinalizeKernel<8, false, false>, grid_few, dim3(256), 0, stream, p, n_ctas, PeerRing{});
    }
  } else {
    launched = quant ? LaunchOverlapped(MlaFinalizeKernel<1, false, true>, grid_many, dim3(128), 0, stream, p, n_ctas, PeerRing{})
                     : LaunchOverlapped(MlaFinalizeKernel<1, false, false>, grid_many, dim3(128), 0, stream, p, n_ctas, PeerRing{});
  }
  return CheckCuda(launched, what);
}

}  // namespace b200kv
