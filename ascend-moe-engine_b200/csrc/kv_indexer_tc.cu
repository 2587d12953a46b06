// The indexer's score stage on the tensor cores: for every token t of a sequence's paged index-key cache,
//   score_t = sum_h w_h * ReLU(qs_h * ks_t * (Q_h . K_t)),   Q_h, K_t FP8 E4M3 vectors of 128
// (aclnnQuantLightningIndexer: contract mock/mock_ops.cpp:1118-1221; key addressing
// third_party/ops_transformer/attention/quant_lightning_indexer/op_kernel/arch35/quant_lightning_indexer_service_cube.h:243-268).
//
// The contraction is one tcgen05.mma kind::f8f6f4 shape: a tile of 128 tokens (M) against the sequence's 64 heads
// (N) over the 128 dimensions (K, four instructions of K = 32), both operands K-major in shared memory behind
// 128-byte-swizzled TMA loads (a token's key is exactly one 128-byte row), the 128 x 64 fp32 dot products in
// TMEM. A thread of the epilogue owns one token (a TMEM lane), reads its 64 dot products and runs the same
// chain over the heads as the CUDA-core kernel: scale, ReLU, weight, sum. Per token the kernel moves 128 bytes
// of key, 4 of key scale and 4 of score: it is bound by HBM, and the tensor cores make the arithmetic free.
//
// Persistent CTAs (one per SM) each take an equal run of the flat list of token tiles. Ten warps: two epilogue
// groups of four (warps 0-3 take the CTA's even tiles and accumulator 0, warps 4-7 the odd ones and accumulator
// 1; warp w reads TMEM lanes 32 (w % 4) ..), warp 8 the TMA producer, warp 9 TMEM allocation and MMA issue. Four
// stages of {keys 16 KB, Q 8 KB}; Q comes with every tile (it is 8 KB per sequence and lives in L2), which
// spares the pipeline a special case where a CTA's run crosses into the next sequence. The epilogue is the
// longest stage of a tile (some 1,300 cycles of dependent fp32 work per thread against 700 for a tile's loads), so
// two groups alternate; what a role needs from memory for a tile (block-table entries, scales) it fetches one
// tile ahead.
//
// The tensor core's sum of 128 exact FP8 products is rounded differently from a chain of fp32 fmas, so scores
// agree with the CUDA-core kernel to a few units in the last place of the largest partial sum, not bit for
// bit; callers that need the reproducible selection ask for the exact variant.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200kv {

int32_t EncodeByteRowMap(const void* base, int64_t stride_bytes, int64_t rows, int32_t box_rows, CUtensorMap* out);

namespace {

constexpr int kDim = 128;          // bytes (and FP8 elements) per key / query vector
constexpr int kTokens = 128;       // tokens per tile = M
constexpr int kHeadsPadded = 64;   // N
constexpr int kHalf = 64;          // rows per key load: a block of 64 tokens is contiguous in the pool
constexpr int kStages = 4;
constexpr int kKeyBytes = kTokens * kDim;       // 16 KB
constexpr int kQBytes = kHeadsPadded * kDim;    // 8 KB
constexpr int kStageBytes = kKeyBytes + kQBytes;
constexpr int kThreads = 320;
constexpr int kEpilogueThreads = 128;  // per group
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kTmemCols = 128;     // two accumulators of 64 columns
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment */ + 2048 /* barriers, scalars, coefficients */;

struct TcScoreParams {
  const float* q_scale;    // [B][heads]
  const __nv_bfloat16* w;  // [B][heads]
  int32_t heads;
  const float* k_scale;  // [rows]
  int64_t pool_rows;
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  int32_t batch;
  int32_t block_size;
  float* scores;  // [B][score_stride]
  int64_t score_stride;
  int32_t* status;
};

struct Shared {  // at most 2048 bytes
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int32_t abort_flag;
  int32_t start_seq, start_tile, n_tiles;
  alignas(16) float qs[2][kHeadsPadded];
  alignas(16) float w[2][kHeadsPadded];
};

static_assert(sizeof(Shared) <= 2048, "the tail of the shared-memory budget");

__device__ __forceinline__ int TilesOf(int len) { return len > 0 ? (len + kTokens - 1) / kTokens : 0; }

__device__ __forceinline__ bool Aborting(const Shared* sh) {
  return *reinterpret_cast<const volatile int32_t*>(&sh->abort_flag) != 0;
}

// Bounded mbarrier wait: false when the CTA is aborting or after about a second, with the place recorded.
__device__ __noinline__ bool Wait(uint32_t bar, uint32_t parity, Shared* sh, int32_t* status, int site) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    if (ptx::MbarTryWait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (Aborting(sh)) return false;
      const uint64_t now = ptx::GlobalTimerNs();
      if (start == 0) start = now;
      if (now - start > 1000000000ull) {
        *reinterpret_cast<volatile int32_t*>(&sh->abort_flag) = 1;
        RecordError(status, B200KV_DEV_TIMEOUT, 100 + site, static_cast<int32_t>(blockIdx.x), static_cast<int32_t>(parity));
        return false;
      }
    }
  }
}

// The CTA's run of the flat tile list, one (sequence, tile) at a time; every role walks it the same way.
struct TileWalker {
  const int32_t* kv_len;
  int batch, seq, tile, remaining;
  __device__ TileWalker(const int32_t* lens, int batch_, int seq_, int tile_, int n)
      : kv_len(lens), batch(batch_), seq(seq_), tile(tile_), remaining(n) {}
  __device__ bool Next(int* seq_out, int* tile_out, int* len_out) {
    while (remaining > 0 && seq < batch) {
      const int len = kv_len[seq];
      if (tile < TilesOf(len)) {
        *seq_out = seq;
        *tile_out = tile;
        *len_out = len;
        ++tile;
        --remaining;
        return true;
      }
      tile = 0;
      ++seq;
    }
    return false;
  }
};

// Instruction descriptor for kind::f8f6f4, E4M3 x E4M3 -> fp32, both operands K-major:
//   bits [4,6) D format (1 = f32); [7,10) A format (0 = E4M3); [10,13) B format (0 = E4M3);
//   bits [17,23) N >> 3; bits [24,29) M >> 4.
constexpr uint32_t kIdesc = (1u << 4) | (static_cast<uint32_t>(kHeadsPadded >> 3) << 17) |
                            (static_cast<uint32_t>(kTokens >> 4) << 24);

__device__ __forceinline__ void MmaF8SS(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
    IndexerScoreTcKernel(const __grid_constant__ CUtensorMap key_map, const __grid_constant__ CUtensorMap q_map, TcScoreParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = ptx::SmemAddr(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;  // swizzled tiles want 1024-byte alignment
  Shared* sh = reinterpret_cast<Shared*>(smem_raw + (stage0 - raw) + kStages * kStageBytes);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto bar = [&](const uint64_t* b) { return ptx::SmemAddr(b); };

  GridDependencyTrigger();
  if (warp == kProducerWarp) {
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) {
        ptx::MbarInit(bar(&sh->full[s]), 1);
        ptx::MbarInit(bar(&sh->empty[s]), 1);
      }
      for (int s = 0; s < 2; ++s) {
        ptx::MbarInit(bar(&sh->acc_full[s]), 1);
        ptx::MbarInit(bar(&sh->acc_empty[s]), kEpilogueThreads / 32);
      }
      sh->abort_flag = 0;
      ptx::FenceBarrierInit();
      ptx::PrefetchTensorMap(&key_map);
      ptx::PrefetchTensorMap(&q_map);
    }
    __syncwarp();
    GridDependencyWait();
    // This CTA's run [lo, hi) of the flat tile list: totals, then the sequence and tile at which lo falls (a scan
    // over the sequences, 32 at a time).
    long long total = 0;
    for (int i = lane; i < p.batch; i += 32) total += TilesOf(p.kv_len[i]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    const long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    long long before = 0, found_before = 0;
    int found_seq = p.batch;
    for (int c = 0; c < p.batch && found_seq == p.batch; c += 32) {
      const int t = c + lane < p.batch ? TilesOf(p.kv_len[c + lane]) : 0;
      int incl = t;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, before + incl > lo);
      if (hit != 0u) {
        const int src = __ffs(hit) - 1;
        found_seq = c + src;
        found_before = before + __shfl_sync(0xffffffffu, incl - t, src);
      }
      before += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      sh->start_seq = found_seq;
      sh->start_tile = static_cast<int32_t>(lo - found_before);
      sh->n_tiles = static_cast<int32_t>(hi - lo);
    }
    __syncwarp();
  }
  if (warp == kMmaWarp) {
    ptx::TmemAlloc(ptx::SmemAddr(&sh->tmem_base), kTmemCols);
    ptx::TmemRelinquish();
  }
  GridDependencyWait();
  ptx::TcFenceBeforeSync();
  __syncthreads();
  ptx::TcFenceAfterSync();
  const uint32_t tmem = sh->tmem_base;
  const int start_seq = sh->start_seq, start_tile = sh->start_tile, n_tiles = sh->n_tiles;

  if (warp == kProducerWarp) {
    // ---- producer: lane 0 brings Q, lanes 1 and 2 a half tile of keys each (its pool row looked up a tile ahead) ----
    TileWalker walk(p.kv_len, p.batch, start_seq, start_tile, n_tiles);
    struct Ahead {
      int seq, tile, len;
      int64_t row;
    };
    auto look = [&](Ahead* a) -> bool {
      if (!walk.Next(&a->seq, &a->tile, &a->len)) return false;
      a->row = 0;  // a half beyond the sequence's end still fills its stage: row 0, masked by the epilogue
      if (lane == 1 || lane == 2) {
        const int tok = a->tile * kTokens + (lane - 1) * kHalf;
        if (tok < a->len) {
          const int64_t column = tok / p.block_size;
          const int64_t block = column < p.max_blocks ? p.block_table[static_cast<int64_t>(a->seq) * p.max_blocks + column] : -1;
          a->row = block * p.block_size + tok % p.block_size;
          if (block < 0 || a->row + kHalf > p.pool_rows) {
            RecordError(p.status, B200KV_DEV_BAD_BLOCK, a->seq, static_cast<int32_t>(column), static_cast<int32_t>(block));
            a->row = 0;
          }
        }
      }
      return true;
    };
    Ahead cur, next;
    bool have = look(&next);
    bool ok = true;
    int issued = 0;
    for (int i = 0; ok && have; ++i) {
      const int stage = i % kStages;
      cur = next;
      have = look(&next);
      if (i >= kStages) ok = __all_sync(0xffffffffu, Wait(bar(&sh->empty[stage]), ((i / kStages) & 1) ^ 1, sh, p.status, 0));
      if (!ok) break;
      const uint32_t dst = stage0 + stage * kStageBytes;
      const uint32_t full = bar(&sh->full[stage]);
      if (lane == 0) {
        ptx::MbarArriveExpectTx(full, kStageBytes);
        ptx::TmaLoad2D(dst + kKeyBytes, &q_map, 0, cur.seq * p.heads, full);
      } else if (lane < 3) {
        ptx::TmaLoad2D(dst + (lane - 1) * (kHalf * kDim), &key_map, 0, static_cast<int32_t>(cur.row), full);
      }
      issued = i + 1;
    }
    if (!ok && lane == 0) {
      // Aborting: the loads already issued land before the CTA gives its shared memory back.
      for (int i = max(0, issued - kStages); i < issued; ++i) {
        const uint64_t t0 = ptx::GlobalTimerNs();
        while (!ptx::MbarTryWait(bar(&sh->full[i % kStages]), (i / kStages) & 1)) {
          if (ptx::GlobalTimerNs() - t0 > 200000000ull) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ---- MMA issue: four K = 32 steps per tile into accumulator i % 2 ----
    const uint64_t key_desc0 = ptx::SmemDescSw128(stage0, 16, 1024);
    const uint64_t q_desc0 = ptx::SmemDescSw128(stage0 + kKeyBytes, 16, 1024);
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int stage = i % kStages, buf = i & 1;
      ok = __all_sync(0xffffffffu, Wait(bar(&sh->full[stage]), (i / kStages) & 1, sh, p.status, 1));
      if (ok && i >= 2) ok = __all_sync(0xffffffffu, Wait(bar(&sh->acc_empty[buf]), ((i >> 1) & 1) ^ 1, sh, p.status, 2));
      if (!ok) break;
      ptx::TcFenceAfterSync();
      const uint32_t off = static_cast<uint32_t>(stage * kStageBytes) >> 4;
      if (ptx::ElectOne()) {
#pragma unroll
        for (int k = 0; k < kDim / 32; ++k) {
          MmaF8SS(tmem + buf * kHeadsPadded, key_desc0 + off + 2 * k, q_desc0 + off + 2 * k, kIdesc, k > 0 ? 1u : 0u);
        }
        ptx::TcCommit(bar(&sh->empty[stage]));
        ptx::TcCommit(bar(&sh->acc_full[buf]));
      }
      __syncwarp();
    }
  } else {
    // ---- epilogue: thread = token; group g = warp / 4 takes tiles g, g + 2, ... of the CTA's run ----
    // What a tile needs from memory besides its accumulator (the sequence's per-head coefficients, one per
    // thread of the first 64, and this token's key scale behind a block-table lookup) is fetched one of the
    // group's tiles ahead: two dependent loads would otherwise stand between every two tiles.
    const int group = warp >> 2;
    const int gtid = tid & (kEpilogueThreads - 1);
    TileWalker walk(p.kv_len, p.batch, start_seq, start_tile, n_tiles);
    {
      int s0, t0, l0;
      if (group == 1) walk.Next(&s0, &t0, &l0);  // the odd group starts at the run's second tile
    }
    struct Fetched {
      int seq, tile, len;
      float qs, w, ks;
      bool valid;
    };
    auto fetch = [&](Fetched* f) -> bool {
      if (!walk.Next(&f->seq, &f->tile, &f->len)) return false;
      {
        int s1, t1, l1;
        walk.Next(&s1, &t1, &l1);  // the other group's tile
      }
      f->qs = 0.0f;
      f->w = 0.0f;
      if (gtid < p.heads) {
        f->qs = p.q_scale[f->seq * p.heads + gtid];
        f->w = __bfloat162float(p.w[f->seq * p.heads + gtid]);
      }
      const int tok = f->tile * kTokens + gtid;
      f->ks = 0.0f;
      f->valid = tok < f->len;
      if (f->valid) {
        const int64_t column = tok / p.block_size;
        const int64_t block = column < p.max_blocks ? p.block_table[static_cast<int64_t>(f->seq) * p.max_blocks + column] : -1;
        const int64_t row = block * p.block_size + tok % p.block_size;
        if (block < 0 || row >= p.pool_rows) {
          f->valid = false;  // recorded by the producer; the score below says that the token does not count
        } else {
          f->ks = p.k_scale[row];
        }
      }
      return true;
    };
    Fetched cur, next;
    bool have = fetch(&next);
    bool ok = true;
    const int buf = group;
    for (int n = 0; ok && have; ++n) {  // the group's n-th tile is the run's tile 2 n + group
      cur = next;
      have = fetch(&next);
      if (gtid < kHeadsPadded) {
        sh->qs[buf][gtid] = cur.qs;
        sh->w[buf][gtid] = cur.w;
      }
      ptx::NamedBarrier(1 + group, kEpilogueThreads);
      ok = __all_sync(0xffffffffu, Wait(bar(&sh->acc_full[buf]), n & 1, sh, p.status, 3));
      if (!ok) break;
      ptx::TcFenceAfterSync();
      uint32_t lo[32], hi[32];
      const uint32_t taddr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + buf * kHeadsPadded;
      ptx::TmemLd32(taddr, lo);
      ptx::TmemLd32(taddr + 32, hi);
      ptx::TmemWaitLd();
      ptx::TcFenceBeforeSync();
      __syncwarp();
      if (lane == 0) ptx::MbarArrive(bar(&sh->acc_empty[buf]));
      float score = 0.0f;
      const float4* qs4 = reinterpret_cast<const float4*>(sh->qs[buf]);
      const float4* w4 = reinterpret_cast<const float4*>(sh->w[buf]);
      // A head beyond the sequence's count is skipped, not multiplied by a zero weight: its column of the
      // accumulator came from rows of Q that belong to the next sequence (or from nothing) and may hold anything.
      auto head = [&](int h, float qs_h, float w_h, uint32_t dot) {
        if (h < p.heads) {
          const float scaled = __fmul_rn(__fmul_rn(qs_h, cur.ks), __uint_as_float(dot));
          score = __fmaf_rn(w_h, scaled > 0.0f ? scaled : 0.0f, score);
        }
      };
#pragma unroll
      for (int h4 = 0; h4 < 8; ++h4) {
        const float4 a = qs4[h4], c = w4[h4];
        head(4 * h4, a.x, c.x, lo[4 * h4]);
        head(4 * h4 + 1, a.y, c.y, lo[4 * h4 + 1]);
        head(4 * h4 + 2, a.z, c.z, lo[4 * h4 + 2]);
        head(4 * h4 + 3, a.w, c.w, lo[4 * h4 + 3]);
      }
#pragma unroll
      for (int h4 = 0; h4 < 8; ++h4) {
        const float4 a = qs4[8 + h4], c = w4[8 + h4];
        head(32 + 4 * h4, a.x, c.x, hi[4 * h4]);
        head(32 + 4 * h4 + 1, a.y, c.y, hi[4 * h4 + 1]);
        head(32 + 4 * h4 + 2, a.z, c.z, hi[4 * h4 + 2]);
        head(32 + 4 * h4 + 3, a.w, c.w, hi[4 * h4 + 3]);
      }
      const int tok = cur.tile * kTokens + gtid;
      if (tok < cur.len) p.scores[cur.seq * p.score_stride + tok] = cur.valid ? score : -INFINITY;
    }
  }

  ptx::TcFenceBeforeSync();
  __syncthreads();
  if (warp == kMmaWarp) {
    ptx::TcFenceAfterSync();
    ptx::TmemDealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool IndexerTcSupports(int32_t heads, int32_t block_size, int64_t key_stride, int64_t pool_rows) {
  return heads >= 1 && heads <= kHeadsPadded && block_size % kHalf == 0 && key_stride % 16 == 0 && pool_rows <= INT32_MAX;
}

int32_t LaunchIndexerScoreTc(const void* q, const float* q_scale, const void* weights, int32_t heads, const void* key_pool,
                             int64_t key_stride, const float* k_scale, int64_t pool_rows, const int32_t* block_table,
                             int64_t max_blocks, const int32_t* kv_len, int32_t batch, int32_t block_size, int64_t max_kv_len,
                             float* scores, int64_t score_stride, cudaStream_t stream, int32_t* status) {
  CUtensorMap key_map, q_map;
  if (int32_t rc = EncodeByteRowMap(key_pool, key_stride, pool_rows, kHalf, &key_map)) return rc;
  if (int32_t rc = EncodeByteRowMap(q, kDim, static_cast<int64_t>(batch) * heads, kHeadsPadded, &q_map)) return rc;
  static thread_local int configured_device = -1;
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device != configured_device) {
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(IndexerScoreTcKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                               "indexer tensor-core score smem opt-in")) {
      return rc;
    }
    configured_device = device;
  }
  TcScoreParams p{};
  p.q_scale = q_scale;
  p.w = static_cast<const __nv_bfloat16*>(weights);
  p.heads = heads;
  p.k_scale = k_scale;
  p.pool_rows = pool_rows;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.kv_len = kv_len;
  p.batch = batch;
  p.block_size = block_size;
  p.scores = scores;
  p.score_stride = score_stride;
  p.status = status;
  const long long most_tiles = static_cast<long long>(batch) * ((max_kv_len + kTokens - 1) / kTokens);
  const int32_t sms = CurrentDeviceSmCount();
  const unsigned grid = static_cast<unsigned>(most_tiles < sms ? (most_tiles > 0 ? most_tiles : 1) : sms);
  return CheckCuda(LaunchOverlapped(IndexerScoreTcKernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, key_map, q_map, p),
                   "indexer tensor-core score launch");
}

}  // namespace b200kv
