// Cross-GPU merge of KV-range shard partials over peer memory (NVLink), without a collective library.
//
// A long sequence is split by KV range over the ranks (one process per GPU). Each rank's decode leaves
// one partial per (sequence, head): m, l and the un-normalised O[512] in fp32. The exchange step is tiny
// (131,584 bytes per rank for 64 heads), so it is latency that counts. Every rank PUSHES its partial
// straight into every rank's inbox with plain peer stores and every rank merges what arrives in its own
// inbox, in ONE kernel, with no fence, flag or counter between the ranks: each fp32 value travels as an
// 8-byte word (epoch << 32 | value bits) written by a single 64-bit store, which is atomic, so a reader
// that sees the epoch in a word has its value. The reader polls the words it needs (bounded) and merges.
// This is the low-latency protocol of collective libraries, applied to one step; it moves twice the bytes
// (263 KB per rank and peer), which is nothing beside the round trip a fence would wait for.
//
// Exchange buffer of a rank (one peer-visible allocation, zero-filled at creation):
//   inbox[2][world][rows][514] u64   parity of the epoch, source rank, row: O[512], m, l as tagged words
//   epoch                      u32   local: epochs completed by this rank's kernel
//   done                       u32   local: CTA counter of the kernel
// Epoch e (1, 2, ...) uses the inbox half e & 1. A rank can run at most one epoch ahead of a peer (its
// merge of epoch e needs the peer's words of e, which the peer writes after finishing e - 1), so words of
// epoch e + 2 can only land in a half whose epoch-e words have all been consumed: two halves are enough.
//
// A warp waits only for words that kernels of OTHER GPUs write (its own rank's words it wrote itself before
// it polls), so no launch waits for another launch on its own GPU. The wait is bounded (about one second):
// a peer that does not arrive leaves B200KV_DEV_TIMEOUT in the status word and the kernel returns.
#include <cstring>

#include "common.cuh"
#include "kv_peer.cuh"

namespace b200kv {
namespace {

constexpr int kRowWords = kPeerRowWords;
constexpr int kMaxWorld = kPeerMaxWorld;

__host__ __device__ inline PeerLayout LayoutOf(int world, int64_t rows) { return PeerLayoutOf(world, rows); }

struct PeerParams {
  unsigned char* peer[kMaxWorld];  // exchange buffers of all ranks as seen from this process (own included)
  int32_t world;
  int32_t rank;
  int64_t rows;
  const float* partial_o;
  const float* partial_m;
  const float* partial_l;
  __nv_bfloat16* out;
  float* lse;
  int32_t* status;
};

__device__ __forceinline__ uint64_t LoadWord(const uint64_t* p) { return PeerLoadWord(p); }
__device__ __forceinline__ void StoreWord(uint64_t* p, uint64_t v) { PeerStoreWord(p, v); }
__device__ __forceinline__ uint64_t TimerNs() { return PeerTimerNs(); }

// One warp per row: pushes the row of this rank's partial to every rank, waits for the row from every rank,
// then the log-sum-exp merge M = max m_r, L = sum l_r e^(m_r - M), out = sum O_r e^(m_r - M) / L,
// lse = M + log L. Lane i holds elements i, i + 32, ... of a row; lanes 0 and 1 also hold m and l.
__global__ void __launch_bounds__(256) PeerMergeKernel(PeerParams p) {
  GridDependencyTrigger();
  GridDependencyWait();
  const PeerLayout lay = LayoutOf(p.world, p.rows);
  unsigned char* mine = p.peer[p.rank];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine + lay.epoch_offset) + 1u;
  const uint64_t tag = static_cast<uint64_t>(epoch) << 32;
  const size_t half = (epoch & 1u) * lay.inbox_bytes;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;

  // ---- push: every row this warp owns, to every rank (own inbox included) ----
  for (int64_t row = warp; row < p.rows; row += n_warps) {
    uint64_t words[17];
#pragma unroll
    for (int i = 0; i < 16; ++i) words[i] = tag | __float_as_uint(p.partial_o[row * B200KV_LATENT_DIM + lane + 32 * i]);
    words[16] = tag | __float_as_uint(lane == 0 ? p.partial_m[row] : (lane == 1 ? p.partial_l[row] : 0.0f));
    for (int dst = 0; dst < p.world; ++dst) {
      uint64_t* inbox = reinterpret_cast<uint64_t*>(p.peer[dst] + half) + (static_cast<size_t>(p.rank) * p.rows + row) * kRowWords;
#pragma unroll
      for (int i = 0; i < 16; ++i) StoreWord(inbox + lane + 32 * i, words[i]);
      if (lane < 2) StoreWord(inbox + B200KV_LATENT_DIM + lane, words[16]);
    }
  }

  // ---- pull and merge ----
  const uint64_t* inbox = reinterpret_cast<const uint64_t*>(mine + half);
  const uint64_t start = TimerNs();
  bool ok = true;
  for (int64_t row = warp; row < p.rows && ok; row += n_warps) {
    float big = -INFINITY, sum_l = 0.0f;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    for (int src = 0; src < p.world && ok; ++src) {
      const uint64_t* words = inbox + (static_cast<size_t>(src) * p.rows + row) * kRowWords;
      uint64_t w[17];
      uint32_t spins = 0;
      for (;;) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = LoadWord(words + lane + 32 * i);
        w[16] = lane < 2 ? LoadWord(words + B200KV_LATENT_DIM + lane) : tag;
        bool here = true;
#pragma unroll
        for (int i = 0; i < 17; ++i) here = here && (w[i] >> 32) == epoch;
        if (__all_sync(0xffffffffu, here)) break;
        if ((++spins & 63u) == 0 && TimerNs() - start > 1000000000ull) {
          if (lane == 0) RecordError(p.status, B200KV_DEV_TIMEOUT, 50, src, static_cast<int32_t>(epoch));
          ok = false;
          break;
        }
      }
      if (!ok) break;
      const float m = __shfl_sync(0xffffffffu, __uint_as_float(static_cast<uint32_t>(w[16])), 0);
      const float l = __shfl_sync(0xffffffffu, __uint_as_float(static_cast<uint32_t>(w[16])), 1);
      if (!(l > 0.0f)) continue;  // an empty shard
      const float new_big = fmaxf(big, m);
      const float carry = big == -INFINITY ? 0.0f : expf(big - new_big);
      const float weight = expf(m - new_big);
      big = new_big;
      sum_l = sum_l * carry + l * weight;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(acc[i], carry, __uint_as_float(static_cast<uint32_t>(w[i])) * weight);
    }
    if (!ok) break;
    const float inv = sum_l > 0.0f ? 1.0f / sum_l : 0.0f;
    __nv_bfloat16* dst = p.out + row * B200KV_LATENT_DIM;
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(acc[i] * inv);
    if (lane == 0 && p.lse != nullptr) p.lse[row] = sum_l > 0.0f ? big + logf(sum_l) : -INFINITY;
  }

  // The epoch is complete for this rank when every CTA is done with the inbox half; a launch whose wait ran
  // out completes it too, so that the ranks that did arrive are not held up in the next one by this one.
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = reinterpret_cast<uint32_t*>(mine + lay.done_offset);
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0;
      *reinterpret_cast<volatile uint32_t*>(mine + lay.epoch_offset) = epoch;
    }
  }
}

}  // namespace
}  // namespace b200kv

using namespace b200kv;

extern "C" size_t b200kv_peer_exchange_bytes(int32_t world, int64_t rows) {
  if (world < 1 || world > kMaxWorld || rows < 1) return 0;
  return LayoutOf(world, rows).total;
}

extern "C" int32_t b200kv_peer_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr) {
    SetLastError("peer_buffer_alloc: ptr and handle must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  *ptr = nullptr;
  if (bytes == 0) {
    SetLastError("peer_buffer_alloc: zero bytes");
    return B200KV_ERR_INVALID;
  }
  void* p = nullptr;
  if (int32_t rc = CheckCuda(cudaMalloc(&p, bytes), "cudaMalloc(peer exchange buffer)")) return rc;
  if (int32_t rc = CheckCuda(cudaMemset(p, 0, bytes), "cudaMemset(peer exchange buffer)")) {
    cudaFree(p);
    return rc;
  }
  cudaIpcMemHandle_t handle;
  if (int32_t rc = CheckCuda(cudaIpcGetMemHandle(&handle, p), "cudaIpcGetMemHandle")) {
    cudaFree(p);
    return rc;
  }
  std::memcpy(handle64, &handle, 64);
  *ptr = p;
  return B200KV_OK;
}

extern "C" int32_t b200kv_peer_buffer_open(const unsigned char* handle64, void** ptr) {
  if (handle64 == nullptr || ptr == nullptr) {
    SetLastError("peer_buffer_open: handle and ptr must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle64, 64);
  return CheckCuda(cudaIpcOpenMemHandle(ptr, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

extern "C" int32_t b200kv_peer_buffer_close(void* ptr) {
  return ptr == nullptr ? B200KV_OK : CheckCuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle");
}

extern "C" int32_t b200kv_peer_buffer_free(void* ptr) {
  return ptr == nullptr ? B200KV_OK : CheckCuda(cudaFree(ptr), "cudaFree(peer exchange buffer)");
}

extern "C" int32_t b200kv_peer_merge(void* const* peer_buffers, int32_t world, int32_t rank, int64_t rows,
                                     const float* partial_o, const float* partial_m, const float* partial_l,
                                     void* out_bf16, float* lse, void* stream, b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_peer_merge")) return rc;
  if (peer_buffers == nullptr || partial_o == nullptr || partial_m == nullptr || partial_l == nullptr || out_bf16 == nullptr) {
    SetLastError("peer_merge: peer_buffers, the three partial arrays and out must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || rows < 1) {
    SetLastError("peer_merge refused: world %d (1..%d), rank %d, rows %lld", world, kMaxWorld, rank,
                 static_cast<long long>(rows));
    return B200KV_ERR_INVALID;
  }
  PeerParams p{};
  for (int r = 0; r < world; ++r) {
    if (peer_buffers[r] == nullptr) {
      SetLastError("peer_merge: the exchange buffer of rank %d is null", r);
      return B200KV_ERR_NULLPTR;
    }
    p.peer[r] = static_cast<unsigned char*>(peer_buffers[r]);
  }
  p.world = world;
  p.rank = rank;
  p.rows = rows;
  p.partial_o = partial_o;
  p.partial_m = partial_m;
  p.partial_l = partial_l;
  p.out = static_cast<__nv_bfloat16*>(out_bf16);
  p.lse = lse;
  p.status = status;
  const int merge_grid = static_cast<int>((rows + 7) / 8 > 148 ? 148 : (rows + 7) / 8);
  return CheckCuda(LaunchOverlapped(PeerMergeKernel, dim3(merge_grid), dim3(256), 0, static_cast<cudaStream_t>(stream), p),
                   "peer merge launch");
}
