// Cross-GPU merge of KV-range shard partials over peer memory (NVLink), without a collective library.
//
// A long sequence is split by KV range over the ranks (one process per GPU). Each rank's decode leaves
// one partial per (sequence, head): m, l and the un-normalised O[512] in fp32, 2,056 bytes. The exchange
// step is tiny (131,584 bytes per rank for 64 heads), so it is latency that counts: instead of an
// all-gather followed by a merge kernel, every rank PUSHES its partial straight into every peer's inbox
// with plain peer stores and then raises a flag there; the merge kernel of each rank waits for the flags
// of all ranks in its own memory and reduces what has arrived. Two small kernels per rank and layer, no
// host synchronisation, capturable in a CUDA graph.
//
// Exchange buffer of a rank (one peer-visible allocation, zero-filled at creation):
//   inbox[2][world][rows][514] fp32   parity of the epoch, source rank, row: O[512], m, l
//   flags[2][world]            u32    the epoch whose data of that source rank is complete
//   epoch                      u32    local: epochs completed by this rank's merge kernel
//   done[2]                    u32    local: CTA counters of the two kernels
// Epoch e uses the inbox half e & 1. A rank can run at most one epoch ahead of a peer (its merge of epoch
// e needs the peer's push of e, which the peer issues after its own merge of e - 1), so when data of epoch
// e + 2 arrives in a half, the merge of epoch e that read it has finished: two halves are enough.
//
// The waits are on kernels of OTHER GPUs only (a push kernel waits for nothing), so no kernel here waits
// for another launch on its own GPU. Every wait is bounded (about one second): a peer that does not
// arrive leaves B200KV_DEV_TIMEOUT in the status word and the kernel returns.
#include <cstring>

#include "common.cuh"

namespace b200kv {
namespace {

constexpr int kRowFloats = B200KV_LATENT_DIM + 2;  // O[512], m, l
constexpr int kMaxWorld = 16;

struct PeerLayout {
  size_t inbox_bytes;  // one half
  size_t flags_offset;
  size_t epoch_offset;
  size_t done_offset;
  size_t total;
};

__host__ __device__ inline PeerLayout LayoutOf(int world, int64_t rows) {
  PeerLayout l;
  l.inbox_bytes = static_cast<size_t>(world) * rows * kRowFloats * sizeof(float);
  l.flags_offset = (2 * l.inbox_bytes + 255) & ~static_cast<size_t>(255);
  l.epoch_offset = l.flags_offset + 2 * kMaxWorld * sizeof(uint32_t);
  l.done_offset = l.epoch_offset + 64;
  l.total = l.done_offset + 64;
  return l;
}

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

__device__ __forceinline__ uint32_t LoadAcquireSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void StoreReleaseSys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint64_t TimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Copies this rank's partial rows into slot `rank` of every rank's inbox half, then raises the flags.
__global__ void __launch_bounds__(256) PeerPushKernel(PeerParams p) {
  GridDependencyTrigger();
  GridDependencyWait();
  const PeerLayout lay = LayoutOf(p.world, p.rows);
  unsigned char* mine = p.peer[p.rank];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine + lay.epoch_offset) + 1u;
  const size_t half = (epoch & 1u) * lay.inbox_bytes;
  const int64_t chunks_per_row = kRowFloats * 4 / 8;  // 8-byte pieces: a row is 2,056 bytes
  const int64_t total = p.rows * chunks_per_row;
  for (int dst = 0; dst < p.world; ++dst) {
    float* inbox = reinterpret_cast<float*>(p.peer[dst] + half) + static_cast<size_t>(p.rank) * p.rows * kRowFloats;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int64_t row = i / chunks_per_row, c = i % chunks_per_row;
      float2 v;
      if (c < B200KV_LATENT_DIM / 2) {
        v = *reinterpret_cast<const float2*>(p.partial_o + row * B200KV_LATENT_DIM + 2 * c);
      } else {
        v = make_float2(p.partial_m[row], p.partial_l[row]);
      }
      *reinterpret_cast<float2*>(inbox + row * kRowFloats + 2 * c) = v;
    }
  }
  // Everything this CTA stored is visible system-wide before it is counted; the last CTA raises the flags.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = reinterpret_cast<uint32_t*>(mine + lay.done_offset);
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0;
      __threadfence_system();
      for (int dst = 0; dst < p.world; ++dst) {
        uint32_t* flags = reinterpret_cast<uint32_t*>(p.peer[dst] + lay.flags_offset);
        StoreReleaseSys(flags + (epoch & 1u) * kMaxWorld + p.rank, epoch);
      }
    }
  }
}

// One warp per row: waits until every rank's data of this epoch is in the local inbox, then the
// log-sum-exp merge M = max m_r, L = sum l_r e^(m_r - M), out = sum O_r e^(m_r - M) / L, lse = M + log L.
__global__ void __launch_bounds__(256) PeerMergeKernel(PeerParams p) {
  GridDependencyTrigger();
  GridDependencyWait();
  const PeerLayout lay = LayoutOf(p.world, p.rows);
  unsigned char* mine = p.peer[p.rank];
  __shared__ int arrived;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine + lay.epoch_offset) + 1u;
  if (threadIdx.x == 0) {
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(mine + lay.flags_offset) + (epoch & 1u) * kMaxWorld;
    int ok = 1;
    const uint64_t start = TimerNs();
    for (int r = 0; r < p.world && ok; ++r) {
      uint32_t it = 0;
      while (LoadAcquireSys(flags + r) != epoch) {
        if ((++it & 255u) == 0 && TimerNs() - start > 1000000000ull) {
          RecordError(p.status, B200KV_DEV_TIMEOUT, 50, r, static_cast<int32_t>(epoch));
          ok = 0;
          break;
        }
      }
    }
    arrived = ok;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  if (arrived) {
    const float* inbox = reinterpret_cast<const float*>(mine + (epoch & 1u) * lay.inbox_bytes);
    for (int64_t row = warp; row < p.rows; row += n_warps) {
      float m = -INFINITY, l = 0.0f;
      if (lane < p.world) {
        const float* src = inbox + (static_cast<size_t>(lane) * p.rows + row) * kRowFloats;
        m = __ldcg(src + B200KV_LATENT_DIM);
        l = __ldcg(src + B200KV_LATENT_DIM + 1);
        if (!(l > 0.0f)) m = -INFINITY;
      }
      float big = m;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
      const float w = (l > 0.0f && big != -INFINITY) ? expf(m - big) : 0.0f;
      float sum_l = l * w;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum_l += __shfl_xor_sync(0xffffffffu, sum_l, off);
      float4 acc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int r = 0; r < p.world; ++r) {
        const float wr = __shfl_sync(0xffffffffu, w, r);
        if (wr == 0.0f) continue;
        const float4* src = reinterpret_cast<const float4*>(inbox + (static_cast<size_t>(r) * p.rows + row) * kRowFloats);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // rows are 2,056 bytes apart: 8-byte aligned, so two 8-byte loads per 16 bytes
          const float2* s2 = reinterpret_cast<const float2*>(src) + 2 * (lane + 32 * i);
          const float2 a = __ldcg(s2), b = __ldcg(s2 + 1);
          acc[i].x = fmaf(a.x, wr, acc[i].x);
          acc[i].y = fmaf(a.y, wr, acc[i].y);
          acc[i].z = fmaf(b.x, wr, acc[i].z);
          acc[i].w = fmaf(b.y, wr, acc[i].w);
        }
      }
      const float inv = sum_l > 0.0f ? 1.0f / sum_l : 0.0f;
      uint2* dst = reinterpret_cast<uint2*>(p.out + row * B200KV_LATENT_DIM);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[i].x * inv, acc[i].y * inv);
        const __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc[i].z * inv, acc[i].w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo2);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi2);
        dst[lane + 32 * i] = packed;
      }
      if (lane == 0 && p.lse != nullptr) p.lse[row] = sum_l > 0.0f ? big + logf(sum_l) : -INFINITY;
    }
  }
  // The epoch is complete for this rank when every CTA is done with the inbox half; a launch whose wait ran
  // out completes it too, so that the ranks that did arrive are not held up in the next one by this one.
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = reinterpret_cast<uint32_t*>(mine + lay.done_offset) + 1;
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t push_items = rows * (kRowFloats / 2);
  const int push_grid = static_cast<int>(push_items / 256 < 1 ? 1 : (push_items / 256 > 64 ? 64 : push_items / 256));
  if (int32_t rc = CheckCuda(LaunchOverlapped(PeerPushKernel, dim3(push_grid), dim3(256), 0, s, p), "peer push launch")) {
    return rc;
  }
  const int merge_grid = static_cast<int>((rows + 7) / 8 > 148 ? 148 : (rows + 7) / 8);
  return CheckCuda(LaunchOverlapped(PeerMergeKernel, dim3(merge_grid), dim3(256), 0, s, p), "peer merge launch");
}
