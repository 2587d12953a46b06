// The tagged-word exchange buffer shared by the kernels that merge KV-range shards across GPUs over peer memory
// (kv_peer.cu: merge of finished shard partials; mla_decode_tc.cu: the decode's own merge kernel pushing
// directly). Layout and protocol are described in kv_peer.cu.
#pragma once

#include "common.cuh"

namespace b200kv {

constexpr int kPeerRowWords = B200KV_LATENT_DIM + 2;  // O[512], m, l
constexpr int kPeerMaxWorld = 16;

struct PeerLayout {
  size_t inbox_bytes;  // one half
  size_t epoch_offset;
  size_t done_offset;
  size_t total;
};

__host__ __device__ inline PeerLayout PeerLayoutOf(int world, int64_t rows) {
  PeerLayout l;
  l.inbox_bytes = static_cast<size_t>(world) * rows * kPeerRowWords * sizeof(uint64_t);
  l.epoch_offset = (2 * l.inbox_bytes + 255) & ~static_cast<size_t>(255);
  l.done_offset = l.epoch_offset + 64;
  l.total = l.done_offset + 64;
  return l;
}

// Exchange buffers of all ranks as seen from this process (own included), and who this rank is.
struct PeerRing {
  unsigned char* peer[kPeerMaxWorld];
  int32_t world;
  int32_t rank;
  int64_t rows;
};

__device__ __forceinline__ uint64_t PeerLoadWord(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void PeerStoreWord(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ uint64_t PeerTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

}  // namespace b200kv
