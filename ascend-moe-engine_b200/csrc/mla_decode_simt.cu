// Absorbed-MLA decode attention on CUDA cores: the geometry-generic implementation (any head count,
// any block size) and the on-device cross-check for the tensor-core kernel. fp32 accumulation
// throughout, online softmax per head, split-KV with a log-sum-exp merge.
//
// Grid (split, sequence, head group of 64). A CTA keeps its 64 query rows in shared memory, streams
// its token range in tiles of 32 rows through shared memory, and every thread owns one head and one
// eighth of the 512 output columns (64 fp32 accumulators).
#include "common.cuh"

namespace b200kv {

namespace {

constexpr int kThreads = 512;
constexpr int kTile = 32;                // tokens per tile
constexpr int kHeadsPerCta = 64;
constexpr int kRowWords = 292;           // 576 bf16 = 288 words, padded by 4 against bank conflicts
constexpr int kLatentWords = B200KV_LATENT_DIM / 2;
constexpr int kRowWidthWords = (B200KV_LATENT_DIM + B200KV_ROPE_DIM) / 2;
constexpr size_t kSmemBytes =
    static_cast<size_t>(kHeadsPerCta + kTile) * kRowWords * 4 + static_cast<size_t>(kHeadsPerCta) * (kTile + 1) * 4;

__device__ __forceinline__ float2 Bf16x2ToFloat2(uint32_t w) {
  float2 r;
  r.x = __uint_as_float(w << 16);
  r.y = __uint_as_float(w & 0xffff0000u);
  return r;
}

struct SimtParams {
  const __nv_bfloat16* q;
  int64_t q_seq_stride;
  int64_t q_head_stride;
  b200kv_pool_view pool;
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  const int32_t* kv_begin;
  int32_t batch;
  int32_t heads;
  int32_t block_size;
  float scale;
  // direct outputs (n_splits == 1 and no partial requested)
  __nv_bfloat16* out;
  float* lse;
  // split partials [split][batch*heads]
  float* part_o;
  float* part_m;
  float* part_l;
  int32_t direct;
  int32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1) MlaDecodeSimtKernel(SimtParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* q_s = reinterpret_cast<uint32_t*>(smem_raw);                 // [64][kRowWords]
  uint32_t* kv_s = q_s + kHeadsPerCta * kRowWords;                       // [32][kRowWords]
  float* p_s = reinterpret_cast<float*>(kv_s + kTile * kRowWords);       // [64][kTile+1]

  const int split = blockIdx.x;
  const int n_splits = gridDim.x;
  const int b = blockIdx.y;
  const int head_base = blockIdx.z * kHeadsPerCta;
  const int tid = threadIdx.x;
  const int h_local = tid >> 3;
  const int part = tid & 7;
  const int h = head_base + h_local;
  const bool head_ok = h < p.heads;

  const int len = p.kv_len[b];
  const int begin = p.kv_begin ? p.kv_begin[b] : 0;
  const int n_tiles = (len + kTile - 1) / kTile;
  const int tile_lo = static_cast<int>(static_cast<int64_t>(n_tiles) * split / n_splits);
  const int tile_hi = static_cast<int>(static_cast<int64_t>(n_tiles) * (split + 1) / n_splits);

  // Stage the query rows (bf16 pairs as 32-bit words).
  for (int idx = tid; idx < kHeadsPerCta * kRowWidthWords; idx += kThreads) {
    const int hh = idx / kRowWidthWords;
    const int w = idx - hh * kRowWidthWords;
    uint32_t v = 0;
    if (head_base + hh < p.heads) {
      const __nv_bfloat16* src = p.q + b * p.q_seq_stride + (head_base + hh) * p.q_head_stride + 2 * w;
      v = *reinterpret_cast<const uint32_t*>(src);
    }
    q_s[hh * kRowWords + w] = v;
  }

  float acc[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
  float m_run = -INFINITY;
  float l_run = 0.0f;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    __syncthreads();  // previous tile fully consumed (and q_s visible on the first pass)
    const int tok0 = tile * kTile;
    const int valid = min(kTile, len - tok0);
    // Load the tile: 32 rows x 72 chunks of 16 bytes.
    for (int idx = tid; idx < kTile * 72; idx += kThreads) {
      const int j = idx / 72;
      const int c = idx - j * 72;
      int4 v = make_int4(0, 0, 0, 0);
      if (j < valid) {
        const int tok = begin + tok0 + j;
        // A length beyond the table's row (the lengths are device data) must not index past it.
        const int64_t column = tok / p.block_size;
        const int64_t block =
            (tok >= 0 && column < p.max_blocks) ? p.block_table[static_cast<int64_t>(b) * p.max_blocks + column] : -1;
        const int64_t row = block * p.block_size + tok % p.block_size;
        if (block < 0 || row >= p.pool.pool_rows) {
          RecordError(p.status, B200KV_DEV_BAD_BLOCK, b, tok / p.block_size, static_cast<int32_t>(block));
        } else if (c < 64) {
          v = *reinterpret_cast<const int4*>(static_cast<const __nv_bfloat16*>(p.pool.latent) +
                                             row * p.pool.latent_row_stride + 8 * c);
        } else {
          v = *reinterpret_cast<const int4*>(static_cast<const __nv_bfloat16*>(p.pool.rope) +
                                             row * p.pool.rope_row_stride + 8 * (c - 64));
        }
      }
      *reinterpret_cast<int4*>(&kv_s[j * kRowWords + 4 * c]) = v;
    }
    __syncthreads();

    // Scores for tokens part, part+8, part+16, part+24 of this thread's head.
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
      const uint32_t* qrow = q_s + h_local * kRowWords;
#pragma unroll 4
      for (int w = 0; w < kRowWidthWords; ++w) {
        const float2 qv = Bf16x2ToFloat2(qrow[w]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 kv = Bf16x2ToFloat2(kv_s[(part + 8 * i) * kRowWords + w]);
          s[i] = fmaf(qv.x, kv.x, s[i]);
          s[i] = fmaf(qv.y, kv.y, s[i]);
        }
      }
    }
    float tile_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] = (part + 8 * i < valid) ? s[i] * p.scale : -INFINITY;
      tile_max = fmaxf(tile_max, s[i]);
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, off));
    const float m_new = fmaxf(m_run, tile_max);
    const float alpha = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_new);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pv = (s[i] == -INFINITY) ? 0.0f : __expf(s[i] - m_new);
      p_s[h_local * (kTile + 1) + part + 8 * i] = pv;
      sum += pv;
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    l_run = l_run * alpha + sum;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] *= alpha;
    __syncthreads();

    // PV: this thread owns latent words part + 8*i (i < 32) of its head's output row.
    for (int j = 0; j < valid; ++j) {
      const float pv = p_s[h_local * (kTile + 1) + j];
      const uint32_t* vrow = kv_s + j * kRowWords;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float2 v = Bf16x2ToFloat2(vrow[part + 8 * i]);
        acc[2 * i] = fmaf(pv, v.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(pv, v.y, acc[2 * i + 1]);
      }
    }
  }

  if (!head_ok) return;
  const int64_t row_index = static_cast<int64_t>(b) * p.heads + h;
  if (p.direct) {
    const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    __nv_bfloat16* dst = p.out + row_index * B200KV_LATENT_DIM;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + 2 * (part + 8 * i)) = v;
    }
    if (part == 0 && p.lse) p.lse[row_index] = l_run > 0.0f ? m_run + logf(l_run) : -INFINITY;
  } else {
    const int64_t slot = static_cast<int64_t>(split) * p.batch * p.heads + row_index;
    float* dst = p.part_o + slot * B200KV_LATENT_DIM;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      *reinterpret_cast<float2*>(dst + 2 * (part + 8 * i)) = make_float2(acc[2 * i], acc[2 * i + 1]);
    }
    if (part == 0) {
      p.part_m[slot] = m_run;
      p.part_l[slot] = l_run;
    }
  }
}

// One warp per (sequence, head) row: merges n_parts partials laid out [part][rows].
// emit_partial != 0 writes the un-normalised merged (m, l, O) instead of (out, lse).
__global__ void __launch_bounds__(256)
    LseMergeKernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                   const float* __restrict__ part_l, int32_t n_parts, int64_t rows, __nv_bfloat16* out, float* lse,
                   float* merged_o, float* merged_m, float* merged_l, int32_t emit_partial) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  float big = -INFINITY;
  for (int r = 0; r < n_parts; ++r) {
    if (part_l[r * rows + row] > 0.0f) big = fmaxf(big, part_m[r * rows + row]);
  }
  float total = 0.0f;
  float4 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int r = 0; r < n_parts; ++r) {
    const float l = part_l[r * rows + row];
    if (!(l > 0.0f)) continue;
    const float w = expf(part_m[r * rows + row] - big);
    total += l * w;
    const float4* src = reinterpret_cast<const float4*>(part_o + (r * rows + row) * B200KV_LATENT_DIM);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = src[lane + 32 * i];
      acc[i].x = fmaf(v.x, w, acc[i].x);
      acc[i].y = fmaf(v.y, w, acc[i].y);
      acc[i].z = fmaf(v.z, w, acc[i].z);
      acc[i].w = fmaf(v.w, w, acc[i].w);
    }
  }
  if (emit_partial) {
    float4* dst = reinterpret_cast<float4*>(merged_o + row * B200KV_LATENT_DIM);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = acc[i];
    if (lane == 0) {
      merged_m[row] = big;
      merged_l[row] = total;
    }
    return;
  }
  const float inv = total > 0.0f ? 1.0f / total : 0.0f;
  uint2* dst = reinterpret_cast<uint2*>(out + row * B200KV_LATENT_DIM);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x * inv, acc[i].y * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z * inv, acc[i].w * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    dst[lane + 32 * i] = packed;
  }
  if (lane == 0 && lse) lse[row] = total > 0.0f ? big + logf(total) : -INFINITY;
}

}  // namespace

int32_t SimtSplitCount(int32_t batch, int32_t sms) {
  int32_t splits = (2 * sms) / (batch > 0 ? batch : 1);
  if (splits < 1) splits = 1;
  if (splits > 32) splits = 32;
  return splits;
}

size_t SimtWorkspaceBytes(int32_t batch, int32_t heads, int32_t sms) {
  const size_t slots = static_cast<size_t>(SimtSplitCount(batch, sms)) * batch * heads;
  return slots * (B200KV_LATENT_DIM + 2) * sizeof(float);
}

int32_t LaunchLseMerge(const float* part_o, const float* part_m, const float* part_l, int32_t n_parts, int64_t rows,
                       void* out, float* lse, float* merged_o, float* merged_m, float* merged_l, cudaStream_t stream) {
  const int64_t ctas = (rows + 7) / 8;
  LseMergeKernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(
      part_o, part_m, part_l, n_parts, rows, static_cast<__nv_bfloat16*>(out), lse, merged_o, merged_m, merged_l,
      merged_o != nullptr);
  return CheckCuda(cudaGetLastError(), "lse merge launch");
}

int32_t LaunchMlaDecodeSimt(const b200kv_decode_args& a, cudaStream_t stream, int32_t* status) {
  static thread_local int configured_device = -1;
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device != configured_device) {
    if (int32_t rc = CheckCuda(cudaFuncSetAttribute(MlaDecodeSimtKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    static_cast<int>(kSmemBytes)),
                               "simt decode smem opt-in")) {
      return rc;
    }
    configured_device = device;
  }
  const int32_t sms = CurrentDeviceSmCount();
  const int32_t splits = SimtSplitCount(a.batch, sms);
  const bool want_partial = a.partial_o != nullptr;
  const int64_t rows = static_cast<int64_t>(a.batch) * a.heads;

  SimtParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.q_seq_stride = a.q_seq_stride;
  p.q_head_stride = a.q_head_stride;
  p.pool = a.pool;
  p.block_table = a.block_table;
  p.max_blocks = a.max_blocks;
  p.kv_len = a.kv_len;
  p.kv_begin = a.kv_begin;
  p.batch = a.batch;
  p.heads = a.heads;
  p.block_size = a.block_size;
  p.scale = a.scale;
  p.status = status;
  p.direct = (splits == 1 && !want_partial) ? 1 : 0;
  if (p.direct) {
    p.out = static_cast<__nv_bfloat16*>(a.out);
    p.lse = a.lse;
  } else if (splits == 1) {
    // A single split writes the caller's partial buffers as its one and only part.
    p.part_o = a.partial_o;
    p.part_m = a.partial_m;
    p.part_l = a.partial_l;
  } else {
    float* ws = static_cast<float*>(a.workspace);
    const size_t slots = static_cast<size_t>(splits) * rows;
    p.part_o = ws;
    p.part_m = ws + slots * B200KV_LATENT_DIM;
    p.part_l = p.part_m + slots;
  }
  dim3 grid(splits, a.batch, (a.heads + kHeadsPerCta - 1) / kHeadsPerCta);
  MlaDecodeSimtKernel<<<grid, kThreads, kSmemBytes, stream>>>(p);
  if (int32_t rc = CheckCuda(cudaGetLastError(), "simt decode launch")) return rc;
  if (splits > 1) {
    return LaunchLseMerge(p.part_o, p.part_m, p.part_l, splits, rows, a.out, a.lse, a.partial_o, a.partial_m,
                          a.partial_l, stream);
  }
  return B200KV_OK;
}

}  // namespace b200kv
