// The stages on either side of the KV path, as kernels of their own:
//
//   producer  RMSNorm of the appended row's 512-wide latent, rotary embedding ("half" pairing) of its
//             64-wide rope slice, and the write of both into the paged pool, in ONE kernel, so the
//             normalised row never makes a round trip through an activation buffer; the same launch
//             rotates the query's rope slices in place (the reference runs these as three operators,
//             stages 6-8 of src/pipeline/pipeline.cpp:212-234).
//   consumer  block-32 MX quantisation of the attention output to FP8 E4M3 with E8M0 scales (stage 10,
//             src/pipeline/pipeline.cpp:250-258).
//
// All three are memory-bound element-wise work: one warp per row or vector, 16-byte accesses. Their
// arithmetic is fixed to the operation (explicit round-to-nearest intrinsics, a fixed reduction order),
// so that results are bit-identical with the CPU statement of the same rules:
//   RMSNorm: lane L sums fma(x, x, a) over elements 8L..8L+7 then 256+8L..256+8L+7; butterfly over
//            xor 16, 8, 4, 2, 1; r = 1 / sqrt(a/512 + eps); y = bf16((x * r) * g).
//   RoPE:    y_i = bf16(fma(-x_(i+32), s_i, x_i * c_i)); y_(i+32) = bf16(fma(x_i, s_(i+32), x_(i+32) * c_(i+32))).
//   MX:      e = floor(log2 max|x|) - 8 clamped to [-127, 127] (all zero: -127); scale byte e + 127;
//            q = e4m3(x * 2^-e), nearest even, saturating; a NaN in the block makes scale and values NaN.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200kv {
namespace {

constexpr int kLatent = B200KV_LATENT_DIM;
constexpr int kRope = B200KV_ROPE_DIM;
static_assert(kLatent == 512 && kRope == 64, "the lane assignment below is written for 512 + 64");
constexpr int kWarpsPerCta = 8;

struct ProducerParams {
  b200kv_pool_view pool;
  const __nv_bfloat16* kv_a;
  int64_t kv_a_stride;
  const __nv_bfloat16* gamma;
  float eps;
  const __nv_bfloat16* cos;
  int64_t cos_stride;
  const __nv_bfloat16* sin;
  int64_t sin_stride;
  const int32_t* slots;
  int64_t tokens;
  __nv_bfloat16* q_rope;  // [tokens][heads][64] rotated in place, or null
  int64_t q_token_stride;
  int64_t q_head_stride;
  int32_t heads;
  __nv_bfloat16* latent_out;  // optional copies of what went into the pool (the reference's act buffers)
  int64_t latent_out_stride;
  __nv_bfloat16* rope_out;
  int64_t rope_out_stride;
  float* rstd_out;
  int32_t* status;
};

__device__ __forceinline__ float Bf16Bits(uint32_t packed, int hi) {
  return __uint_as_float(hi ? (packed & 0xffff0000u) : (packed << 16));
}

__device__ __forceinline__ uint32_t PackBf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Rotates eight pairs (i, i + 32) held as two 16-byte chunks: x1 = elements 8j..8j+7, x2 = 32+8j..32+8j+7.
__device__ __forceinline__ void RotateChunks(const int4& x1, const int4& x2, const int4& c1, const int4& c2, const int4& s1,
                                             const int4& s2, int4* y1, int4* y2) {
  const uint32_t a[4] = {static_cast<uint32_t>(x1.x), static_cast<uint32_t>(x1.y), static_cast<uint32_t>(x1.z), static_cast<uint32_t>(x1.w)};
  const uint32_t b[4] = {static_cast<uint32_t>(x2.x), static_cast<uint32_t>(x2.y), static_cast<uint32_t>(x2.z), static_cast<uint32_t>(x2.w)};
  const uint32_t ca[4] = {static_cast<uint32_t>(c1.x), static_cast<uint32_t>(c1.y), static_cast<uint32_t>(c1.z), static_cast<uint32_t>(c1.w)};
  const uint32_t cb[4] = {static_cast<uint32_t>(c2.x), static_cast<uint32_t>(c2.y), static_cast<uint32_t>(c2.z), static_cast<uint32_t>(c2.w)};
  const uint32_t sa[4] = {static_cast<uint32_t>(s1.x), static_cast<uint32_t>(s1.y), static_cast<uint32_t>(s1.z), static_cast<uint32_t>(s1.w)};
  const uint32_t sb[4] = {static_cast<uint32_t>(s2.x), static_cast<uint32_t>(s2.y), static_cast<uint32_t>(s2.z), static_cast<uint32_t>(s2.w)};
  uint32_t ya[4], yb[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    float lo[2], hi[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float x_lo = Bf16Bits(a[w], h), x_hi = Bf16Bits(b[w], h);
      lo[h] = __fmaf_rn(-x_hi, Bf16Bits(sa[w], h), __fmul_rn(x_lo, Bf16Bits(ca[w], h)));
      hi[h] = __fmaf_rn(x_lo, Bf16Bits(sb[w], h), __fmul_rn(x_hi, Bf16Bits(cb[w], h)));
    }
    ya[w] = PackBf16(lo[0], lo[1]);
    yb[w] = PackBf16(hi[0], hi[1]);
  }
  *y1 = make_int4(ya[0], ya[1], ya[2], ya[3]);
  *y2 = make_int4(yb[0], yb[1], yb[2], yb[3]);
}

__device__ __forceinline__ int4 LoadChunk(const __nv_bfloat16* p) { return *reinterpret_cast<const int4*>(p); }
__device__ __forceinline__ void StoreChunk(__nv_bfloat16* p, const int4& v) { *reinterpret_cast<int4*>(p) = v; }

constexpr int kRowsPerPass = 2;  // rows a warp has in flight; with 64 registers four CTAs share an SM, which
                                 // hides the arithmetic of one warp behind the loads of the others

__global__ void __launch_bounds__(kWarpsPerCta * 32, 4) ProducerKernel(ProducerParams p) {
  GridDependencyTrigger();
  GridDependencyWait();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t rows = p.kv_a != nullptr ? p.tokens : 0;  // no rows: only vectors are rotated
  const int64_t row_items = (rows + kRowsPerPass - 1) / kRowsPerPass;
  // Vectors (query rope slices, [tokens][heads][64], in place): eight per warp pass, four lanes each.
  const int64_t vectors = p.q_rope != nullptr ? p.tokens * p.heads : 0;
  const int64_t vector_items = (vectors + 7) / 8;
  int4 ga = make_int4(0, 0, 0, 0), gb = ga;
  if (rows > 0) {
    ga = *reinterpret_cast<const int4*>(p.gamma + 8 * lane);
    gb = *reinterpret_cast<const int4*>(p.gamma + 256 + 8 * lane);
  }
  const uint32_t gw[8] = {static_cast<uint32_t>(ga.x), static_cast<uint32_t>(ga.y), static_cast<uint32_t>(ga.z),
                          static_cast<uint32_t>(ga.w), static_cast<uint32_t>(gb.x), static_cast<uint32_t>(gb.y),
                          static_cast<uint32_t>(gb.z), static_cast<uint32_t>(gb.w)};
  for (int64_t item = warp; item < row_items + vector_items; item += n_warps) {
    if (item >= row_items) {
      const int64_t v = (item - row_items) * 8 + (lane >> 2);
      const int j = lane & 3;
      if (v < vectors) {
        const int64_t t = v / p.heads, h = v % p.heads;
        __nv_bfloat16* x = p.q_rope + t * p.q_token_stride + h * p.q_head_stride;
        const __nv_bfloat16* c = p.cos + t * p.cos_stride;
        const __nv_bfloat16* s = p.sin + t * p.sin_stride;
        int4 y1, y2;
        RotateChunks(LoadChunk(x + 8 * j), LoadChunk(x + 32 + 8 * j), LoadChunk(c + 8 * j), LoadChunk(c + 32 + 8 * j),
                     LoadChunk(s + 8 * j), LoadChunk(s + 32 + 8 * j), &y1, &y2);
        StoreChunk(x + 8 * j, y1);
        StoreChunk(x + 32 + 8 * j, y2);
      }
      continue;
    }
    const int64_t t0 = item * kRowsPerPass;
    // Everything the pass reads leaves before anything is computed: the slots (lanes 0-3), the four rows'
    // latent halves, and the rope chunks with their cos/sin (lanes 8r..8r+3 for row r).
    int my_slot = -1;
    if (lane < kRowsPerPass && t0 + lane < rows && p.slots != nullptr) my_slot = p.slots[t0 + lane];
    int4 xa[kRowsPerPass], xb[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
      xa[r] = xb[r] = make_int4(0, 0, 0, 0);
      if (t0 + r < rows) {
        const __nv_bfloat16* row = p.kv_a + (t0 + r) * p.kv_a_stride;
        xa[r] = LoadStream16(row + 8 * lane);
        xb[r] = LoadStream16(row + 256 + 8 * lane);
      }
    }
    // The rope slice of row rr goes out first (its registers are then free for the rows' arithmetic).
    const int rr = lane >> 3, j = lane & 7;  // row rr of the pass, chunk j (only j < 4 works)
    const int rope_slot = __shfl_sync(0xffffffffu, my_slot, rr < kRowsPerPass ? rr : 0);  // by every lane
    if (p.cos != nullptr && j < 4 && rr < kRowsPerPass && t0 + rr < rows) {
      const int64_t t = t0 + rr;
      const __nv_bfloat16* x = p.kv_a + t * p.kv_a_stride + kLatent;
      const __nv_bfloat16* c = p.cos + t * p.cos_stride;
      const __nv_bfloat16* s = p.sin + t * p.sin_stride;
      int4 y1, y2;
      RotateChunks(LoadChunk(x + 8 * j), LoadChunk(x + 32 + 8 * j), LoadChunk(c + 8 * j), LoadChunk(c + 32 + 8 * j),
                   LoadChunk(s + 8 * j), LoadChunk(s + 32 + 8 * j), &y1, &y2);
      if (rope_slot >= 0 && rope_slot < p.pool.pool_rows) {
        __nv_bfloat16* dst =
            static_cast<__nv_bfloat16*>(p.pool.rope) + static_cast<int64_t>(rope_slot) * p.pool.rope_row_stride;
        StoreChunk(dst + 8 * j, y1);
        StoreChunk(dst + 32 + 8 * j, y2);
      }
      if (p.rope_out != nullptr) {
        __nv_bfloat16* dst = p.rope_out + t * p.rope_out_stride;
        StoreChunk(dst + 8 * j, y1);
        StoreChunk(dst + 32 + 8 * j, y2);
      }
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
      const int64_t t = t0 + r;
      const int slot = __shfl_sync(0xffffffffu, my_slot, r);
      if (t >= rows) continue;  // warp-uniform
      const uint32_t xw[8] = {static_cast<uint32_t>(xa[r].x), static_cast<uint32_t>(xa[r].y), static_cast<uint32_t>(xa[r].z),
                              static_cast<uint32_t>(xa[r].w), static_cast<uint32_t>(xb[r].x), static_cast<uint32_t>(xb[r].y),
                              static_cast<uint32_t>(xb[r].z), static_cast<uint32_t>(xb[r].w)};
      float a = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float lo = Bf16Bits(xw[w], 0), hi = Bf16Bits(xw[w], 1);
        a = __fmaf_rn(lo, lo, a);
        a = __fmaf_rn(hi, hi, a);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, off));
      const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(a, 1.0f / 512.0f), p.eps)));
      uint32_t yw[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float lo = __fmul_rn(__fmul_rn(Bf16Bits(xw[w], 0), rstd), Bf16Bits(gw[w], 0));
        const float hi = __fmul_rn(__fmul_rn(Bf16Bits(xw[w], 1), rstd), Bf16Bits(gw[w], 1));
        yw[w] = PackBf16(lo, hi);
      }
      const int4 ya = make_int4(yw[0], yw[1], yw[2], yw[3]), yb = make_int4(yw[4], yw[5], yw[6], yw[7]);
      if (p.latent_out != nullptr) {
        __nv_bfloat16* dst = p.latent_out + t * p.latent_out_stride;
        *reinterpret_cast<int4*>(dst + 8 * lane) = ya;
        *reinterpret_cast<int4*>(dst + 256 + 8 * lane) = yb;
      }
      if (p.rstd_out != nullptr && lane == 0) p.rstd_out[t] = rstd;
      if (slot >= p.pool.pool_rows) {
        if (lane == 0) RecordError(p.status, B200KV_DEV_BAD_SLOT, static_cast<int32_t>(t), slot);
      } else if (slot >= 0) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.pool.latent) + static_cast<int64_t>(slot) * p.pool.latent_row_stride;
        StoreStream16(dst + 8 * lane, ya);
        StoreStream16(dst + 256 + 8 * lane, yb);
      }
    }
  }
}

// A warp takes 32 consecutive blocks of a row (2 KB): lane l loads the 16-byte chunks l, l + 32, l + 64 and
// l + 96 of that span, so loads and stores are contiguous across the warp; a block's four chunks sit in four
// neighbouring lanes, which agree on the block's maximum with two shuffles.
__global__ void __launch_bounds__(256)
    MxQuantKernel(const __nv_bfloat16* x, int64_t x_stride, int64_t rows, int64_t blocks_per_row, uint8_t* q,
                  int64_t q_stride, uint8_t* scales, int64_t scale_stride) {
  GridDependencyTrigger();
  GridDependencyWait();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t spans_per_row = (blocks_per_row + 31) / 32;
  for (int64_t item = warp; item < rows * spans_per_row; item += n_warps) {
    const int64_t r = item / spans_per_row, first_block = (item % spans_per_row) * 32;
    const __nv_bfloat16* src = x + r * x_stride + 32 * first_block;
    const int64_t chunks = (blocks_per_row - first_block < 32 ? blocks_per_row - first_block : 32) * 4;
    int4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k;
      v[k] = c < chunks ? LoadStream16(src + 8 * c) : make_int4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k;
      const uint32_t w[4] = {static_cast<uint32_t>(v[k].x), static_cast<uint32_t>(v[k].y), static_cast<uint32_t>(v[k].z),
                             static_cast<uint32_t>(v[k].w)};
      float amax = 0.0f;
      int nan = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = fabsf(Bf16Bits(w[i], 0)), hi = fabsf(Bf16Bits(w[i], 1));
        nan |= (lo != lo || hi != hi) ? 1 : 0;
        amax = fmaxf(amax, fmaxf(lo, hi));
      }
#pragma unroll
      for (int off = 1; off <= 2; off <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        nan |= __shfl_xor_sync(0xffffffffu, nan, off);
      }
      uint32_t out[2];
      const MxScale block = MxScaleOf(amax, nan != 0);
      const uint8_t scale = static_cast<uint8_t>(block.code);
      if (nan) {
        out[0] = (((w[0] >> 8) & 0x80u) | 0x7fu) | ((((w[0] >> 24) & 0x80u) | 0x7fu) << 8) |
                 ((((w[1] >> 8) & 0x80u) | 0x7fu) << 16) | ((((w[1] >> 24) & 0x80u) | 0x7fu) << 24);
        out[1] = (((w[2] >> 8) & 0x80u) | 0x7fu) | ((((w[2] >> 24) & 0x80u) | 0x7fu) << 8) |
                 ((((w[3] >> 8) & 0x80u) | 0x7fu) << 16) | ((((w[3] >> 24) & 0x80u) | 0x7fu) << 24);
      } else {
        const float inv = block.inv;
        uint32_t b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          b[i] = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(Bf16Bits(w[i], 0), inv), __fmul_rn(Bf16Bits(w[i], 1), inv)),
                                          __NV_SATFINITE, __NV_E4M3);
        }
        out[0] = b[0] | (b[1] << 16);
        out[1] = b[2] | (b[3] << 16);
      }
      if (c < chunks) {
        *reinterpret_cast<uint2*>(q + r * q_stride + 32 * first_block + 8 * c) = make_uint2(out[0], out[1]);
        if ((c & 3) == 0) scales[r * scale_stride + first_block + (c >> 2)] = scale;
      }
    }
  }
}

bool Aligned(const void* p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; }

int32_t LaunchProducer(const ProducerParams& p, void* stream, const char* what) {
  const int64_t items = (p.kv_a != nullptr ? (p.tokens + kRowsPerPass - 1) / kRowsPerPass : 0) +
                        (p.q_rope != nullptr ? (p.tokens * p.heads + 7) / 8 : 0);
  const int64_t want = (items + kWarpsPerCta - 1) / kWarpsPerCta;
  const int64_t cap = static_cast<int64_t>(CurrentDeviceSmCount()) * 8;
  const int grid = static_cast<int>(want < cap ? want : cap);
  return CheckCuda(LaunchOverlapped(ProducerKernel, dim3(grid), dim3(kWarpsPerCta * 32), 0,
                                    static_cast<cudaStream_t>(stream), p),
                   what);
}

}  // namespace

int32_t ValidatePoolView(const b200kv_pool_view* pool);

}  // namespace b200kv

using namespace b200kv;

extern "C" int32_t b200kv_append_fused(const b200kv_producer_args* args, void* stream, b200kv_status_word* status) {
  if (int32_t rc = FaultCheck("b200kv_append_fused")) return rc;
  if (args == nullptr) {
    SetLastError("append_fused: args is null");
    return B200KV_ERR_NULLPTR;
  }
  const b200kv_producer_args& a = *args;
  if (int32_t rc = ValidatePoolView(&a.pool)) return rc;
  if (a.n_tokens == 0) return B200KV_OK;
  if (a.kv_a == nullptr || a.gamma == nullptr || a.cos == nullptr || a.sin == nullptr || a.slot_mapping == nullptr) {
    SetLastError("append_fused: kv_a, gamma, cos, sin and slot_mapping must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (a.n_tokens < 0 || !(a.eps >= 0.0f) || a.kv_a_stride < B200KV_LATENT_DIM + B200KV_ROPE_DIM || a.kv_a_stride % 8 != 0 ||
      !Aligned(a.kv_a, 16) || !Aligned(a.gamma, 16) || a.cos_stride < 0 || a.sin_stride < 0 || a.cos_stride % 8 != 0 ||
      a.sin_stride % 8 != 0 || !Aligned(a.cos, 16) || !Aligned(a.sin, 16) || a.pool.rope_row_stride % 8 != 0 ||
      (a.q_rope != nullptr && (a.heads <= 0 || a.q_head_stride < B200KV_ROPE_DIM || a.q_head_stride % 8 != 0 ||
                               a.q_token_stride % 8 != 0 || !Aligned(a.q_rope, 16))) ||
      (a.latent_out != nullptr && (!Aligned(a.latent_out, 16) || a.latent_out_stride % 8 != 0 ||
                                   a.latent_out_stride < B200KV_LATENT_DIM)) ||
      (a.rope_out != nullptr && (a.rope_out_stride < B200KV_ROPE_DIM || a.rope_out_stride % 8 != 0 ||
                                 !Aligned(a.rope_out, 16)))) {
    SetLastError("append_fused refused: n_tokens %lld, eps %g, kv_a stride %lld (>= 576), heads %d; every tensor needs a "
                 "16-byte aligned base and strides that are multiples of 8 elements",
                 static_cast<long long>(a.n_tokens), static_cast<double>(a.eps), static_cast<long long>(a.kv_a_stride),
                 a.heads);
    return B200KV_ERR_INVALID;
  }
  ProducerParams p{};
  p.pool = a.pool;
  p.kv_a = static_cast<const __nv_bfloat16*>(a.kv_a);
  p.kv_a_stride = a.kv_a_stride;
  p.gamma = static_cast<const __nv_bfloat16*>(a.gamma);
  p.eps = a.eps;
  p.cos = static_cast<const __nv_bfloat16*>(a.cos);
  p.cos_stride = a.cos_stride;
  p.sin = static_cast<const __nv_bfloat16*>(a.sin);
  p.sin_stride = a.sin_stride;
  p.slots = a.slot_mapping;
  p.tokens = a.n_tokens;
  p.q_rope = static_cast<__nv_bfloat16*>(a.q_rope);
  p.q_token_stride = a.q_token_stride;
  p.q_head_stride = a.q_head_stride;
  p.heads = a.heads;
  p.latent_out = static_cast<__nv_bfloat16*>(a.latent_out);
  p.latent_out_stride = a.latent_out_stride;
  p.rope_out = static_cast<__nv_bfloat16*>(a.rope_out);
  p.rope_out_stride = a.rope_out_stride;
  p.rstd_out = a.rstd_out;
  p.status = status;
  return LaunchProducer(p, stream, "append_fused launch");
}

extern "C" int32_t b200kv_rmsnorm512(const void* x, int64_t x_stride, const void* gamma, float eps, int64_t rows, void* y,
                                     int64_t y_stride, float* rstd, void* stream) {
  if (rows == 0) return B200KV_OK;
  if (x == nullptr || gamma == nullptr || y == nullptr) {
    SetLastError("rmsnorm512: x, gamma and y must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (rows < 0 || !(eps >= 0.0f) || x_stride < B200KV_LATENT_DIM || x_stride % 8 != 0 || y_stride < B200KV_LATENT_DIM ||
      y_stride % 8 != 0 || !Aligned(x, 16) || !Aligned(y, 16) || !Aligned(gamma, 16)) {
    SetLastError("rmsnorm512 refused: rows %lld, strides %lld/%lld (multiples of 8, >= 512), 16-byte aligned x, gamma, y",
                 static_cast<long long>(rows), static_cast<long long>(x_stride), static_cast<long long>(y_stride));
    return B200KV_ERR_INVALID;
  }
  ProducerParams p{};
  p.kv_a = static_cast<const __nv_bfloat16*>(x);
  p.kv_a_stride = x_stride;
  p.gamma = static_cast<const __nv_bfloat16*>(gamma);
  p.eps = eps;
  p.tokens = rows;
  p.latent_out = static_cast<__nv_bfloat16*>(y);
  p.latent_out_stride = y_stride;
  p.rstd_out = rstd;
  return LaunchProducer(p, stream, "rmsnorm512 launch");
}

extern "C" int32_t b200kv_rope_half64(void* x, int64_t token_stride, int64_t vector_stride, const void* cos,
                                      int64_t cos_stride, const void* sin, int64_t sin_stride, int64_t tokens,
                                      int32_t vectors, void* stream) {
  if (tokens == 0 || vectors == 0) return B200KV_OK;
  if (x == nullptr || cos == nullptr || sin == nullptr) {
    SetLastError("rope_half64: x, cos and sin must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (tokens < 0 || vectors < 0 || vector_stride < B200KV_ROPE_DIM || cos_stride < 0 || sin_stride < 0 ||
      vector_stride % 8 != 0 || token_stride % 8 != 0 || cos_stride % 8 != 0 || sin_stride % 8 != 0 || !Aligned(x, 16) ||
      !Aligned(cos, 16) || !Aligned(sin, 16)) {
    SetLastError("rope_half64 refused: tokens %lld, vectors %d, vector stride %lld (>= 64); x, cos and sin need 16-byte "
                 "aligned bases and strides that are multiples of 8 elements",
                 static_cast<long long>(tokens), vectors, static_cast<long long>(vector_stride));
    return B200KV_ERR_INVALID;
  }
  ProducerParams p{};
  p.cos = static_cast<const __nv_bfloat16*>(cos);
  p.cos_stride = cos_stride;
  p.sin = static_cast<const __nv_bfloat16*>(sin);
  p.sin_stride = sin_stride;
  p.tokens = tokens;
  p.q_rope = static_cast<__nv_bfloat16*>(x);
  p.q_token_stride = token_stride;
  p.q_head_stride = vector_stride;
  p.heads = vectors;
  return LaunchProducer(p, stream, "rope_half64 launch");
}

extern "C" int32_t b200kv_mx_quant_e4m3(const void* x, int64_t x_stride, int64_t rows, int64_t cols, void* q,
                                        int64_t q_stride, void* scales, int64_t scale_stride, void* stream) {
  if (int32_t rc = FaultCheck("b200kv_mx_quant_e4m3")) return rc;
  if (rows == 0 || cols == 0) return B200KV_OK;
  if (x == nullptr || q == nullptr || scales == nullptr) {
    SetLastError("mx_quant_e4m3: x, q and scales must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (rows < 0 || cols < 0 || cols % 32 != 0 || x_stride < cols || x_stride % 8 != 0 || q_stride < cols ||
      q_stride % 16 != 0 || scale_stride < cols / 32 || !Aligned(x, 16) || !Aligned(q, 16)) {
    SetLastError("mx_quant_e4m3 refused: rows %lld, cols %lld (multiple of 32), strides %lld/%lld/%lld, x and q 16-byte "
                 "aligned with strides that keep every block of 32 aligned",
                 static_cast<long long>(rows), static_cast<long long>(cols), static_cast<long long>(x_stride),
                 static_cast<long long>(q_stride), static_cast<long long>(scale_stride));
    return B200KV_ERR_INVALID;
  }
  const int64_t total = rows * ((cols / 32 + 31) / 32);  // warp items: spans of 32 blocks
  const int64_t want = (total + 7) / 8;
  const int64_t cap = static_cast<int64_t>(CurrentDeviceSmCount()) * 8;
  const int grid = static_cast<int>(want < cap ? want : cap);
  return CheckCuda(LaunchOverlapped(MxQuantKernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                    static_cast<const __nv_bfloat16*>(x), x_stride, rows, cols / 32,
                                    static_cast<uint8_t*>(q), q_stride, static_cast<uint8_t*>(scales), scale_stride),
                   "mx_quant_e4m3 launch");
}
