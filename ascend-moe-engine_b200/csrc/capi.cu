// C-ABI entry points that are not pure kernel launches: error text, decode dispatch, merge, and the
// seeded device-side generator.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"
#include "kv_peer.cuh"

namespace b200kv {

namespace {
thread_local char g_error[512] = "";
}

void SetLastError(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

// ---- host-side fault injection -------------------------------------------------------------------------
// Tests of failure handling make a named entry point fail BEFORE it reaches the device, as the reference's
// stand-in runtime does (mock/runtime_faults.cpp:8-23: FailRuntimeCall(name, calls) lets `calls` calls of that
// name through and fails the next). Nothing on the GPU is ever made to fault. Off unless armed: one relaxed
// load per call.
namespace {
std::atomic<bool> g_fault_armed{false};
std::mutex g_fault_mutex;
std::string g_fault_name;
int32_t g_fault_remaining = 0;
int64_t g_fault_fired = 0;
}  // namespace

int32_t FaultCheck(const char* entry_point) {
  if (!g_fault_armed.load(std::memory_order_relaxed)) return B200KV_OK;
  std::lock_guard<std::mutex> lock(g_fault_mutex);
  if (g_fault_name != entry_point) return B200KV_OK;
  if (g_fault_remaining-- > 0) return B200KV_OK;
  g_fault_armed.store(false, std::memory_order_relaxed);
  g_fault_name.clear();
  ++g_fault_fired;
  SetLastError("injected failure: %s", entry_point);
  return B200KV_ERR_RUNTIME;
}

int32_t CheckCuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return B200KV_OK;
  SetLastError("%s: %s (%s)", what, cudaGetErrorString(err), cudaGetErrorName(err));
  return B200KV_ERR_RUNTIME;
}

int32_t ValidatePoolView(const b200kv_pool_view* pool);
int32_t SimtSplitCount(int32_t batch, int32_t sms);
size_t SimtWorkspaceBytes(int32_t batch, int32_t heads, int32_t sms);
size_t TcWorkspaceBytes(int32_t n_ctas);
bool TcSupports(const b200kv_decode_args& a);
bool TcPeerSupports(const b200kv_decode_args& a);
int32_t LaunchMlaDecodeSimt(const b200kv_decode_args& a, cudaStream_t stream, int32_t* status);
int32_t LaunchMlaDecodeTc(const b200kv_decode_args& a, int32_t n_ctas, cudaStream_t stream, int32_t* status,
                          const PeerRing* ring);
int32_t LaunchLseMerge(const float* part_o, const float* part_m, const float* part_l, int32_t n_parts, int64_t rows,
                       void* out, float* lse, float* merged_o, float* merged_m, float* merged_l, cudaStream_t stream);

namespace {

constexpr unsigned long long kGolden = 0x9E3779B97F4A7C15ull;

__host__ __device__ inline unsigned long long Mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// One thread per pair of elements: the two Box-Muller outputs of one (u1, u2) draw.
__global__ void FillNormalKernel(__nv_bfloat16* dst, int64_t count, unsigned long long key,
                                 unsigned long long first_element, double scale) {
  const unsigned long long first_pair = first_element >> 1;
  const unsigned long long last_pair = (first_element + static_cast<unsigned long long>(count) - 1) >> 1;
  const unsigned long long n_pairs = last_pair - first_pair + 1;
  for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs;
       i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const unsigned long long pair = first_pair + i;
    const double u1 = static_cast<double>((Mix64(key + (2 * pair + 1) * kGolden) >> 11) + 1) * 0x1.0p-53;
    const double u2 = static_cast<double>(Mix64(key + (2 * pair + 2) * kGolden) >> 11) * 0x1.0p-53;
    const double radius = sqrt(-2.0 * log(u1));
    const double angle = 6.283185307179586476925286766559 * u2;
    const unsigned long long e0 = 2 * pair;
    if (e0 >= first_element) {
      dst[e0 - first_element] = __float2bfloat16_rn(static_cast<float>(radius * cos(angle) * scale));
    }
    if (e0 + 1 >= first_element && e0 + 1 < first_element + static_cast<unsigned long long>(count)) {
      dst[e0 + 1 - first_element] = __float2bfloat16_rn(static_cast<float>(radius * sin(angle) * scale));
    }
  }
}

}  // namespace
}  // namespace b200kv

namespace b200kv {

// The argument refusals every decode entry point shares (pointers, sizes, strides, variant).
int32_t ValidateDecodeArgs(const b200kv_decode_args& a, const char* who) {
  if (int32_t rc = ValidatePoolView(&a.pool)) return rc;
  if (a.batch == 0) return B200KV_OK;
  const bool want_partial = a.partial_o != nullptr || a.partial_m != nullptr || a.partial_l != nullptr;
  if (a.q == nullptr || (a.block_table == nullptr && a.row_index == nullptr) || a.kv_len == nullptr ||
      (want_partial && (a.partial_o == nullptr || a.partial_m == nullptr || a.partial_l == nullptr)) ||
      (!want_partial && a.out == nullptr)) {
    SetLastError("%s: q, block_table (or row_index), kv_len and either out or all three partial_* buffers must be non-null", who);
    return B200KV_ERR_NULLPTR;
  }
  if (a.row_index != nullptr) {
    if (a.row_index_stride <= 0 || a.kv_begin != nullptr || a.new_latent != nullptr || a.new_rope != nullptr) {
      SetLastError("%s refused: row_index wants a positive row_index_stride (%lld given), no kv_begin and no fused append",
                   who, static_cast<long long>(a.row_index_stride));
      return B200KV_ERR_INVALID;
    }
  }
  if ((a.out_fp8 == nullptr) != (a.out_scale == nullptr) || (a.out_fp8 != nullptr && (want_partial || a.heads != B200KV_HEADS))) {
    SetLastError("%s refused: out_fp8 and out_scale come together, with out (not partial_*) and 64 heads", who);
    return B200KV_ERR_INVALID;
  }
  const bool table_ok = a.row_index != nullptr ||
                        (a.block_size > 0 && a.max_blocks > 0 && a.pool.pool_rows % a.block_size == 0);
  if (a.batch < 0 || a.heads <= 0 || !table_ok ||
      !(a.scale > 0.0f) || a.q_head_stride < B200KV_LATENT_DIM + B200KV_ROPE_DIM || a.q_head_stride % 2 != 0 ||
      a.q_seq_stride % 2 != 0 || (a.batch > 1 && a.q_seq_stride < 0) || (reinterpret_cast<uintptr_t>(a.q) & 3u) != 0 ||
      (a.variant != B200KV_DECODE_AUTO && a.variant != B200KV_DECODE_SIMT && a.variant != B200KV_DECODE_TCGEN05)) {
    SetLastError("%s refused: batch %d heads %d block_size %d max_blocks %lld scale %g q strides %lld/%lld variant %d",
                 who, a.batch, a.heads, a.block_size, static_cast<long long>(a.max_blocks), static_cast<double>(a.scale),
                 static_cast<long long>(a.q_seq_stride), static_cast<long long>(a.q_head_stride), a.variant);
    return B200KV_ERR_INVALID;
  }
  return B200KV_OK;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" const char* b200kv_last_error(void) { return g_error; }

extern "C" int32_t b200kv_fault_inject(const char* entry_point, int32_t after_calls) {
  if (entry_point == nullptr || after_calls < 0) {
    SetLastError("fault_inject: a name and a count of calls to let through (>= 0)");
    return entry_point == nullptr ? B200KV_ERR_NULLPTR : B200KV_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lock(g_fault_mutex);
  g_fault_name = entry_point;
  g_fault_remaining = after_calls;
  g_fault_armed.store(true, std::memory_order_relaxed);
  return B200KV_OK;
}

extern "C" int64_t b200kv_fault_clear(void) {
  std::lock_guard<std::mutex> lock(g_fault_mutex);
  g_fault_armed.store(false, std::memory_order_relaxed);
  g_fault_name.clear();
  const int64_t fired = g_fault_fired;
  g_fault_fired = 0;
  return fired;
}

extern "C" int32_t b200kv_abi_version(void) { return 6; }

extern "C" size_t b200kv_mla_decode_workspace_bytes(int32_t batch, int32_t heads, int32_t max_ctas) {
  if (batch <= 0 || heads <= 0) return 0;
  const int32_t sms = CurrentDeviceSmCount();
  const int32_t ctas = max_ctas > 0 ? max_ctas : sms;
  const size_t simt = SimtWorkspaceBytes(batch, heads, sms);
  const size_t tc = TcWorkspaceBytes(ctas);
  return (simt > tc ? simt : tc) + 256;
}

extern "C" int32_t b200kv_mla_decode(const b200kv_decode_args* args, void* stream, b200kv_status_word* status) {
  if (args == nullptr) {
    SetLastError("decode: args is null");
    return B200KV_ERR_NULLPTR;
  }
  const b200kv_decode_args& a = *args;
  if (int32_t rc = FaultCheck("b200kv_mla_decode")) return rc;
  if (int32_t rc = ValidateDecodeArgs(a, "decode")) return rc;
  if (a.batch == 0) return B200KV_OK;
  const bool tc_ok = TcSupports(a);
  if (a.variant == B200KV_DECODE_TCGEN05 && !tc_ok) {
    SetLastError("decode: the tcgen05 kernel needs 64 heads, block_size %% 64 == 0 (or row_index), 16-byte aligned q "
                 "with strides that are multiples of 8 elements");
    return B200KV_ERR_INVALID;
  }
  const bool use_tc = a.variant == B200KV_DECODE_TCGEN05 || (a.variant == B200KV_DECODE_AUTO && tc_ok);
  if ((a.new_latent != nullptr || a.new_rope != nullptr) && !use_tc) {
    SetLastError("decode: the fused append runs in the tcgen05 kernel only");
    return B200KV_ERR_INVALID;
  }
  const int32_t sms = CurrentDeviceSmCount();
  const int32_t ctas = a.max_ctas > 0 ? a.max_ctas : sms;
  const size_t need = use_tc ? TcWorkspaceBytes(ctas) : (SimtSplitCount(a.batch, sms) > 1 ? SimtWorkspaceBytes(a.batch, a.heads, sms) : 0);
  if (need > 0 && (a.workspace == nullptr || a.workspace_bytes < need ||
                   (reinterpret_cast<uintptr_t>(a.workspace) & 15u) != 0)) {
    SetLastError("decode: workspace of %zu bytes (16-byte aligned) required, %zu given", need, a.workspace_bytes);
    return a.workspace == nullptr ? B200KV_ERR_NULLPTR : B200KV_ERR_INVALID;
  }
  if (use_tc) return LaunchMlaDecodeTc(a, ctas, static_cast<cudaStream_t>(stream), status, nullptr);
  b200kv_decode_args simt = a;
  if (a.row_index != nullptr) {  // the CUDA-core kernel reads a row list as a table of single-row blocks
    simt.block_table = a.row_index;
    simt.max_blocks = a.row_index_stride;
    simt.block_size = 1;
    simt.row_index = nullptr;
  }
  if (int32_t rc = LaunchMlaDecodeSimt(simt, static_cast<cudaStream_t>(stream), status)) return rc;
  if (a.out_fp8 == nullptr) return B200KV_OK;
  const int64_t cols = static_cast<int64_t>(a.heads) * B200KV_LATENT_DIM;
  return b200kv_mx_quant_e4m3(a.out, cols, a.batch, cols, a.out_fp8, cols, a.out_scale, cols / 32, stream);
}

extern "C" int32_t b200kv_mla_decode_peer(const b200kv_decode_args* args, void* const* peer_buffers, int32_t world,
                                          int32_t rank, void* stream, b200kv_status_word* status) {
  if (args == nullptr || peer_buffers == nullptr) {
    SetLastError("decode_peer: args and peer_buffers must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  const b200kv_decode_args& a = *args;
  if (int32_t rc = FaultCheck("b200kv_mla_decode_peer")) return rc;
  if (int32_t rc = ValidateDecodeArgs(a, "decode_peer")) return rc;
  if (a.batch == 0) return B200KV_OK;
  if (a.out == nullptr || a.partial_o != nullptr || world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world ||
      a.new_latent != nullptr || a.new_rope != nullptr) {
    SetLastError("decode_peer refused: it writes the merged result to out (no partial_* buffers, no fused append); "
                 "world %d (1..%d), rank %d", world, kPeerMaxWorld, rank);
    return B200KV_ERR_INVALID;
  }
  if (!TcSupports(a) || !TcPeerSupports(a) || a.variant == B200KV_DECODE_SIMT) {
    SetLastError("decode_peer: it runs on the tensor-core kernel (64 heads, block_size %% 64 == 0, 16-byte aligned q) for "
                 "batches of fewer than 16 sequences; otherwise decode into partial_* and call b200kv_peer_merge");
    return B200KV_ERR_INVALID;
  }
  PeerRing ring{};
  for (int r = 0; r < world; ++r) {
    if (peer_buffers[r] == nullptr) {
      SetLastError("decode_peer: the exchange buffer of rank %d is null", r);
      return B200KV_ERR_NULLPTR;
    }
    ring.peer[r] = static_cast<unsigned char*>(peer_buffers[r]);
  }
  ring.world = world;
  ring.rank = rank;
  ring.rows = static_cast<int64_t>(a.batch) * a.heads;
  const int32_t ctas = a.max_ctas > 0 ? a.max_ctas : CurrentDeviceSmCount();
  const size_t need = TcWorkspaceBytes(ctas);
  if (a.workspace == nullptr || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 15u) != 0) {
    SetLastError("decode_peer: workspace of %zu bytes (16-byte aligned) required, %zu given", need, a.workspace_bytes);
    return a.workspace == nullptr ? B200KV_ERR_NULLPTR : B200KV_ERR_INVALID;
  }
  return LaunchMlaDecodeTc(a, ctas, static_cast<cudaStream_t>(stream), status, &ring);
}

extern "C" int32_t b200kv_lse_merge(const float* partial_o, const float* partial_m, const float* partial_l,
                                    int32_t n_parts, int64_t rows, void* out_bf16, float* lse, void* stream) {
  if (int32_t rc = FaultCheck("b200kv_lse_merge")) return rc;
  if (rows == 0) return B200KV_OK;
  if (partial_o == nullptr || partial_m == nullptr || partial_l == nullptr || out_bf16 == nullptr) {
    SetLastError("lse_merge: partial buffers and out must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (n_parts <= 0 || rows < 0 || (reinterpret_cast<uintptr_t>(partial_o) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(out_bf16) & 7u) != 0) {
    SetLastError("lse_merge refused: n_parts %d rows %lld (partial_o 16-byte, out 8-byte aligned)", n_parts,
                 static_cast<long long>(rows));
    return B200KV_ERR_INVALID;
  }
  return LaunchLseMerge(partial_o, partial_m, partial_l, n_parts, rows, out_bf16, lse, nullptr, nullptr, nullptr,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int32_t b200kv_fill_normal_bf16(void* dst, int64_t count, uint64_t seed, uint64_t stream_id,
                                           uint64_t first_element, double scale, void* stream) {
  if (count == 0) return B200KV_OK;
  if (dst == nullptr) {
    SetLastError("fill_normal_bf16: dst is null");
    return B200KV_ERR_NULLPTR;
  }
  if (count < 0) {
    SetLastError("fill_normal_bf16: negative count");
    return B200KV_ERR_INVALID;
  }
  const unsigned long long key = Mix64(seed ^ (stream_id * kGolden + kGolden));
  const int64_t pairs = count / 2 + 2;
  int64_t ctas = (pairs + 255) / 256;
  const int64_t cap = static_cast<int64_t>(CurrentDeviceSmCount()) * 16;
  if (ctas > cap) ctas = cap;
  FillNormalKernel<<<static_cast<unsigned>(ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(dst), count, key, first_element, scale);
  return CheckCuda(cudaGetLastError(), "fill launch");
}
