// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention: a serving
// loop that has sealed its arena (the reference engine refuses every allocation after Seal and asserts
// zero allocations per decode step), a plugin that runs inside another runtime's memory budget, or code
// that is not allowed to touch the allocator at all. b200kv_mla_decode needs a caller-provided workspace;
// this variant carries its own, a fixed array in the library's device image, so the caller passes only
// inputs and outputs. The array is part of the loaded module: every GPU that loads the library holds
// kStaticScratchBytes of it until the process exits.
#include "common.cuh"

namespace b200kv {
bool TcSupports(const b200kv_decode_args& a);
size_t TcWorkspaceBytes(int32_t n_ctas);
int32_t LaunchMlaDecodeTc(const b200kv_decode_args& a, int32_t n_ctas, cudaStream_t stream, int32_t* status);
int32_t ValidatePoolView(const b200kv_pool_view* pool);
}  // namespace b200kv

using namespace b200kv;

namespace {

// Two partial slots per CTA of 64 heads x (512 + 2) fp32: 263,168 bytes per CTA, 32 CTAs at most.
constexpr int kStaticMaxCtas = B200KV_STATIC_MAX_CTAS;
constexpr size_t kStaticScratchBytes = static_cast<size_t>(kStaticMaxCtas) * 2 * 64 * (512 + 2) * sizeof(float);

// In host code this name is only a handle for the runtime's symbol lookup, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_address[kMaxDevices] = {};  // per device, filled by the first call on that device

// Resolves the array's device address for the current device (once per device).
int32_t ScratchForCurrentDevice(void** out) {
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device < 0 || device >= kMaxDevices) {
    SetLastError("mla_decode_static: device ordinal %d outside [0, %d)", device, kMaxDevices);
    return B200KV_ERR_INVALID;
  }
  if (g_scratch_address[device] == nullptr) {
    void* ptr = nullptr;
    if (int32_t rc = CheckCuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)")) {
      return rc;
    }
    g_scratch_address[device] = ptr;
  }
  *out = g_scratch_address[device];
  return B200KV_OK;
}

}  // namespace

extern "C" size_t b200kv_mla_decode_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int32_t b200kv_mla_decode_static(const b200kv_decode_args* args, void* stream,
                                            b200kv_status_word* status) {
  if (args == nullptr) {
    SetLastError("mla_decode_static: args is null");
    return B200KV_ERR_NULLPTR;
  }
  b200kv_decode_args a = *args;
  if (int32_t rc = ValidatePoolView(&a.pool)) return rc;
  if (a.batch == 0) return B200KV_OK;
  const bool want_partial = a.partial_o != nullptr || a.partial_m != nullptr || a.partial_l != nullptr;
  if (a.q == nullptr || a.block_table == nullptr || a.kv_len == nullptr ||
      (want_partial && (a.partial_o == nullptr || a.partial_m == nullptr || a.partial_l == nullptr)) ||
      (!want_partial && a.out == nullptr)) {
    SetLastError("mla_decode_static: q, block_table, kv_len and either out or all three partial_* must be non-null");
    return B200KV_ERR_NULLPTR;
  }
  if (a.batch < 0 || a.block_size <= 0 || a.max_blocks <= 0 || a.pool.pool_rows % a.block_size != 0 ||
      !(a.scale > 0.0f) || !TcSupports(a)) {
    SetLastError("mla_decode_static refused: it runs the tensor-core kernel only (64 heads, block_size %% 64 == 0, "
                 "16-byte aligned q with strides that are multiples of 8 elements); batch %d heads %d block_size %d",
                 a.batch, a.heads, a.block_size);
    return B200KV_ERR_INVALID;
  }
  const int32_t ctas = a.max_ctas > 0 ? a.max_ctas : kStaticMaxCtas;
  if (ctas > kStaticMaxCtas || TcWorkspaceBytes(ctas) > kStaticScratchBytes) {
    SetLastError("mla_decode_static: %d CTAs need %zu bytes of scratch, the built-in array holds %zu (at most %d "
                 "CTAs); use b200kv_mla_decode with a caller workspace for wider grids",
                 ctas, TcWorkspaceBytes(ctas), kStaticScratchBytes, kStaticMaxCtas);
    return B200KV_ERR_INVALID;
  }
  void* scratch = nullptr;
  if (int32_t rc = ScratchForCurrentDevice(&scratch)) return rc;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchBytes;
  a.variant = B200KV_DECODE_TCGEN05;
  // Nothing in the scratch has to start at zero: every partial slot a launch reads was written by the
  // same launch's decode kernel first.
  return LaunchMlaDecodeTc(a, ctas, static_cast<cudaStream_t>(stream), status);
}
