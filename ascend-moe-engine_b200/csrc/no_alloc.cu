// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention: a serving
// loop that has sealed its arena (the reference engine refuses every allocation after Seal and asserts
// zero allocations per decode step), a plugin that runs inside another runtime's memory budget, or code
// that is not allowed to touch the allocator at all. b200kv_mla_decode needs a caller-provided workspace;
// this variant carries its own, a fixed array in the library's device image, so the caller passes only
// inputs and outputs. The array is part of the loaded module: every GPU that loads the library holds
// kStaticScratchBytes of it until the process exits.
#include <atomic>

#include "common.cuh"

namespace b200kv {
int32_t ValidateDecodeArgs(const b200kv_decode_args& a, const char* who);
bool TcSupports(const b200kv_decode_args& a);
size_t TcWorkspaceBytes(int32_t n_ctas);
struct PeerRing;
int32_t LaunchMlaDecodeTc(const b200kv_decode_args& a, int32_t n_ctas, cudaStream_t stream, int32_t* status,
                          const PeerRing* ring);
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
std::atomic<void*> g_scratch_address[kMaxDevices];  // per device, filled by the first call on that device

// Resolves the array's device address for the current device (once per device).
int32_t ScratchForCurrentDevice(void** out) {
  int device = 0;
  if (int32_t rc = CheckCuda(cudaGetDevice(&device), "cudaGetDevice")) return rc;
  if (device < 0 || device >= kMaxDevices) {
    SetLastError("mla_decode_static: device ordinal %d outside [0, %d)", device, kMaxDevices);
    return B200KV_ERR_INVALID;
  }
  void* ptr = g_scratch_address[device].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // Threads that get here together each look the address up and store the same value.
    if (int32_t rc = CheckCuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)")) {
      return rc;
    }
    g_scratch_address[device].store(ptr, std::memory_order_release);
  }
  *out = ptr;
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
  a.variant = B200KV_DECODE_TCGEN05;  // the caller's choice is ignored: only the tensor-core kernel runs here
  // The same refusals as b200kv_mla_decode, then the tensor-core kernel's own geometry.
  if (int32_t rc = ValidateDecodeArgs(a, "mla_decode_static")) return rc;
  if (a.batch == 0) return B200KV_OK;
  if (!TcSupports(a)) {
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
  // Nothing in the scratch has to start at zero: every partial slot a launch reads was written by the
  // same launch's decode kernel first.
  return LaunchMlaDecodeTc(a, ctas, static_cast<cudaStream_t>(stream), status, nullptr);
}
