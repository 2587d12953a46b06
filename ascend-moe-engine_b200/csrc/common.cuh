// Shared device/host helpers for the KV-cache path kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200kv.h"

namespace b200kv {

// Host: per-thread error text behind b200kv_last_error().
void SetLastError(const char* fmt, ...);
int32_t CheckCuda(cudaError_t err, const char* what);
// Host-side fault injection (b200kv_fault_inject): B200KV_ERR_RUNTIME when this call of `entry_point` is the one a
// test asked to fail, before anything reaches the device; B200KV_OK otherwise.
int32_t FaultCheck(const char* entry_point);

// Device: record the first error in the caller's status word and carry on. Kernels never trap:
// the failing access is skipped and the host reads the word after its next synchronisation.
__device__ __forceinline__ void RecordError(int32_t* status, int32_t code, int32_t d0, int32_t d1, int32_t d2 = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = d0;
    status[2] = d1;
    status[3] = d2;
  }
}

__device__ __forceinline__ int4 LoadStream16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void StoreStream16(void* p, int4 v) {
  asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// MX (block-32) quantisation to FP8 E4M3 with an E8M0 scale, the arithmetic of the reference's attn_quant stage
// (src/pipeline/pipeline.cpp:250-258) as every kernel of this library that quantises applies it. A block's scale
// is 2^e, e = floor(log2 amax) - 8 clamped to [-127, 127] and stored as e + 127; a block that holds a NaN gets
// scale 0xff and every value of it the code sign | 0x7f.
struct MxScale {
  uint32_t code;  // the E8M0 byte
  float inv;      // 2^-e
};
__device__ __forceinline__ MxScale MxScaleOf(float amax, bool has_nan) {
  MxScale s;
  if (has_nan) {
    s.code = 0xffu;
    s.inv = 0.0f;
    return s;
  }
  // floor(log2 amax) from the exponent field: a subnormal maximum (field 0) is below 2^-126, where the
  // clamp to -127 applies anyway, and an infinite one (field 255) takes the upper clamp.
  const int field = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);
  int e = field == 0 ? -127 : (field == 255 ? 127 : field - 127 - 8);
  e = e < -127 ? -127 : e;
  s.code = static_cast<uint32_t>(e + 127);
  // 2^-e as a float (2^-127 is the subnormal 0x00400000); the product is exact wherever it matters:
  // it can only round where the result is far below the smallest FP8 value, and overflow saturates.
  s.inv = __uint_as_float(e == 127 ? 0x00400000u : static_cast<uint32_t>(127 - e) << 23);
  return s;
}

// Programmatic dependent launch: a kernel launched with LaunchOverlapped may be scheduled while its
// predecessor in the stream is still draining; it must call GridDependencyWait() before it reads anything
// the predecessor wrote. A kernel lets its successor start early with GridDependencyTrigger(). Both are
// no-ops for ordinary launches.
__device__ __forceinline__ void GridDependencyWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void GridDependencyTrigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KernelArgs, typename... Args>
inline cudaError_t LaunchOverlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

inline int32_t CurrentDeviceSmCount() {
  static thread_local int cached_device = -1;
  static thread_local int cached_sms = 0;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 148;
  if (device != cached_device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
    cached_device = device;
    cached_sms = sms;
  }
  return cached_sms;
}

}  // namespace b200kv
