// The reference engine's operator-library ABI (include/b200kv_aclnn.h) on top of the b200kv kernels:
// descriptor handles, the plan / repoint / launch executor protocol, the two operators of the KV path
// in their two-phase form, and the runtime calls as thin wrappers over the CUDA runtime.
//
// Ownership follows the reference's use: the caller owns tensors, lists, arrays, workspaces and
// executors (src/core/op_table.cpp:230-243); a tensor list owns the tensor handles given to it
// (src/memory/static_arena.cpp:175-176); dims and strides are copied at creation. A plan freezes shapes
// and parameters and keeps the caller's tensor handles; aclSetTensorAddr changes a handle's address and
// the next launch uses it (src/pipeline/pipeline.cpp:390-400). No exception leaves this file.
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "aclnn_types.h"
#include "b200kv_aclnn.h"
#include "common.cuh"

using namespace b200kv;

// ---- descriptors --------------------------------------------------------------------------------------
extern "C" aclTensor* aclCreateTensor(const int64_t* view_dims, uint64_t view_dims_num, aclDataType dtype,
                                      const int64_t* view_strides, int64_t storage_offset, aclFormat format,
                                      const int64_t* storage_dims, uint64_t storage_dims_num, void* device_data) {
  if (view_dims == nullptr && view_dims_num > 0) return nullptr;
  auto* t = new (std::nothrow) aclTensor();
  if (t == nullptr) return nullptr;
  t->dims.assign(view_dims, view_dims + view_dims_num);
  if (view_strides != nullptr) {
    t->strides.assign(view_strides, view_strides + view_dims_num);
  } else {
    t->strides.assign(view_dims_num, 1);
    for (int64_t i = static_cast<int64_t>(view_dims_num) - 2; i >= 0; --i) t->strides[i] = t->strides[i + 1] * t->dims[i + 1];
  }
  if (storage_dims != nullptr) {
    t->storage_dims.assign(storage_dims, storage_dims + storage_dims_num);
  } else {
    t->storage_dims = t->dims;  // a tensor described without a storage shape is dense over its view
  }
  t->offset = storage_offset;
  t->dtype = dtype;
  t->format = format;
  t->data = device_data;
  return t;
}
extern "C" aclnnStatus aclDestroyTensor(const aclTensor* tensor) {
  delete tensor;
  return 0;
}
// The three shape getters hand the caller a copy it owns and releases with delete[]: the reference wraps each
// result in std::unique_ptr<int64_t[]> (src/memory/static_arena.cpp:181-188, src/core/matmul_contract.cpp:16-23).
namespace {
aclnnStatus CopyOut(const std::vector<int64_t>& values, int64_t** out, uint64_t* count) {
  int64_t* copy = new (std::nothrow) int64_t[values.size() > 0 ? values.size() : 1];
  if (copy == nullptr) return kErrNull;
  if (!values.empty()) std::memcpy(copy, values.data(), values.size() * sizeof(int64_t));
  *out = copy;
  *count = values.size();
  return 0;
}
}  // namespace
extern "C" aclnnStatus aclGetViewShape(const aclTensor* t, int64_t** dims, uint64_t* count) {
  if (t == nullptr || dims == nullptr || count == nullptr) return kErrNull;
  return CopyOut(t->dims, dims, count);
}
extern "C" aclnnStatus aclGetStorageShape(const aclTensor* t, int64_t** dims, uint64_t* count) {
  if (t == nullptr || dims == nullptr || count == nullptr) return kErrNull;
  return CopyOut(t->storage_dims, dims, count);
}
extern "C" aclnnStatus aclGetViewStrides(const aclTensor* t, int64_t** strides, uint64_t* count) {
  if (t == nullptr || strides == nullptr || count == nullptr) return kErrNull;
  return CopyOut(t->strides, strides, count);
}
extern "C" aclnnStatus aclGetDataType(const aclTensor* t, aclDataType* dtype) {
  if (t == nullptr || dtype == nullptr) return kErrNull;
  *dtype = t->dtype;
  return 0;
}
extern "C" aclnnStatus aclGetFormat(const aclTensor* t, aclFormat* format) {
  if (t == nullptr || format == nullptr) return kErrNull;
  *format = t->format;
  return 0;
}
extern "C" aclnnStatus aclGetRawTensorAddr(const aclTensor* t, void** address) {
  if (t == nullptr || address == nullptr) return kErrNull;
  *address = t->data;
  return 0;
}
extern "C" aclnnStatus aclGetViewOffset(const aclTensor* t, int64_t* offset) {
  if (t == nullptr || offset == nullptr) return kErrNull;
  *offset = t->offset;
  return 0;
}
extern "C" aclTensorList* aclCreateTensorList(const aclTensor* const* tensors, uint64_t size) {
  if (tensors == nullptr && size > 0) return nullptr;
  auto* list = new (std::nothrow) aclTensorList();
  if (list == nullptr) return nullptr;
  for (uint64_t i = 0; i < size; ++i) list->items.push_back(const_cast<aclTensor*>(tensors[i]));
  return list;
}
extern "C" aclnnStatus aclDestroyTensorList(const aclTensorList* list) {
  if (list != nullptr) {
    for (aclTensor* t : list->items) delete t;  // the list owns the handles it was given
    delete list;
  }
  return 0;
}
extern "C" aclIntArray* aclCreateIntArray(const int64_t* value, uint64_t size) {
  if (value == nullptr && size > 0) return nullptr;
  auto* a = new (std::nothrow) aclIntArray();
  if (a != nullptr) a->values.assign(value, value + size);
  return a;
}
extern "C" aclnnStatus aclDestroyIntArray(const aclIntArray* array) {
  delete array;
  return 0;
}
extern "C" aclScalar* aclCreateScalar(void* value, aclDataType dtype) {
  if (value == nullptr) return nullptr;
  auto* s = new (std::nothrow) aclScalar();
  if (s != nullptr) {
    std::memcpy(s->bytes, value, static_cast<size_t>(ElementBytes(dtype)));
    s->dtype = dtype;
  }
  return s;
}
extern "C" aclnnStatus aclDestroyScalar(const aclScalar* scalar) {
  delete scalar;
  return 0;
}
extern "C" aclnnStatus aclSetTensorAddr(aclOpExecutor* executor, uint64_t, const aclTensor* tensor, void* address) {
  if (executor == nullptr || tensor == nullptr || address == nullptr) return kErrNull;
  if (reinterpret_cast<uintptr_t>(address) % 32 != 0) {
    SetLastError("aclSetTensorAddr: replacement address %p is not 32-byte aligned", address);
    return kErrInvalid;
  }
  const_cast<aclTensor*>(tensor)->data = address;
  return 0;
}
extern "C" aclnnStatus aclSetDynamicTensorAddr(aclOpExecutor* executor, uint64_t, uint64_t relative_index,
                                               const aclTensorList* list, void* address) {
  if (executor == nullptr || list == nullptr || address == nullptr) return kErrNull;
  if (relative_index >= list->items.size() || reinterpret_cast<uintptr_t>(address) % 32 != 0) {
    SetLastError("aclSetDynamicTensorAddr: entry %llu of a %zu-entry list, address %p",
                 static_cast<unsigned long long>(relative_index), list->items.size(), address);
    return kErrInvalid;
  }
  list->items[relative_index]->data = address;
  return 0;
}
extern "C" aclnnStatus aclSetAclOpExecutorRepeatable(aclOpExecutor* executor) {
  if (executor == nullptr) return kErrNull;
  executor->repeatable = true;
  return 0;
}
extern "C" aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor) {
  delete executor;
  return 0;
}

// ---- runtime: thin wrappers over the CUDA runtime --------------------------------------------------------
namespace {
aclError Rt(cudaError_t err, const char* what) { return CheckCuda(err, what) == B200KV_OK ? ACL_SUCCESS : ACL_ERROR_RT_FAILURE; }
cudaMemcpyKind Kind(aclrtMemcpyKind k) {
  switch (k) {
    case ACL_MEMCPY_HOST_TO_HOST: return cudaMemcpyHostToHost;
    case ACL_MEMCPY_HOST_TO_DEVICE: return cudaMemcpyHostToDevice;
    case ACL_MEMCPY_DEVICE_TO_HOST: return cudaMemcpyDeviceToHost;
    default: return cudaMemcpyDeviceToDevice;
  }
}
}  // namespace

extern "C" aclError aclInit(const char*) { return ACL_SUCCESS; }
extern "C" aclError aclFinalize(void) { return ACL_SUCCESS; }
extern "C" aclnnStatus aclnnInit(const char*) { return 0; }
extern "C" aclnnStatus aclnnFinalize(void) { return 0; }
extern "C" const char* aclGetRecentErrMsg(void) { return b200kv_last_error(); }
extern "C" aclError aclrtSetDevice(int32_t device_id) { return Rt(cudaSetDevice(device_id), "aclrtSetDevice"); }
extern "C" aclError aclrtResetDevice(int32_t) { return ACL_SUCCESS; }  // the context is left to the process
extern "C" aclError aclrtCreateContext(aclrtContext* context, int32_t device_id) {
  if (context == nullptr) return ACL_ERROR_INVALID_PARAM;
  *context = reinterpret_cast<aclrtContext>(static_cast<intptr_t>(device_id) + 1);  // the primary context
  return Rt(cudaSetDevice(device_id), "aclrtCreateContext");
}
extern "C" aclError aclrtDestroyContext(aclrtContext) { return ACL_SUCCESS; }
extern "C" aclError aclrtSetCurrentContext(aclrtContext context) {
  return Rt(cudaSetDevice(static_cast<int>(reinterpret_cast<intptr_t>(context)) - 1), "aclrtSetCurrentContext");
}
extern "C" aclError aclrtGetDeviceCount(uint32_t* device_count) {
  if (device_count == nullptr) return ACL_ERROR_INVALID_PARAM;
  int n = 0;
  const aclError rc = Rt(cudaGetDeviceCount(&n), "aclrtGetDeviceCount");
  *device_count = static_cast<uint32_t>(n);
  return rc;
}
extern "C" const char* aclrtGetSocName(void) { return "NVIDIA-B200-sm_100a"; }
extern "C" aclError aclrtMalloc(void** device_ptr, size_t size, aclrtMemMallocPolicy) {
  if (device_ptr == nullptr || size == 0) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMalloc(device_ptr, size), "aclrtMalloc");
}
extern "C" aclError aclrtFree(void* device_ptr) { return Rt(cudaFree(device_ptr), "aclrtFree"); }
extern "C" aclError aclrtMallocHost(void** host_ptr, size_t size) {
  if (host_ptr == nullptr || size == 0) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMallocHost(host_ptr, size), "aclrtMallocHost");
}
extern "C" aclError aclrtFreeHost(void* host_ptr) { return Rt(cudaFreeHost(host_ptr), "aclrtFreeHost"); }
extern "C" aclError aclrtMemcpy(void* destination, size_t capacity, const void* source, size_t count,
                                aclrtMemcpyKind kind) {
  if (destination == nullptr || source == nullptr || count > capacity) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMemcpy(destination, source, count, Kind(kind)), "aclrtMemcpy");
}
extern "C" aclError aclrtMemcpyAsync(void* destination, size_t capacity, const void* source, size_t count,
                                     aclrtMemcpyKind kind, aclrtStream stream) {
  if (destination == nullptr || source == nullptr || count > capacity) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMemcpyAsync(destination, source, count, Kind(kind), static_cast<cudaStream_t>(stream)), "aclrtMemcpyAsync");
}
extern "C" aclError aclrtMemset(void* destination, size_t capacity, int32_t value, size_t count) {
  if (destination == nullptr || count > capacity) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMemset(destination, value, count), "aclrtMemset");
}
extern "C" aclError aclrtCreateStream(aclrtStream* stream) {
  if (stream == nullptr) return ACL_ERROR_INVALID_PARAM;
  cudaStream_t s = nullptr;
  const aclError rc = Rt(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "aclrtCreateStream");
  *stream = s;
  return rc;
}
extern "C" aclError aclrtDestroyStream(aclrtStream stream) {
  return Rt(cudaStreamDestroy(static_cast<cudaStream_t>(stream)), "aclrtDestroyStream");
}
extern "C" aclError aclrtDestroyStreamForce(aclrtStream stream) { return aclrtDestroyStream(stream); }
extern "C" aclError aclrtCreateEventExWithFlag(aclrtEvent* event, uint32_t) {
  if (event == nullptr) return ACL_ERROR_INVALID_PARAM;
  cudaEvent_t e = nullptr;
  const aclError rc = Rt(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "aclrtCreateEventExWithFlag");
  *event = e;
  return rc;
}
extern "C" aclError aclrtDestroyEvent(aclrtEvent event) {
  return Rt(cudaEventDestroy(static_cast<cudaEvent_t>(event)), "aclrtDestroyEvent");
}
extern "C" aclError aclrtRecordEvent(aclrtEvent event, aclrtStream stream) {
  return Rt(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)), "aclrtRecordEvent");
}
extern "C" aclError aclrtStreamWaitEvent(aclrtStream stream, aclrtEvent event) {
  return Rt(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0),
            "aclrtStreamWaitEvent");
}
extern "C" aclError aclrtSynchronizeStream(aclrtStream stream) {
  return Rt(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "aclrtSynchronizeStream");
}
// Bounded wait: polls the stream instead of blocking in the driver (the reference gives its
// synchronisations a deadline, src/core/device_ops.cpp:213-216).
extern "C" aclError aclrtSynchronizeStreamWithTimeout(aclrtStream stream, int32_t timeout_ms) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  for (;;) {
    const cudaError_t q = cudaStreamQuery(static_cast<cudaStream_t>(stream));
    if (q == cudaSuccess) return ACL_SUCCESS;
    if (q != cudaErrorNotReady) return Rt(q, "aclrtSynchronizeStreamWithTimeout");
    if (timeout_ms >= 0 && std::chrono::steady_clock::now() >= deadline) {
      SetLastError("aclrtSynchronizeStreamWithTimeout: stream still busy after %d ms", timeout_ms);
      return ACL_ERROR_RT_FAILURE;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}
extern "C" aclError aclrtSynchronizeEvent(aclrtEvent event) {
  return Rt(cudaEventSynchronize(static_cast<cudaEvent_t>(event)), "aclrtSynchronizeEvent");
}
extern "C" aclError aclrtGetMemInfo(aclrtMemAttr, size_t* free_bytes, size_t* total_bytes) {
  if (free_bytes == nullptr || total_bytes == nullptr) return ACL_ERROR_INVALID_PARAM;
  return Rt(cudaMemGetInfo(free_bytes, total_bytes), "aclrtGetMemInfo");
}

// ---- the two operators of the KV path ----------------------------------------------------------------------
namespace {

bool IsBf16(const aclTensor* t) { return t != nullptr && t->dtype == ACL_BF16; }
bool InnerContiguous(const aclTensor* t) { return !t->strides.empty() && t->strides.back() == 1; }

aclnnStatus Refuse(const char* op, const char* why) {
  SetLastError("%s: %s", op, why);
  return kErrInvalid;
}

// Rows x width view of a paged cache [blocks, block_size, 1, width] (or any shape whose last dimension
// is `width` and whose rows are `row_stride` apart).
bool CacheGeometry(const aclTensor* cache, int64_t width, int64_t* rows, int64_t* row_stride) {
  if (cache->dims.size() < 2 || cache->dims.back() != width || !InnerContiguous(cache)) return false;
  *rows = cache->Elements() / width;
  // The stride of the innermost dimension with extent > 1 above the feature axis is the row stride.
  *row_stride = width;
  for (int64_t i = static_cast<int64_t>(cache->dims.size()) - 2; i >= 0; --i) {
    if (cache->dims[i] > 1) {
      *row_stride = cache->strides[i];
      break;
    }
  }
  return *row_stride >= width;
}

// Gathers query [B, H, 512] and query_rope [B, H, 64] into one [B, H, 576] buffer (the layout the decode
// kernel reads) when the caller keeps them apart.
__global__ void PackQueryKernel(const __nv_bfloat16* q, int64_t q_seq, int64_t q_head, const __nv_bfloat16* r,
                                int64_t r_seq, int64_t r_head, __nv_bfloat16* dst, int32_t batch, int32_t heads) {
  const int64_t chunks = static_cast<int64_t>(batch) * heads * 72;  // 16-byte chunks of a 576-wide row
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % 72);
    const int64_t row = i / 72;
    const int64_t b = row / heads, h = row % heads;
    const __nv_bfloat16* src = c < 64 ? q + b * q_seq + h * q_head + 8 * c : r + b * r_seq + h * r_head + 8 * (c - 64);
    int4 v;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      v = *reinterpret_cast<const int4*>(src);
    } else {
      const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
      uint16_t tmp[8];
      for (int k = 0; k < 8; ++k) tmp[k] = s16[k];
      v = *reinterpret_cast<const int4*>(tmp);
    }
    *reinterpret_cast<int4*>(dst + row * 576 + 8 * c) = v;
  }
}

}  // namespace

extern "C" aclnnStatus aclnnScatterPaKvCacheGetWorkspaceSize(
    const aclTensor* key, aclTensor* key_cache_ref, const aclTensor* slot_mapping, const aclTensor* value,
    aclTensor* value_cache_ref, const aclTensor* compress_lens_optional, const aclTensor* compress_seq_offset_optional,
    const aclTensor* seq_lens_optional, char* cache_mode_optional, char* scatter_mode_optional,
    const aclIntArray* strides_optional, const aclIntArray* offsets_optional, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const char* op = "aclnnScatterPaKvCache";
  if (key == nullptr || key_cache_ref == nullptr || slot_mapping == nullptr || value == nullptr ||
      value_cache_ref == nullptr || workspace_size == nullptr || executor == nullptr) {
    SetLastError("%s: a required argument is null", op);
    return kErrNull;
  }
  if (compress_lens_optional || compress_seq_offset_optional || seq_lens_optional || scatter_mode_optional ||
      strides_optional || offsets_optional) {
    return Refuse(op, "compression, sequence-length, scatter-mode, stride and offset arguments are not supported");
  }
  if (cache_mode_optional != nullptr && std::strcmp(cache_mode_optional, "Norm") != 0) {
    return Refuse(op, "only cache mode \"Norm\" is supported");
  }
  if (!IsBf16(key) || !IsBf16(value) || !IsBf16(key_cache_ref) || !IsBf16(value_cache_ref) ||
      slot_mapping->dtype != ACL_INT32) {
    return Refuse(op, "key, value and caches must be BF16 and slot_mapping INT32");
  }
  int64_t rows_k = 0, stride_k = 0, rows_v = 0, stride_v = 0;
  if (!CacheGeometry(key_cache_ref, B200KV_LATENT_DIM, &rows_k, &stride_k) ||
      !CacheGeometry(value_cache_ref, B200KV_ROPE_DIM, &rows_v, &stride_v) || rows_k != rows_v) {
    return Refuse(op, "caches must be [blocks, block_size, 1, 512] and [blocks, block_size, 1, 64] with equal rows");
  }
  const int64_t tokens = slot_mapping->Elements();
  if (key->Elements() != tokens * B200KV_LATENT_DIM || value->Elements() != tokens * B200KV_ROPE_DIM ||
      !InnerContiguous(key) || !InnerContiguous(value)) {
    return Refuse(op, "key must be [T, 512], value [T, 1, 64] and slot_mapping [T]");
  }
  auto* exec = new (std::nothrow) aclOpExecutor();
  if (exec == nullptr) return kErrRuntime;
  exec->kind = aclOpExecutor::kScatter;
  exec->key = key;
  exec->value = value;
  exec->slots = slot_mapping;
  exec->key_cache = key_cache_ref;
  exec->value_cache = value_cache_ref;
  *workspace_size = 0;
  *executor = exec;
  return 0;
}

extern "C" aclnnStatus aclnnScatterPaKvCache(void*, uint64_t, aclOpExecutor* exec, aclrtStream stream) {
  if (exec == nullptr || exec->kind != aclOpExecutor::kScatter) {
    SetLastError("aclnnScatterPaKvCache: not an executor planned for this operator");
    return kErrNull;
  }
  int64_t rows = 0, stride_k = 0, stride_v = 0, rows_v = 0;
  CacheGeometry(exec->key_cache, B200KV_LATENT_DIM, &rows, &stride_k);
  CacheGeometry(exec->value_cache, B200KV_ROPE_DIM, &rows_v, &stride_v);
  b200kv_pool_view pool{exec->key_cache->Address(), exec->value_cache->Address(), stride_k, stride_v, rows};
  const int64_t tokens = exec->slots->Elements();
  const int64_t key_stride = exec->key->dims.size() >= 2 ? exec->key->strides[0] : B200KV_LATENT_DIM;
  const int64_t value_stride = exec->value->dims.size() >= 2 ? exec->value->strides[0] : B200KV_ROPE_DIM;
  const int32_t rc = b200kv_append(&pool, exec->key->Address(), tokens > 1 ? key_stride : B200KV_LATENT_DIM,
                                   exec->value->Address(), tokens > 1 ? value_stride : B200KV_ROPE_DIM,
                                   static_cast<const int32_t*>(exec->slots->Address()), tokens, stream, nullptr);
  const bool once = !exec->repeatable;
  if (once) delete exec;  // a launch consumes an executor that was not marked repeatable
  return rc == B200KV_OK ? 0 : (rc == B200KV_ERR_RUNTIME ? kErrRuntime : rc);
}

extern "C" aclnnStatus aclnnFusedInferAttentionScoreV5GetWorkspaceSize(
    const aclTensor* query, const aclTensorList* key, const aclTensorList* value, const aclTensor* pse_shift,
    const aclTensor* atten_mask, const aclIntArray* actual_seq_lengths, const aclIntArray* actual_seq_lengths_kv,
    const aclTensor* deq_scale1, const aclTensor* quant_scale1, const aclTensor* deq_scale2,
    const aclTensor* quant_scale2, const aclTensor* quant_offset2, const aclTensor* antiquant_scale,
    const aclTensor* antiquant_offset, const aclTensor* block_table, const aclTensor* query_padding_size,
    const aclTensor* kv_padding_size, const aclTensor* key_antiquant_scale, const aclTensor* key_antiquant_offset,
    const aclTensor* value_antiquant_scale, const aclTensor* value_antiquant_offset,
    const aclTensor* key_shared_prefix, const aclTensor* value_shared_prefix,
    const aclIntArray* actual_shared_prefix_len, const aclTensor* query_rope, const aclTensor* key_rope,
    const aclTensor* key_rope_antiquant_scale, const aclTensor* dequant_scale_query, const aclTensor* learnable_sink,
    const aclIntArray* q_start_idx, const aclIntArray* kv_start_idx, int64_t num_heads, double scale_value,
    int64_t pre_tokens, int64_t next_tokens, char* input_layout, int64_t num_key_value_heads, int64_t sparse_mode,
    int64_t inner_precise, int64_t block_size, int64_t antiquant_mode, bool softmax_lse_flag,
    int64_t key_antiquant_mode, int64_t value_antiquant_mode, int64_t query_quant_mode, int64_t pse_type,
    const aclTensor* attention_out, const aclTensor* softmax_lse, uint64_t* workspace_size, aclOpExecutor** executor) {
  const char* op = "aclnnFusedInferAttentionScoreV5";
  (void)pre_tokens; (void)next_tokens; (void)sparse_mode; (void)inner_precise;  // one query token: no window applies
  if (query == nullptr || key == nullptr || value == nullptr || block_table == nullptr || query_rope == nullptr ||
      key_rope == nullptr || actual_seq_lengths_kv == nullptr || attention_out == nullptr ||
      workspace_size == nullptr || executor == nullptr) {
    SetLastError("%s: a required argument is null (paged MLA needs query, key, value, block_table, query_rope, "
                 "key_rope, actual_seq_lengths_kv and attention_out)", op);
    return kErrNull;
  }
  if (pse_shift || atten_mask || deq_scale1 || quant_scale1 || deq_scale2 || quant_scale2 || quant_offset2 ||
      antiquant_scale || antiquant_offset || query_padding_size || kv_padding_size || key_antiquant_scale ||
      key_antiquant_offset || value_antiquant_scale || value_antiquant_offset || key_shared_prefix ||
      value_shared_prefix || actual_shared_prefix_len || key_rope_antiquant_scale || dequant_scale_query ||
      learnable_sink || q_start_idx || kv_start_idx || antiquant_mode != 0 || key_antiquant_mode != 0 ||
      value_antiquant_mode != 0 || query_quant_mode != 0 || pse_type != 0) {
    return Refuse(op, "masks, position terms, quantisation, padding, shared prefixes, sinks and start indices "
                      "are not supported: pass null / 0");
  }
  if (input_layout == nullptr || std::strcmp(input_layout, "TND") != 0) return Refuse(op, "only layout TND is supported");
  if (num_key_value_heads != 1 || num_heads <= 0 || !(scale_value > 0.0) || block_size <= 0) {
    return Refuse(op, "needs one key/value head, positive head count, scale and block size");
  }
  if (key->items.empty() || value->items.empty() || key->items[0] == nullptr) {
    return Refuse(op, "key and value lists must hold the latent cache");
  }
  const aclTensor* latent = key->items[0];
  if (!IsBf16(query) || !IsBf16(query_rope) || !IsBf16(latent) || !IsBf16(key_rope) || !IsBf16(attention_out) ||
      block_table->dtype != ACL_INT32) {
    return Refuse(op, "query, caches and output must be BF16 and block_table INT32");
  }
  if (query->dims.size() != 3 || query->dims[1] != num_heads || query->dims[2] != B200KV_LATENT_DIM ||
      query_rope->dims.size() != 3 || query_rope->dims[0] != query->dims[0] || query_rope->dims[1] != num_heads ||
      query_rope->dims[2] != B200KV_ROPE_DIM || !InnerContiguous(query) || !InnerContiguous(query_rope)) {
    return Refuse(op, "query must be [T, heads, 512] and query_rope [T, heads, 64]");
  }
  const int64_t batch = query->dims[0];
  if (actual_seq_lengths != nullptr) {
    for (size_t i = 0; i < actual_seq_lengths->values.size(); ++i) {
      // TND lengths are cumulative; one query token per sequence is the only supported case.
      if (actual_seq_lengths->values[i] != static_cast<int64_t>(i) + 1) {
        return Refuse(op, "one query token per sequence is required (actual_seq_lengths = 1, 2, 3, ...)");
      }
    }
  }
  if (static_cast<int64_t>(actual_seq_lengths_kv->values.size()) != batch) {
    return Refuse(op, "actual_seq_lengths_kv must hold one length per sequence");
  }
  int64_t rows_k = 0, stride_k = 0, rows_r = 0, stride_r = 0;
  if (!CacheGeometry(latent, B200KV_LATENT_DIM, &rows_k, &stride_k) ||
      !CacheGeometry(key_rope, B200KV_ROPE_DIM, &rows_r, &stride_r) || rows_k != rows_r || rows_k % block_size != 0) {
    return Refuse(op, "caches must be [blocks, block_size, 1, 512] and [blocks, block_size, 1, 64] with equal rows");
  }
  if (block_table->dims.size() != 2 || block_table->dims[0] != batch || !InnerContiguous(block_table)) {
    return Refuse(op, "block_table must be [sequences, blocks]");
  }
  if (attention_out->Elements() != batch * num_heads * B200KV_LATENT_DIM) {
    return Refuse(op, "attention_out must be [T, heads, 512]");
  }
  if (softmax_lse_flag && (softmax_lse == nullptr || softmax_lse->dtype != ACL_FLOAT32 ||
                           softmax_lse->Elements() != batch * num_heads)) {
    return Refuse(op, "softmax_lse must be FP32 [T, heads, 1] when the flag is set");
  }
  auto* exec = new (std::nothrow) aclOpExecutor();
  if (exec == nullptr) return kErrRuntime;
  exec->kind = aclOpExecutor::kAttention;
  exec->query = query;
  exec->query_rope = query_rope;
  exec->latent_cache = latent;
  exec->rope_cache = key_rope;
  exec->block_table = block_table;
  exec->out = attention_out;
  exec->lse = softmax_lse_flag ? softmax_lse : nullptr;
  exec->batch = static_cast<int32_t>(batch);
  exec->heads = static_cast<int32_t>(num_heads);
  exec->block_size = static_cast<int32_t>(block_size);
  exec->scale = static_cast<float>(scale_value);
  for (int64_t v : actual_seq_lengths_kv->values) exec->kv_len.push_back(static_cast<int32_t>(v));
  exec->decode_ws = (b200kv_mla_decode_workspace_bytes(exec->batch, exec->heads, 0) + 255) / 256 * 256;
  exec->q_pack_bytes = (static_cast<uint64_t>(batch) * num_heads * 576 * 2 + 255) / 256 * 256;
  *workspace_size = exec->decode_ws + exec->q_pack_bytes + (static_cast<uint64_t>(batch) * 4 + 255) / 256 * 256;
  *executor = exec;
  return 0;
}

extern "C" aclnnStatus aclnnFusedInferAttentionScoreV5(void* workspace, uint64_t workspace_size, aclOpExecutor* exec,
                                                       aclrtStream stream) {
  if (exec == nullptr || exec->kind != aclOpExecutor::kAttention || workspace == nullptr) {
    SetLastError("aclnnFusedInferAttentionScoreV5: null workspace or an executor of another operator");
    return kErrNull;
  }
  const uint64_t need = exec->decode_ws + exec->q_pack_bytes + (static_cast<uint64_t>(exec->batch) * 4 + 255) / 256 * 256;
  if (workspace_size < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0) {
    SetLastError("aclnnFusedInferAttentionScoreV5: workspace of %llu bytes (256-byte aligned) planned, %llu given",
                 static_cast<unsigned long long>(need), static_cast<unsigned long long>(workspace_size));
    return kErrInvalid;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  __nv_bfloat16* q_packed = reinterpret_cast<__nv_bfloat16*>(ws + exec->decode_ws);
  int32_t* kv_len_dev = reinterpret_cast<int32_t*>(ws + exec->decode_ws + exec->q_pack_bytes);
  if (CheckCuda(cudaMemcpyAsync(kv_len_dev, exec->kv_len.data(), exec->kv_len.size() * 4, cudaMemcpyHostToDevice, cs),
                "sequence lengths upload") != B200KV_OK) {
    return kErrRuntime;
  }
  const aclTensor* q = exec->query;
  const aclTensor* r = exec->query_rope;
  b200kv_decode_args a{};
  const bool fused = static_cast<const __nv_bfloat16*>(r->Address()) ==
                         static_cast<const __nv_bfloat16*>(q->Address()) + B200KV_LATENT_DIM &&
                     q->strides[1] == r->strides[1] && q->strides[0] == r->strides[0] && q->strides[1] >= 576;
  if (fused) {
    a.q = q->Address();
    a.q_seq_stride = q->strides[0];
    a.q_head_stride = q->strides[1];
  } else {
    const int64_t chunks = static_cast<int64_t>(exec->batch) * exec->heads * 72;
    const int ctas = static_cast<int>((chunks + 255) / 256 < 1184 ? (chunks + 255) / 256 : 1184);
    PackQueryKernel<<<ctas, 256, 0, cs>>>(static_cast<const __nv_bfloat16*>(q->Address()), q->strides[0], q->strides[1],
                                          static_cast<const __nv_bfloat16*>(r->Address()), r->strides[0], r->strides[1],
                                          q_packed, exec->batch, exec->heads);
    if (CheckCuda(cudaGetLastError(), "query pack launch") != B200KV_OK) return kErrRuntime;
    a.q = q_packed;
    a.q_seq_stride = static_cast<int64_t>(exec->heads) * 576;
    a.q_head_stride = 576;
  }
  int64_t rows = 0, stride_k = 0, rows_r = 0, stride_r = 0;
  CacheGeometry(exec->latent_cache, B200KV_LATENT_DIM, &rows, &stride_k);
  CacheGeometry(exec->rope_cache, B200KV_ROPE_DIM, &rows_r, &stride_r);
  a.pool = b200kv_pool_view{exec->latent_cache->Address(), exec->rope_cache->Address(), stride_k, stride_r, rows};
  a.block_table = static_cast<const int32_t*>(exec->block_table->Address());
  a.max_blocks = exec->block_table->strides[0];
  a.kv_len = kv_len_dev;
  a.batch = exec->batch;
  a.heads = exec->heads;
  a.block_size = exec->block_size;
  a.scale = exec->scale;
  a.out = exec->out->Address();
  a.lse = exec->lse != nullptr ? static_cast<float*>(exec->lse->Address()) : nullptr;
  a.workspace = ws;
  a.workspace_bytes = exec->decode_ws;
  a.variant = B200KV_DECODE_AUTO;
  const int32_t rc = b200kv_mla_decode(&a, stream, nullptr);
  if (!exec->repeatable) delete exec;
  return rc == B200KV_OK ? 0 : (rc == B200KV_ERR_RUNTIME ? kErrRuntime : rc);
}
