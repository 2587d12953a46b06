/*
 * b200kv_aclnn.h: the operator-library ABI of the reference engine, served by libb200kv.so.
 *
 * The reference resolves its operators by name at run time (dlsym(RTLD_DEFAULT, ...),
 * src/core/op_table.cpp:95-121) and talks to the device through the aclrt calls below
 * (src/core/device_ops.cpp:96-262). Its mock operator library (mock/include/acl/acl.h,
 * mock/include/acl/acl_base.h, mock/include/aclnn/acl_meta.h, mock/include/aclnn/aclnn_base.h)
 * shows that a replacement library exporting the same C symbols runs the engine unchanged. This
 * header declares the part of that ABI the KV path crosses; every symbol has C linkage and the
 * signature and status convention of the file cited beside it.
 *
 *   descriptors + executor protocol      mock/include/aclnn/acl_meta.h:58-91
 *   aclnnScatterPaKvCache (two phases)   include/moe/core/op_table.hpp:365-372, :1022
 *   aclnnFusedInferAttentionScoreV5      include/moe/core/op_table.hpp:438-454, :1022
 *   runtime (aclrt*, aclInit, ...)       mock/include/acl/acl.h:33-72
 *
 * Not exported: the other operators of the decode graph (GEMMs, norms, RoPE, MoE); they are outside the
 * KV path, so an unmodified engine still needs its own library for those.
 *
 * Semantics that differ from a no-op mock: the launches do the work. ScatterPaKvCache writes rows into
 * the two caches; FusedInferAttentionScoreV5 attends over actual_seq_lengths_kv[b] tokens of sequence b
 * through block_table, with scale_value, for TND layout, one query token per sequence, 64 query heads
 * over one latent KV head (value list = key list = latent cache, key_rope = rope cache). Quantisation,
 * masks, shared prefixes and position terms must be null / "none": anything else is refused at plan
 * time with 161002.
 */
#ifndef B200KV_ACLNN_H_
#define B200KV_ACLNN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t aclError;
typedef int32_t aclnnStatus;
typedef void* aclrtStream;
typedef void* aclrtEvent;
typedef void* aclrtContext;

/* Values of the reference's headers (mock/include/aclnn/acl_meta.h:32-52, acl_base.h:33-57). */
typedef enum aclDataType {
  ACL_FLOAT32 = 0, ACL_FLOAT16 = 1, ACL_INT8 = 2, ACL_INT32 = 3, ACL_UINT8 = 4, ACL_INT16 = 6, ACL_UINT16 = 7,
  ACL_INT64 = 9, ACL_UINT64 = 10, ACL_FLOAT64 = 11, ACL_BOOL = 12, ACL_DT_UNDEFINED = 17, ACL_BF16 = 27,
  ACL_FLOAT8_E5M2 = 35, ACL_FLOAT8_E4M3FN = 36, ACL_FLOAT8_E8M0 = 37, ACL_FP4X2_E2M1 = 40
} aclDataType;
typedef enum aclFormat { ACL_FORMAT_ND = 2 } aclFormat;
typedef enum aclrtMemcpyKind {
  ACL_MEMCPY_HOST_TO_HOST = 0, ACL_MEMCPY_HOST_TO_DEVICE = 1, ACL_MEMCPY_DEVICE_TO_HOST = 2,
  ACL_MEMCPY_DEVICE_TO_DEVICE = 3
} aclrtMemcpyKind;
typedef enum aclrtMemMallocPolicy {
  ACL_MEM_MALLOC_HUGE_FIRST = 0, ACL_MEM_MALLOC_HUGE_ONLY = 1, ACL_MEM_MALLOC_NORMAL_FIRST = 2,
  ACL_MEM_MALLOC_NORMAL_ONLY = 3
} aclrtMemMallocPolicy;
typedef enum aclrtMemAttr { ACL_HBM_MEM = 0, ACL_DDR_MEM = 1 } aclrtMemAttr;

#define ACL_SUCCESS 0
#define ACL_ERROR_INVALID_PARAM 100000
#define ACL_ERROR_RT_FAILURE 107000

typedef struct aclOpExecutor aclOpExecutor;
typedef struct aclTensor aclTensor;
typedef struct aclScalar aclScalar;
typedef struct aclIntArray aclIntArray;
typedef struct aclTensorList aclTensorList;

/* ---- descriptors (mock/include/aclnn/acl_meta.h:58-91) ---- */
aclTensor* aclCreateTensor(const int64_t* view_dims, uint64_t view_dims_num, aclDataType dtype,
                           const int64_t* view_strides, int64_t storage_offset, aclFormat format,
                           const int64_t* storage_dims, uint64_t storage_dims_num, void* device_data);
aclnnStatus aclDestroyTensor(const aclTensor* tensor);
aclnnStatus aclGetViewShape(const aclTensor* tensor, int64_t** dims, uint64_t* count);
aclnnStatus aclGetStorageShape(const aclTensor* tensor, int64_t** dims, uint64_t* count);
aclnnStatus aclGetViewStrides(const aclTensor* tensor, int64_t** strides, uint64_t* count);
aclnnStatus aclGetDataType(const aclTensor* tensor, aclDataType* dtype);
aclnnStatus aclGetFormat(const aclTensor* tensor, aclFormat* format);
aclnnStatus aclGetRawTensorAddr(const aclTensor* tensor, void** address);
aclnnStatus aclGetViewOffset(const aclTensor* tensor, int64_t* offset);
aclTensorList* aclCreateTensorList(const aclTensor* const* tensors, uint64_t size);
aclnnStatus aclDestroyTensorList(const aclTensorList* tensor_list);
aclIntArray* aclCreateIntArray(const int64_t* value, uint64_t size);
aclnnStatus aclDestroyIntArray(const aclIntArray* array);
aclScalar* aclCreateScalar(void* value, aclDataType dtype);
aclnnStatus aclDestroyScalar(const aclScalar* scalar);
/* Repoint a planned executor's tensor: the handle keeps the new address until changed again. */
aclnnStatus aclSetTensorAddr(aclOpExecutor* executor, uint64_t index, const aclTensor* tensor, void* address);
aclnnStatus aclSetDynamicTensorAddr(aclOpExecutor* executor, uint64_t ir_index, uint64_t relative_index,
                                    const aclTensorList* tensor_list, void* address);
aclnnStatus aclSetAclOpExecutorRepeatable(aclOpExecutor* executor);
aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor);

/* ---- the two operators on the KV path, plan + launch ---- */
aclnnStatus aclnnScatterPaKvCacheGetWorkspaceSize(
    const aclTensor* key, aclTensor* key_cache_ref, const aclTensor* slot_mapping, const aclTensor* value,
    aclTensor* value_cache_ref, const aclTensor* compress_lens_optional, const aclTensor* compress_seq_offset_optional,
    const aclTensor* seq_lens_optional, char* cache_mode_optional, char* scatter_mode_optional,
    const aclIntArray* strides_optional, const aclIntArray* offsets_optional, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnScatterPaKvCache(void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                                  aclrtStream stream);
aclnnStatus aclnnFusedInferAttentionScoreV5GetWorkspaceSize(
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
    const aclTensor* attention_out, const aclTensor* softmax_lse, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnFusedInferAttentionScoreV5(void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                                            aclrtStream stream);

/* ---- runtime (mock/include/acl/acl.h:33-72), thin wrappers over the CUDA runtime ---- */
aclError aclInit(const char* config_path);
aclError aclFinalize(void);
aclnnStatus aclnnInit(const char* config_path);
aclnnStatus aclnnFinalize(void);
const char* aclGetRecentErrMsg(void);
aclError aclrtSetDevice(int32_t device_id);
aclError aclrtResetDevice(int32_t device_id);
aclError aclrtCreateContext(aclrtContext* context, int32_t device_id);
aclError aclrtDestroyContext(aclrtContext context);
aclError aclrtSetCurrentContext(aclrtContext context);
aclError aclrtGetDeviceCount(uint32_t* device_count);
const char* aclrtGetSocName(void);
aclError aclrtMalloc(void** device_ptr, size_t size, aclrtMemMallocPolicy policy);
aclError aclrtFree(void* device_ptr);
aclError aclrtMallocHost(void** host_ptr, size_t size);
aclError aclrtFreeHost(void* host_ptr);
aclError aclrtMemcpy(void* destination, size_t destination_capacity, const void* source, size_t count,
                     aclrtMemcpyKind kind);
aclError aclrtMemcpyAsync(void* destination, size_t destination_capacity, const void* source, size_t count,
                          aclrtMemcpyKind kind, aclrtStream stream);
aclError aclrtMemset(void* destination, size_t destination_capacity, int32_t value, size_t count);
aclError aclrtCreateStream(aclrtStream* stream);
aclError aclrtDestroyStream(aclrtStream stream);
aclError aclrtDestroyStreamForce(aclrtStream stream);
aclError aclrtCreateEventExWithFlag(aclrtEvent* event, uint32_t flag);
aclError aclrtDestroyEvent(aclrtEvent event);
aclError aclrtRecordEvent(aclrtEvent event, aclrtStream stream);
aclError aclrtStreamWaitEvent(aclrtStream stream, aclrtEvent event);
aclError aclrtSynchronizeStream(aclrtStream stream);
aclError aclrtSynchronizeStreamWithTimeout(aclrtStream stream, int32_t timeout_ms);
aclError aclrtSynchronizeEvent(aclrtEvent event);
aclError aclrtGetMemInfo(aclrtMemAttr attr, size_t* free_bytes, size_t* total_bytes);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_ACLNN_H_ */
