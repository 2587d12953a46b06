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
 * The other 25 operators of the decode graph (GEMMs, norms, RoPE, MoE, ...) are exported as plan-checking
 * stand-ins whose launches do nothing (see below): they are outside the KV path.
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

/*
 * ---- the other operators of the decode graph: plan checks, launch does nothing ----
 * Exported so that an engine that resolves every operator from this library still builds and steps;
 * they are outside the KV path and are NOT implemented: each plan checks its required arguments, needs no
 * workspace and returns an executor, each launch checks that the executor belongs to it and enqueues
 * nothing. Signatures: the plan-function types of include/moe/core/op_table.hpp, lines 169 (RmsNorm),
 * 199 (RmsNormDynamicMxQuant), 230 (DynamicMxQuant), 253 (Cast), 277 (Matmul), 308 (QuantMatmulV5),
 * 335 (ApplyRotaryPosEmbV2), 473 (Sigmoid, Sqrt), 494 (Mul), 514 (InplaceAdd), 534 (SwiGlu), 555 (ArgMax),
 * 580 (Softplus), 615 (MoeGatingTopKV2), 658 (MoeInitRoutingV4), 711 (GroupedMatmulV5), 757 (SwigluMxQuant),
 * 785 (MoeTokenUnpermute), 821 (GroupedMatmulSwigluQuantV2), 864 (GroupedMatmulFinalizeRoutingV3),
 * 907 (MhcPre), 938 (MhcSinkhorn), 960 (MhcPost), 998 (QuantLightningIndexer); names: src/core/op_table.cpp:47-88.
 */
aclnnStatus aclnnRmsNormGetWorkspaceSize(const aclTensor* x, const aclTensor* gamma, double epsilon,
    const aclTensor* y_out, const aclTensor* rstd_out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnRmsNorm(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnRmsNormDynamicMxQuantGetWorkspaceSize(const aclTensor* x, const aclTensor* gamma,
    const aclTensor* beta, double epsilon, int64_t scale_alg, char* round_mode, int64_t dst_type, bool output_rstd,
    aclTensor* y_out, aclTensor* mxscale_out, aclTensor* rstd_out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnRmsNormDynamicMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnDynamicMxQuantGetWorkspaceSize(const aclTensor* x, int64_t axis, char* round_mode_optional,
    int64_t dst_type, int64_t blocksize, int64_t scale_alg, const aclTensor* y_out, const aclTensor* mxscale_out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnDynamicMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnCastGetWorkspaceSize(const aclTensor* self, aclDataType dtype, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnCast(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMatmulGetWorkspaceSize(const aclTensor* self, const aclTensor* mat2, aclTensor* out,
    int8_t cube_math_type, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMatmul(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnQuantMatmulV5GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* x1_scale,
    const aclTensor* x2_scale, const aclTensor* y_scale, const aclTensor* x1_offset, const aclTensor* x2_offset,
    const aclTensor* y_offset, const aclTensor* bias, bool transpose_x1, bool transpose_x2, int64_t group_size,
    aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnQuantMatmulV5(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnApplyRotaryPosEmbV2GetWorkspaceSize(aclTensor* query_ref, aclTensor* key_ref, const aclTensor* cos,
    const aclTensor* sin, int64_t layout, char* rotary_mode, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnApplyRotaryPosEmbV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnSigmoidGetWorkspaceSize(const aclTensor* self, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnSigmoid(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnSqrtGetWorkspaceSize(const aclTensor* self, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnSqrt(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMulGetWorkspaceSize(const aclTensor* self, const aclTensor* other, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMul(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnInplaceAddGetWorkspaceSize(const aclTensor* self_ref, const aclTensor* other, const aclScalar* alpha,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnInplaceAdd(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnSwiGluGetWorkspaceSize(const aclTensor* x, int64_t dim, const aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnSwiGlu(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnArgMaxGetWorkspaceSize(const aclTensor* self, int64_t dim, bool keepdim, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnArgMax(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnSoftplusGetWorkspaceSize(const aclTensor* self, const aclScalar* beta, const aclScalar* threshold,
    aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnSoftplus(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMoeGatingTopKV2GetWorkspaceSize(const aclTensor* x, const aclTensor* bias_optional,
    const aclTensor* input_ids_optional, const aclTensor* tid2eid_optional, int64_t k, int64_t k_group,
    int64_t group_count, int64_t group_select_mode, int64_t renorm, int64_t norm_type, bool out_flag,
    double routed_scaling_factor, double eps, const aclTensor* y_out, const aclTensor* expert_idx_out,
    const aclTensor* out_out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMoeGatingTopKV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMoeInitRoutingV4GetWorkspaceSize(const aclTensor* x, const aclTensor* expert_idx,
    const aclTensor* scale_optional, const aclTensor* offset_optional, const aclTensor* active_num_optional,
    const aclTensor* topk_weight_optional, int64_t expert_capacity, int64_t expert_num, int64_t drop_pad_mode,
    int64_t expert_tokens_num_type, bool expert_tokens_num_flag, int64_t quant_mode,
    const aclIntArray* active_expert_range_optional, int64_t row_idx_type, const aclTensor* expanded_x_out,
    const aclTensor* expanded_row_idx_out, const aclTensor* expert_tokens_count_or_cumsum_out,
    const aclTensor* expanded_scale_out, const aclTensor* expanded_topk_weight_out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnMoeInitRoutingV4(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnGroupedMatmulV5GetWorkspaceSize(const aclTensorList* x, const aclTensorList* weight,
    const aclTensorList* bias_optional, const aclTensorList* scale_optional, const aclTensorList* offset_optional,
    const aclTensorList* antiquant_scale_optional, const aclTensorList* antiquant_offset_optional,
    const aclTensorList* per_token_scale_optional, const aclTensor* group_list_optional,
    const aclTensorList* activation_input_optional, const aclTensorList* activation_quant_scale_optional,
    const aclTensorList* activation_quant_offset_optional, int64_t split_item, int64_t group_type,
    int64_t group_list_type, int64_t act_type, aclIntArray* tuning_config_optional, aclTensorList* out,
    aclTensorList* activation_feature_out_optional, aclTensorList* dyn_quant_scale_out_optional,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnGroupedMatmulV5(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnSwigluMxQuantGetWorkspaceSize(const aclTensor* x, const aclTensor* group_index_optional,
    int64_t activate_dim, bool activate_left, int64_t swiglu_mode, double clamp_limit, double glu_alpha,
    double glu_bias, int64_t group_mode, int64_t axis, int64_t dst_type, char* round_mode_optional, int64_t scale_alg,
    double max_dtype_value, const aclTensor* y_out, const aclTensor* mxscale_out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnSwigluMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMoeTokenUnpermuteGetWorkspaceSize(const aclTensor* permuted_tokens, const aclTensor* sorted_indices,
    const aclTensor* probs_optional, bool padded_mode, const aclIntArray* restore_shape_optional, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMoeTokenUnpermute(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnGroupedMatmulSwigluQuantV2GetWorkspaceSize(const aclTensor* x, const aclTensorList* weight,
    const aclTensorList* weight_scale, const aclTensorList* weight_assist_matrix, const aclTensor* bias,
    const aclTensor* x_scale, const aclTensor* smooth_scale, const aclTensor* group_list, int64_t dequant_mode,
    int64_t dequant_dtype, int64_t quant_mode, int64_t group_list_type, const aclIntArray* tuning_config_optional,
    aclTensor* output, aclTensor* output_scale, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnGroupedMatmulSwigluQuantV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnGroupedMatmulFinalizeRoutingV3GetWorkspaceSize(const aclTensor* x1, aclTensor* x2,
    const aclTensor* scale_optional, const aclTensor* bias_optional, const aclTensor* offset_optional,
    const aclTensor* antiquant_scale_optional, const aclTensor* antiquant_offset_optional,
    const aclTensor* pertoken_scale_optional, const aclTensor* group_list_optional,
    const aclTensor* shared_input_optional, const aclTensor* logit_optional, const aclTensor* row_index_optional,
    int64_t dtype, float shared_input_weight, int64_t shared_input_offset, bool transpose_x1, bool transpose_x2,
    int64_t group_list_type, const aclIntArray* tuning_config_optional, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnGroupedMatmulFinalizeRoutingV3(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMhcPreGetWorkspaceSize(const aclTensor* x, const aclTensor* phi, const aclTensor* alpha,
    const aclTensor* bias, const aclTensor* gamma_optional, double norm_eps, double hc_eps, aclTensor* h_in,
    aclTensor* h_post, aclTensor* h_res, aclTensor* inv_rms_optional, aclTensor* h_mix_optional,
    aclTensor* h_pre_optional, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMhcPre(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMhcSinkhornGetWorkspaceSize(const aclTensor* x, float eps, int64_t num_iters, aclTensor* output,
    aclTensor* norm_out, aclTensor* sum_out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMhcSinkhorn(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnMhcPostGetWorkspaceSize(const aclTensor* x, const aclTensor* h_res, const aclTensor* h_out,
    const aclTensor* h_post, aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor);
aclnnStatus aclnnMhcPost(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);
aclnnStatus aclnnQuantLightningIndexerGetWorkspaceSize(const aclTensor* query, const aclTensor* key,
    const aclTensor* weights, const aclTensor* query_dequant_scale, const aclTensor* key_dequant_scale,
    const aclTensor* actual_seq_lengths_query_optional, const aclTensor* actual_seq_lengths_key_optional,
    const aclTensor* block_table_optional, int64_t query_quant_mode, int64_t key_quant_mode,
    char* layout_query_optional, char* layout_key_optional, int64_t sparse_count, int64_t sparse_mode,
    int64_t pre_tokens, int64_t next_tokens, const aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor);
aclnnStatus aclnnQuantLightningIndexer(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream);

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
