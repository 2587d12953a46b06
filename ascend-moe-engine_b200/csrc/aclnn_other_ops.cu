// The operators of the reference's decode graph that lie outside the KV path (GEMMs, norms, RoPE,
// activation quantisation, MoE routing, the hyper-connection maps, the sparse indexer): exported so that
// an engine resolving all of its operators from this library (src/core/op_table.cpp:47-88 lists them,
// :95-121 resolves them) still builds and steps, but not implemented. A plan checks the arguments that
// the operator cannot do without, asks for no workspace and returns an executor that remembers which
// operator it belongs to; the launch checks that pairing and enqueues nothing, so the tensors such an
// operator should have written keep whatever they held. Signatures follow the plan-function types of
// include/moe/core/op_table.hpp (line given in include/b200kv_aclnn.h beside each declaration).
#include <cstring>
#include <new>

#include "aclnn_types.h"
#include "b200kv_aclnn.h"
#include "common.cuh"

using namespace b200kv;

namespace {

aclnnStatus PlanOnly(const char* op, const void* const* required, size_t n_required, uint64_t* workspace_size,
                     aclOpExecutor** executor) {
  if (workspace_size == nullptr || executor == nullptr) {
    SetLastError("%s: workspace_size and executor must be non-null", op);
    return kErrNull;
  }
  *executor = nullptr;
  for (size_t i = 0; i < n_required; ++i) {
    if (required[i] == nullptr) {
      SetLastError("%s: required argument %zu of its tensor list is null", op, i);
      return kErrNull;
    }
  }
  auto* exec = new (std::nothrow) aclOpExecutor();
  if (exec == nullptr) return kErrRuntime;
  exec->kind = aclOpExecutor::kPlanOnly;
  exec->op = op;
  *workspace_size = 0;
  *executor = exec;
  return 0;
}

aclnnStatus LaunchNothing(const char* op, void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                          aclrtStream stream) {
  (void)workspace;
  (void)workspace_size;
  (void)stream;
  if (executor == nullptr) {
    SetLastError("%s: executor is null", op);
    return kErrNull;
  }
  if (executor->kind != aclOpExecutor::kPlanOnly || executor->op != op) {
    SetLastError("%s: the executor was planned for %s", op, executor->op != nullptr ? executor->op : "a KV-path operator");
    return kErrInvalid;
  }
  if (!executor->repeatable) delete executor;  // a launch consumes an executor that was not marked repeatable
  return 0;
}

constexpr char kNameRmsNormDynamicMxQuant[] = "aclnnRmsNormDynamicMxQuant";
constexpr char kNameCast[] = "aclnnCast";
constexpr char kNameMatmul[] = "aclnnMatmul";
constexpr char kNameQuantMatmulV5[] = "aclnnQuantMatmulV5";
constexpr char kNameSigmoid[] = "aclnnSigmoid";
constexpr char kNameSqrt[] = "aclnnSqrt";
constexpr char kNameMul[] = "aclnnMul";
constexpr char kNameInplaceAdd[] = "aclnnInplaceAdd";
constexpr char kNameSwiGlu[] = "aclnnSwiGlu";
constexpr char kNameArgMax[] = "aclnnArgMax";
constexpr char kNameSoftplus[] = "aclnnSoftplus";
constexpr char kNameMoeGatingTopKV2[] = "aclnnMoeGatingTopKV2";
constexpr char kNameMoeInitRoutingV4[] = "aclnnMoeInitRoutingV4";
constexpr char kNameGroupedMatmulV5[] = "aclnnGroupedMatmulV5";
constexpr char kNameSwigluMxQuant[] = "aclnnSwigluMxQuant";
constexpr char kNameMoeTokenUnpermute[] = "aclnnMoeTokenUnpermute";
constexpr char kNameGroupedMatmulSwigluQuantV2[] = "aclnnGroupedMatmulSwigluQuantV2";
constexpr char kNameGroupedMatmulFinalizeRoutingV3[] = "aclnnGroupedMatmulFinalizeRoutingV3";
constexpr char kNameMhcPre[] = "aclnnMhcPre";
constexpr char kNameMhcSinkhorn[] = "aclnnMhcSinkhorn";
constexpr char kNameMhcPost[] = "aclnnMhcPost";

}  // namespace

// ---- the three stages beside the KV path: working for the shapes the path produces and consumes -----------
// aclnnRmsNorm on a 512-wide bf16 row (stage 6, kv_a_norm), aclnnApplyRotaryPosEmbV2 in mode "half" on 64-wide
// bf16 slices (stage 7, rope) and aclnnDynamicMxQuant to FP8 E4M3 with E8M0 block-32 scales on the last axis
// (stage 10, attn_quant) run the kernels of kv_stages.cu. The engine also uses these operators elsewhere with
// other shapes (a 4096-wide norm, for instance): those plans succeed as stand-ins like the operators below.
namespace {

constexpr char kNameRmsNorm[] = "aclnnRmsNorm";
constexpr char kNameApplyRotaryPosEmbV2[] = "aclnnApplyRotaryPosEmbV2";
constexpr char kNameDynamicMxQuant[] = "aclnnDynamicMxQuant";

bool Contiguous(const aclTensor* t) {
  int64_t expect = 1;
  for (int64_t i = static_cast<int64_t>(t->dims.size()) - 1; i >= 0; --i) {
    if (t->dims[i] != 1 && t->strides[i] != expect) return false;
    expect *= t->dims[i];
  }
  return true;
}

aclnnStatus NewStageExecutor(aclOpExecutor::Kind kind, const char* op, uint64_t* workspace_size, aclOpExecutor** executor,
                             aclOpExecutor** out) {
  auto* exec = new (std::nothrow) aclOpExecutor();
  if (exec == nullptr) return kErrRuntime;
  exec->kind = kind;
  exec->op = op;
  *workspace_size = 0;
  *executor = exec;
  *out = exec;
  return 0;
}

// Checks the executor of a stage launch; `*plan_only` tells the caller that the plan was a stand-in.
aclnnStatus CheckStageLaunch(const char* op, aclOpExecutor::Kind kind, aclOpExecutor* executor, bool* plan_only) {
  if (executor == nullptr) {
    SetLastError("%s: executor is null", op);
    return kErrNull;
  }
  *plan_only = executor->kind == aclOpExecutor::kPlanOnly;
  if ((executor->kind != kind && !*plan_only) || executor->op != op) {
    SetLastError("%s: the executor was planned for %s", op, executor->op != nullptr ? executor->op : "a KV-path operator");
    return kErrInvalid;
  }
  return 0;
}

aclnnStatus Finish(aclOpExecutor* executor, int32_t rc) {
  if (!executor->repeatable) delete executor;
  return rc == B200KV_OK ? 0 : (rc == B200KV_ERR_NULLPTR ? kErrNull : (rc == B200KV_ERR_INVALID ? kErrInvalid : kErrRuntime));
}

}  // namespace

extern "C" aclnnStatus aclnnRmsNormGetWorkspaceSize(const aclTensor* x, const aclTensor* gamma, double epsilon,
                                                    const aclTensor* y_out, const aclTensor* rstd_out,
                                                    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, gamma, y_out};
  const bool ours = x != nullptr && gamma != nullptr && y_out != nullptr && workspace_size != nullptr &&
                    executor != nullptr && x->dtype == ACL_BF16 && gamma->dtype == ACL_BF16 && y_out->dtype == ACL_BF16 &&
                    !x->dims.empty() && x->dims.back() == B200KV_LATENT_DIM && gamma->Elements() == B200KV_LATENT_DIM &&
                    y_out->Elements() == x->Elements() && Contiguous(x) && Contiguous(y_out) && Contiguous(gamma) &&
                    (rstd_out == nullptr || (rstd_out->dtype == ACL_FLOAT32 && Contiguous(rstd_out) &&
                                             rstd_out->Elements() == x->Elements() / B200KV_LATENT_DIM)) &&
                    epsilon >= 0.0;
  if (!ours) return PlanOnly(kNameRmsNorm, required, 3, workspace_size, executor);
  aclOpExecutor* exec = nullptr;
  if (aclnnStatus rc = NewStageExecutor(aclOpExecutor::kRmsNorm, kNameRmsNorm, workspace_size, executor, &exec)) return rc;
  exec->stage_tensor[0] = x;
  exec->stage_tensor[1] = gamma;
  exec->stage_tensor[2] = y_out;
  exec->stage_tensor[3] = rstd_out;
  exec->stage_scalar = epsilon;
  return 0;
}

extern "C" aclnnStatus aclnnRmsNorm(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  bool plan_only = false;
  if (aclnnStatus rc = CheckStageLaunch(kNameRmsNorm, aclOpExecutor::kRmsNorm, executor, &plan_only)) return rc;
  if (plan_only) return LaunchNothing(kNameRmsNorm, workspace, workspace_size, executor, stream);
  const aclTensor* x = executor->stage_tensor[0];
  const aclTensor* rstd = executor->stage_tensor[3];
  const int32_t rc = b200kv_rmsnorm512(x->Address(), B200KV_LATENT_DIM, executor->stage_tensor[1]->Address(),
                                       static_cast<float>(executor->stage_scalar), x->Elements() / B200KV_LATENT_DIM,
                                       executor->stage_tensor[2]->Address(), B200KV_LATENT_DIM,
                                       rstd != nullptr ? static_cast<float*>(rstd->Address()) : nullptr, stream);
  return Finish(executor, rc);
}

extern "C" aclnnStatus aclnnApplyRotaryPosEmbV2GetWorkspaceSize(aclTensor* query_ref, aclTensor* key_ref,
                                                                const aclTensor* cos, const aclTensor* sin, int64_t layout,
                                                                char* rotary_mode, uint64_t* workspace_size,
                                                                aclOpExecutor** executor) {
  (void)layout;
  const void* required[] = {query_ref, cos, sin};
  auto slices = [](const aclTensor* t) {  // [T, vectors, 64] bf16, contiguous
    return t->dtype == ACL_BF16 && t->dims.size() == 3 && t->dims[2] == B200KV_ROPE_DIM && Contiguous(t);
  };
  const bool ours = query_ref != nullptr && cos != nullptr && sin != nullptr && workspace_size != nullptr &&
                    executor != nullptr && rotary_mode != nullptr && std::strcmp(rotary_mode, "half") == 0 &&
                    slices(query_ref) && (key_ref == nullptr || (slices(key_ref) && key_ref->dims[0] == query_ref->dims[0])) &&
                    cos->dtype == ACL_BF16 && sin->dtype == ACL_BF16 && Contiguous(cos) && Contiguous(sin) &&
                    cos->Elements() == query_ref->dims[0] * B200KV_ROPE_DIM && sin->Elements() == cos->Elements();
  if (!ours) return PlanOnly(kNameApplyRotaryPosEmbV2, required, 3, workspace_size, executor);
  aclOpExecutor* exec = nullptr;
  if (aclnnStatus rc = NewStageExecutor(aclOpExecutor::kRope, kNameApplyRotaryPosEmbV2, workspace_size, executor, &exec)) {
    return rc;
  }
  exec->stage_tensor[0] = query_ref;
  exec->stage_tensor[1] = key_ref;
  exec->stage_tensor[2] = cos;
  exec->stage_tensor[3] = sin;
  return 0;
}

extern "C" aclnnStatus aclnnApplyRotaryPosEmbV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                                                aclrtStream stream) {
  bool plan_only = false;
  if (aclnnStatus rc = CheckStageLaunch(kNameApplyRotaryPosEmbV2, aclOpExecutor::kRope, executor, &plan_only)) return rc;
  if (plan_only) return LaunchNothing(kNameApplyRotaryPosEmbV2, workspace, workspace_size, executor, stream);
  const aclTensor* q = executor->stage_tensor[0];
  const aclTensor* k = executor->stage_tensor[1];
  const void* cos = executor->stage_tensor[2]->Address();
  const void* sin = executor->stage_tensor[3]->Address();
  int32_t rc = b200kv_rope_half64(q->Address(), q->dims[1] * B200KV_ROPE_DIM, B200KV_ROPE_DIM, cos, B200KV_ROPE_DIM, sin,
                                  B200KV_ROPE_DIM, q->dims[0], static_cast<int32_t>(q->dims[1]), stream);
  if (rc == B200KV_OK && k != nullptr) {
    rc = b200kv_rope_half64(k->Address(), k->dims[1] * B200KV_ROPE_DIM, B200KV_ROPE_DIM, cos, B200KV_ROPE_DIM, sin,
                            B200KV_ROPE_DIM, k->dims[0], static_cast<int32_t>(k->dims[1]), stream);
  }
  return Finish(executor, rc);
}

extern "C" aclnnStatus aclnnDynamicMxQuantGetWorkspaceSize(const aclTensor* x, int64_t axis, char* round_mode_optional,
                                                           int64_t dst_type, int64_t blocksize, int64_t scale_alg,
                                                           const aclTensor* y_out, const aclTensor* mxscale_out,
                                                           uint64_t* workspace_size, aclOpExecutor** executor) {
  (void)scale_alg;
  const void* required[] = {x, y_out, mxscale_out};
  const bool ours = x != nullptr && y_out != nullptr && mxscale_out != nullptr && workspace_size != nullptr &&
                    executor != nullptr && x->dtype == ACL_BF16 && y_out->dtype == ACL_FLOAT8_E4M3FN &&
                    dst_type == ACL_FLOAT8_E4M3FN && mxscale_out->dtype == ACL_FLOAT8_E8M0 && blocksize == 32 &&
                    !x->dims.empty() && (axis == -1 || axis == static_cast<int64_t>(x->dims.size()) - 1) &&
                    x->dims.back() % 32 == 0 && (round_mode_optional == nullptr || std::strcmp(round_mode_optional, "rint") == 0) &&
                    Contiguous(x) && Contiguous(y_out) && Contiguous(mxscale_out) && y_out->Elements() == x->Elements() &&
                    mxscale_out->Elements() == x->Elements() / 32;
  if (!ours) return PlanOnly(kNameDynamicMxQuant, required, 3, workspace_size, executor);
  aclOpExecutor* exec = nullptr;
  if (aclnnStatus rc = NewStageExecutor(aclOpExecutor::kMxQuant, kNameDynamicMxQuant, workspace_size, executor, &exec)) {
    return rc;
  }
  exec->stage_tensor[0] = x;
  exec->stage_tensor[1] = y_out;
  exec->stage_tensor[2] = mxscale_out;
  return 0;
}

extern "C" aclnnStatus aclnnDynamicMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                                           aclrtStream stream) {
  bool plan_only = false;
  if (aclnnStatus rc = CheckStageLaunch(kNameDynamicMxQuant, aclOpExecutor::kMxQuant, executor, &plan_only)) return rc;
  if (plan_only) return LaunchNothing(kNameDynamicMxQuant, workspace, workspace_size, executor, stream);
  const aclTensor* x = executor->stage_tensor[0];
  const int64_t cols = x->dims.back(), rows = x->Elements() / cols;
  const int32_t rc = b200kv_mx_quant_e4m3(x->Address(), cols, rows, cols, executor->stage_tensor[1]->Address(), cols,
                                          executor->stage_tensor[2]->Address(), cols / 32, stream);
  return Finish(executor, rc);
}

// aclnnQuantLightningIndexer for the decode step: one query token per sequence (TND query [T, N1, 128], T =
// sequences), paged FP8 keys [blocks, block_size, 1, 128] with their block table and lengths, out [T, 1, k].
// The positions come out best first, -1 beyond min(k, length). Other layouts plan as stand-ins.
namespace {
constexpr char kNameQuantLightningIndexer[] = "aclnnQuantLightningIndexer";
}

extern "C" aclnnStatus aclnnQuantLightningIndexerGetWorkspaceSize(
    const aclTensor* query, const aclTensor* key, const aclTensor* weights, const aclTensor* query_dequant_scale,
    const aclTensor* key_dequant_scale, const aclTensor* actual_seq_lengths_query_optional,
    const aclTensor* actual_seq_lengths_key_optional, const aclTensor* block_table_optional, int64_t query_quant_mode,
    int64_t key_quant_mode, char* layout_query_optional, char* layout_key_optional, int64_t sparse_count,
    int64_t sparse_mode, int64_t pre_tokens, int64_t next_tokens, const aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  (void)actual_seq_lengths_query_optional;
  (void)sparse_mode;
  (void)pre_tokens;
  (void)next_tokens;
  (void)layout_query_optional;
  const void* required[] = {query, key, weights, query_dequant_scale, key_dequant_scale, out};
  const bool ours =
      query != nullptr && key != nullptr && weights != nullptr && query_dequant_scale != nullptr &&
      key_dequant_scale != nullptr && out != nullptr && workspace_size != nullptr && executor != nullptr &&
      actual_seq_lengths_key_optional != nullptr && block_table_optional != nullptr && layout_key_optional != nullptr &&
      std::strcmp(layout_key_optional, "PA_BSND") == 0 && query_quant_mode == 0 && key_quant_mode == 0 &&
      query->dtype == ACL_FLOAT8_E4M3FN && key->dtype == ACL_FLOAT8_E4M3FN && query->dims.size() == 3 &&
      query->dims[2] == 128 && query->dims[1] >= 1 && query->dims[1] <= 64 && key->dims.size() == 4 && key->dims[2] == 1 &&
      key->dims[3] == 128 && Contiguous(query) && Contiguous(key) && weights->dtype == ACL_BF16 &&
      weights->Elements() == query->dims[0] * query->dims[1] && Contiguous(weights) &&
      query_dequant_scale->dtype == ACL_FLOAT32 && query_dequant_scale->Elements() == weights->Elements() &&
      Contiguous(query_dequant_scale) && key_dequant_scale->dtype == ACL_FLOAT32 &&
      key_dequant_scale->Elements() == key->dims[0] * key->dims[1] && Contiguous(key_dequant_scale) &&
      actual_seq_lengths_key_optional->dtype == ACL_INT32 && actual_seq_lengths_key_optional->Elements() == query->dims[0] &&
      block_table_optional->dtype == ACL_INT32 && block_table_optional->dims.size() == 2 &&
      block_table_optional->dims[0] == query->dims[0] && Contiguous(block_table_optional) && out->dtype == ACL_INT32 &&
      out->Elements() == query->dims[0] * sparse_count && Contiguous(out) && sparse_count >= 1 && sparse_count <= 2048;
  if (!ours) return PlanOnly(kNameQuantLightningIndexer, required, 6, workspace_size, executor);
  aclOpExecutor* exec = nullptr;
  if (aclnnStatus rc = NewStageExecutor(aclOpExecutor::kIndexer, kNameQuantLightningIndexer, workspace_size, executor, &exec)) {
    return rc;
  }
  exec->stage_tensor[0] = query;
  exec->stage_tensor[1] = key;
  exec->stage_tensor[2] = weights;
  exec->stage_tensor[3] = query_dequant_scale;
  exec->stage_tensor[4] = key_dequant_scale;
  exec->stage_tensor[5] = actual_seq_lengths_key_optional;
  exec->stage_tensor[6] = block_table_optional;
  exec->stage_tensor[7] = out;
  exec->stage_scalar = static_cast<double>(sparse_count);
  // scores for the longest sequence the table can address, then one count per sequence
  const int64_t batch = query->dims[0];
  const int64_t max_len = block_table_optional->dims[1] * key->dims[1];
  *workspace_size = b200kv_indexer_workspace_bytes(static_cast<int32_t>(batch), max_len) + ((batch * 4 + 255) & ~255ll);
  return 0;
}

extern "C" aclnnStatus aclnnQuantLightningIndexer(void* workspace, uint64_t workspace_size, aclOpExecutor* executor,
                                                  aclrtStream stream) {
  bool plan_only = false;
  if (aclnnStatus rc = CheckStageLaunch(kNameQuantLightningIndexer, aclOpExecutor::kIndexer, executor, &plan_only)) return rc;
  if (plan_only) return LaunchNothing(kNameQuantLightningIndexer, workspace, workspace_size, executor, stream);
  const aclTensor* query = executor->stage_tensor[0];
  const aclTensor* key = executor->stage_tensor[1];
  const aclTensor* table = executor->stage_tensor[6];
  const int64_t batch = query->dims[0];
  const int64_t max_len = table->dims[1] * key->dims[1];
  const size_t score_bytes = b200kv_indexer_workspace_bytes(static_cast<int32_t>(batch), max_len);
  if (workspace == nullptr || workspace_size < score_bytes + static_cast<size_t>(batch) * 4) {
    SetLastError("%s: workspace of %zu bytes required", kNameQuantLightningIndexer, score_bytes + static_cast<size_t>(batch) * 4);
    return workspace == nullptr ? kErrNull : kErrInvalid;
  }
  b200kv_indexer_args a{};
  a.q = query->Address();
  a.q_scale = static_cast<const float*>(executor->stage_tensor[3]->Address());
  a.weights = executor->stage_tensor[2]->Address();
  a.heads = static_cast<int32_t>(query->dims[1]);
  a.key_pool = key->Address();
  a.key_stride = 128;
  a.k_scale = static_cast<const float*>(executor->stage_tensor[4]->Address());
  a.pool_rows = key->dims[0] * key->dims[1];
  a.block_table = static_cast<const int32_t*>(table->Address());
  a.max_blocks = table->dims[1];
  a.kv_len = static_cast<const int32_t*>(executor->stage_tensor[5]->Address());
  a.batch = static_cast<int32_t>(batch);
  a.block_size = static_cast<int32_t>(key->dims[1]);
  a.max_kv_len = max_len;
  a.k = static_cast<int32_t>(executor->stage_scalar);
  a.index_out = static_cast<int32_t*>(executor->stage_tensor[7]->Address());
  a.n_selected_out = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + score_bytes);
  a.workspace = workspace;
  a.workspace_bytes = score_bytes;
  return Finish(executor, b200kv_indexer_topk(&a, stream, nullptr));
}

// ---- every other operator: plan checks, launch enqueues nothing ------------------------------------------------

extern "C" aclnnStatus aclnnRmsNormDynamicMxQuantGetWorkspaceSize(const aclTensor* x, const aclTensor* gamma,
    const aclTensor* beta, double epsilon, int64_t scale_alg, char* round_mode, int64_t dst_type, bool output_rstd,
    aclTensor* y_out, aclTensor* mxscale_out, aclTensor* rstd_out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x, gamma, y_out, mxscale_out};
  return PlanOnly(kNameRmsNormDynamicMxQuant, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnRmsNormDynamicMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameRmsNormDynamicMxQuant, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnCastGetWorkspaceSize(const aclTensor* self, aclDataType dtype, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self, out};
  return PlanOnly(kNameCast, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnCast(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameCast, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMatmulGetWorkspaceSize(const aclTensor* self, const aclTensor* mat2, aclTensor* out,
    int8_t cube_math_type, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self, mat2, out};
  return PlanOnly(kNameMatmul, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMatmul(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMatmul, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnQuantMatmulV5GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2,
    const aclTensor* x1_scale, const aclTensor* x2_scale, const aclTensor* y_scale, const aclTensor* x1_offset,
    const aclTensor* x2_offset, const aclTensor* y_offset, const aclTensor* bias, bool transpose_x1,
    bool transpose_x2, int64_t group_size, aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x1, x2, out};
  return PlanOnly(kNameQuantMatmulV5, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnQuantMatmulV5(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameQuantMatmulV5, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnSigmoidGetWorkspaceSize(const aclTensor* self, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {self, out};
  return PlanOnly(kNameSigmoid, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnSigmoid(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameSigmoid, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnSqrtGetWorkspaceSize(const aclTensor* self, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {self, out};
  return PlanOnly(kNameSqrt, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnSqrt(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameSqrt, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMulGetWorkspaceSize(const aclTensor* self, const aclTensor* other, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self, other, out};
  return PlanOnly(kNameMul, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMul(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMul, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnInplaceAddGetWorkspaceSize(const aclTensor* self_ref, const aclTensor* other,
    const aclScalar* alpha, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self_ref, other, alpha};
  return PlanOnly(kNameInplaceAdd, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnInplaceAdd(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameInplaceAdd, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnSwiGluGetWorkspaceSize(const aclTensor* x, int64_t dim, const aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, out};
  return PlanOnly(kNameSwiGlu, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnSwiGlu(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameSwiGlu, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnArgMaxGetWorkspaceSize(const aclTensor* self, int64_t dim, bool keepdim, aclTensor* out,
    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self, out};
  return PlanOnly(kNameArgMax, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnArgMax(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameArgMax, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnSoftplusGetWorkspaceSize(const aclTensor* self, const aclScalar* beta,
    const aclScalar* threshold, aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {self, beta, threshold, out};
  return PlanOnly(kNameSoftplus, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnSoftplus(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameSoftplus, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMoeGatingTopKV2GetWorkspaceSize(const aclTensor* x, const aclTensor* bias_optional,
    const aclTensor* input_ids_optional, const aclTensor* tid2eid_optional, int64_t k, int64_t k_group,
    int64_t group_count, int64_t group_select_mode, int64_t renorm, int64_t norm_type, bool out_flag,
    double routed_scaling_factor, double eps, const aclTensor* y_out, const aclTensor* expert_idx_out,
    const aclTensor* out_out, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, y_out, expert_idx_out};
  return PlanOnly(kNameMoeGatingTopKV2, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMoeGatingTopKV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMoeGatingTopKV2, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMoeInitRoutingV4GetWorkspaceSize(const aclTensor* x, const aclTensor* expert_idx,
    const aclTensor* scale_optional, const aclTensor* offset_optional, const aclTensor* active_num_optional,
    const aclTensor* topk_weight_optional, int64_t expert_capacity, int64_t expert_num, int64_t drop_pad_mode,
    int64_t expert_tokens_num_type, bool expert_tokens_num_flag, int64_t quant_mode,
    const aclIntArray* active_expert_range_optional, int64_t row_idx_type, const aclTensor* expanded_x_out,
    const aclTensor* expanded_row_idx_out, const aclTensor* expert_tokens_count_or_cumsum_out,
    const aclTensor* expanded_scale_out, const aclTensor* expanded_topk_weight_out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x, expert_idx, expanded_x_out, expanded_row_idx_out, expert_tokens_count_or_cumsum_out};
  return PlanOnly(kNameMoeInitRoutingV4, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMoeInitRoutingV4(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMoeInitRoutingV4, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnGroupedMatmulV5GetWorkspaceSize(const aclTensorList* x, const aclTensorList* weight,
    const aclTensorList* bias_optional, const aclTensorList* scale_optional, const aclTensorList* offset_optional,
    const aclTensorList* antiquant_scale_optional, const aclTensorList* antiquant_offset_optional,
    const aclTensorList* per_token_scale_optional, const aclTensor* group_list_optional,
    const aclTensorList* activation_input_optional, const aclTensorList* activation_quant_scale_optional,
    const aclTensorList* activation_quant_offset_optional, int64_t split_item, int64_t group_type,
    int64_t group_list_type, int64_t act_type, aclIntArray* tuning_config_optional, aclTensorList* out,
    aclTensorList* activation_feature_out_optional, aclTensorList* dyn_quant_scale_out_optional,
    uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, weight, out};
  return PlanOnly(kNameGroupedMatmulV5, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnGroupedMatmulV5(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameGroupedMatmulV5, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnSwigluMxQuantGetWorkspaceSize(const aclTensor* x, const aclTensor* group_index_optional,
    int64_t activate_dim, bool activate_left, int64_t swiglu_mode, double clamp_limit, double glu_alpha,
    double glu_bias, int64_t group_mode, int64_t axis, int64_t dst_type, char* round_mode_optional, int64_t scale_alg,
    double max_dtype_value, const aclTensor* y_out, const aclTensor* mxscale_out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x, y_out, mxscale_out};
  return PlanOnly(kNameSwigluMxQuant, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnSwigluMxQuant(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameSwigluMxQuant, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMoeTokenUnpermuteGetWorkspaceSize(const aclTensor* permuted_tokens,
    const aclTensor* sorted_indices, const aclTensor* probs_optional, bool padded_mode,
    const aclIntArray* restore_shape_optional, aclTensor* out, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {permuted_tokens, sorted_indices, out};
  return PlanOnly(kNameMoeTokenUnpermute, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMoeTokenUnpermute(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMoeTokenUnpermute, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnGroupedMatmulSwigluQuantV2GetWorkspaceSize(const aclTensor* x,
    const aclTensorList* weight, const aclTensorList* weight_scale, const aclTensorList* weight_assist_matrix,
    const aclTensor* bias, const aclTensor* x_scale, const aclTensor* smooth_scale, const aclTensor* group_list,
    int64_t dequant_mode, int64_t dequant_dtype, int64_t quant_mode, int64_t group_list_type,
    const aclIntArray* tuning_config_optional, aclTensor* output, aclTensor* output_scale, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x, weight, weight_scale, group_list, output, output_scale};
  return PlanOnly(kNameGroupedMatmulSwigluQuantV2, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnGroupedMatmulSwigluQuantV2(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameGroupedMatmulSwigluQuantV2, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnGroupedMatmulFinalizeRoutingV3GetWorkspaceSize(const aclTensor* x1, aclTensor* x2,
    const aclTensor* scale_optional, const aclTensor* bias_optional, const aclTensor* offset_optional,
    const aclTensor* antiquant_scale_optional, const aclTensor* antiquant_offset_optional,
    const aclTensor* pertoken_scale_optional, const aclTensor* group_list_optional,
    const aclTensor* shared_input_optional, const aclTensor* logit_optional, const aclTensor* row_index_optional,
    int64_t dtype, float shared_input_weight, int64_t shared_input_offset, bool transpose_x1, bool transpose_x2,
    int64_t group_list_type, const aclIntArray* tuning_config_optional, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x1, x2, out};
  return PlanOnly(kNameGroupedMatmulFinalizeRoutingV3, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnGroupedMatmulFinalizeRoutingV3(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameGroupedMatmulFinalizeRoutingV3, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMhcPreGetWorkspaceSize(const aclTensor* x, const aclTensor* phi, const aclTensor* alpha,
    const aclTensor* bias, const aclTensor* gamma_optional, double norm_eps, double hc_eps, aclTensor* h_in,
    aclTensor* h_post, aclTensor* h_res, aclTensor* inv_rms_optional, aclTensor* h_mix_optional,
    aclTensor* h_pre_optional, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, phi, alpha, bias, h_in, h_post, h_res};
  return PlanOnly(kNameMhcPre, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMhcPre(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMhcPre, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMhcSinkhornGetWorkspaceSize(const aclTensor* x, float eps, int64_t num_iters,
    aclTensor* output, aclTensor* norm_out, aclTensor* sum_out, uint64_t* workspace_size, aclOpExecutor** executor) {
  const void* required[] = {x, output};
  return PlanOnly(kNameMhcSinkhorn, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMhcSinkhorn(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMhcSinkhorn, workspace, workspace_size, executor, stream);
}

extern "C" aclnnStatus aclnnMhcPostGetWorkspaceSize(const aclTensor* x, const aclTensor* h_res,
    const aclTensor* h_out, const aclTensor* h_post, aclTensor* out, uint64_t* workspace_size,
    aclOpExecutor** executor) {
  const void* required[] = {x, h_res, h_out, h_post, out};
  return PlanOnly(kNameMhcPost, required, sizeof(required) / sizeof(required[0]), workspace_size, executor);
}
extern "C" aclnnStatus aclnnMhcPost(void* workspace, uint64_t workspace_size, aclOpExecutor* executor, aclrtStream stream) {
  return LaunchNothing(kNameMhcPost, workspace, workspace_size, executor, stream);
}

