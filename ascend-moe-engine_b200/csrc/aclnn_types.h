// Handle types behind the operator-library ABI (include/b200kv_aclnn.h), shared by the files that
// implement it. Not installed: callers see these only as opaque pointers.
#pragma once

#include <stdint.h>

#include <vector>

#include "b200kv_aclnn.h"

namespace b200kv {
constexpr aclnnStatus kErrNull = 161001;     // ACLNN_ERR_PARAM_NULLPTR (include/moe/core/op_table.hpp:142-147)
constexpr aclnnStatus kErrInvalid = 161002;  // ACLNN_ERR_PARAM_INVALID
constexpr aclnnStatus kErrRuntime = 361001;  // ACLNN_ERR_RUNTIME_ERROR

inline int64_t ElementBytes(aclDataType t) {
  switch (t) {
    case ACL_FLOAT32: case ACL_INT32: return 4;
    case ACL_FLOAT16: case ACL_BF16: case ACL_INT16: case ACL_UINT16: return 2;
    case ACL_INT64: case ACL_UINT64: case ACL_FLOAT64: return 8;
    default: return 1;
  }
}
}  // namespace b200kv

struct aclTensor {
  std::vector<int64_t> dims, strides, storage_dims;
  int64_t offset = 0;
  aclDataType dtype = ACL_DT_UNDEFINED;
  aclFormat format = ACL_FORMAT_ND;
  void* data = nullptr;
  int64_t Elements() const {
    int64_t n = 1;
    for (int64_t d : dims) n *= d;
    return n;
  }
  void* Address() const { return static_cast<char*>(data) + offset * b200kv::ElementBytes(dtype); }
};
struct aclTensorList {
  std::vector<aclTensor*> items;
};
struct aclIntArray {
  std::vector<int64_t> values;
};
struct aclScalar {
  unsigned char bytes[8] = {};
  aclDataType dtype = ACL_DT_UNDEFINED;
};
struct aclOpExecutor {
  // kScatter and kAttention are the KV path; kRmsNorm, kRope, kMxQuant and kIndexer the stages beside it, which work
  // for the shapes the path produces and consumes; kPlanOnly belongs to any other operator, whose launch
  // checks the pairing and enqueues nothing.
  enum Kind { kScatter, kAttention, kRmsNorm, kRope, kMxQuant, kIndexer, kPlanOnly } kind = kScatter;
  const char* op = nullptr;  // operator name the executor was planned for (kPlanOnly)
  bool repeatable = false;
  // scatter
  const aclTensor* key = nullptr;
  const aclTensor* value = nullptr;
  const aclTensor* slots = nullptr;
  aclTensor* key_cache = nullptr;
  aclTensor* value_cache = nullptr;
  // attention
  const aclTensor* query = nullptr;
  const aclTensor* query_rope = nullptr;
  const aclTensor* latent_cache = nullptr;
  const aclTensor* rope_cache = nullptr;
  const aclTensor* block_table = nullptr;
  const aclTensor* out = nullptr;
  const aclTensor* lse = nullptr;
  std::vector<int32_t> kv_len;
  int32_t batch = 0, heads = 0, block_size = 0;
  float scale = 0.0f;
  bool q_is_fused = false;  // query_rope directly follows query inside one 576-wide row
  uint64_t decode_ws = 0, q_pack_bytes = 0;
  // the stages beside the path (kRmsNorm, kRope, kMxQuant): their tensors in argument order, one scalar
  const aclTensor* stage_tensor[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  double stage_scalar = 0.0;
};
