// Test infrastructure, not product code: the reference engine's own host code for the KV path, compiled
// where it lies, driving this repository's library through the operator ABI.
//
// The reference resolves its operators with dlsym (OpTable, src/core/op_table.cpp:95-159), plans each
// stage once (PlanAclnnOp<>, include/moe/core/op_table.hpp:1114-1133), keeps the executor in a
// StaticOpSlot (src/core/op_table.cpp:230-270) and, per layer, repoints the caches and launches
// (src/pipeline/pipeline.cpp:390-416). Memory and streams come from AclDeviceOps
// (src/core/device_ops.cpp:96-262). This driver does exactly that with the reference's classes, with the
// argument lists of stages 8 and 9 of the reference's Build (src/pipeline/pipeline.cpp:226-248) and the
// descriptor shapes of StaticArenaManager::CreateDescriptors (src/memory/static_arena_manager.cpp:480-497,
// 567-588), but linked against libb200kv.so instead of the vendor's operator library. The Python test
// writes the inputs, runs this binary on the GPU and checks its outputs against the oracle.
//
//   op_slot_probe <input file> <output file>
//
// Input (little endian): int64 header {layers, blocks, block_size, context, heads, scale_bits(float in low
// 32 bits), slot}; then per layer: latent pool bf16 [blocks*block_size][512], rope pool bf16
// [blocks*block_size][64], new latent row [512], new rope row [64], q_latent [heads][512], q_rope
// [heads][64]; then the block table int32 [blocks]. The new row of every layer is appended at pool row
// `slot` (the engine's batch-1 loop uses the position, which is the same row under an identity table) and
// attention runs over `context` tokens.
// Output: per layer attention output bf16 [heads][512], then per layer the pool row at the slot
// (latent [512] + rope [64]) read back after the step, then one line of text per resolved operator.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "moe/core/device_ops.hpp"
#include "moe/core/error.hpp"
#include "moe/core/op_table.hpp"

using namespace ascend_moe;

namespace {

constexpr int kLatent = 512;
constexpr int kRope = 64;
constexpr int32_t kBf16 = 27;   // ACL_BF16
constexpr int32_t kInt32 = 3;   // ACL_INT32
constexpr int32_t kFloat = 0;   // ACL_FLOAT
// Positions of the repointed tensors in the operators' argument lists (include/moe/pipeline/pipeline.hpp:177-184).
constexpr size_t kScatterKeyCache = 1, kScatterValueCache = 4, kFiaKeyList = 1, kFiaValueList = 2, kFiaKeyRope = 25;

aclTensor* Tensor(const std::vector<int64_t>& dims, int32_t dtype, void* data) {
  std::vector<int64_t> strides(dims.size(), 1);
  for (int64_t i = static_cast<int64_t>(dims.size()) - 2; i >= 0; --i) strides[i] = strides[i + 1] * dims[i + 1];
  aclTensor* t = aclCreateTensor(dims.data(), dims.size(), static_cast<aclDataType>(dtype), strides.data(), 0,
                                 ACL_FORMAT_ND, dims.data(), dims.size(), data);
  if (t == nullptr) throw Dsv4Error("aclCreateTensor returned null");
  return t;
}

template <typename T>
std::vector<T> ReadArray(std::ifstream& in, size_t count) {
  std::vector<T> v(count);
  in.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(count * sizeof(T)));
  if (!in) throw Dsv4Error("input file is shorter than its header says");
  return v;
}

int Run(const std::string& in_path, const std::string& out_path) {
  std::ifstream in(in_path, std::ios::binary);
  if (!in) throw Dsv4Error("cannot open " + in_path);
  const std::vector<int64_t> header = ReadArray<int64_t>(in, 7);
  const int64_t layers = header[0], blocks = header[1], block_size = header[2], context = header[3], heads = header[4];
  float scale;
  const uint32_t scale_bits = static_cast<uint32_t>(header[5]);
  std::memcpy(&scale, &scale_bits, 4);
  const int64_t rows = blocks * block_size;
  if (layers < 1 || rows < context || context < 1 || heads < 1 || header[6] < 0 || header[6] >= rows) {
    throw Dsv4Error("implausible header");
  }

  AclDeviceOps device(0);
  OpTable table;
  DeviceStream stream = device.CreateStream();

  // Device buffers. One allocation per role, all layers of a pool contiguous (layer-major, as
  // src/memory/static_arena_manager.cpp:315-318 lays them out).
  const size_t latent_layer = static_cast<size_t>(rows) * kLatent * 2, rope_layer = static_cast<size_t>(rows) * kRope * 2;
  auto* latent_pool = static_cast<uint8_t*>(device.DeviceMalloc(latent_layer * layers));
  auto* rope_pool = static_cast<uint8_t*>(device.DeviceMalloc(rope_layer * layers));
  auto* new_latent = static_cast<uint8_t*>(device.DeviceMalloc(kLatent * 2));
  auto* new_rope = static_cast<uint8_t*>(device.DeviceMalloc(kRope * 2));
  auto* q_latent = static_cast<uint8_t*>(device.DeviceMalloc(static_cast<size_t>(heads) * kLatent * 2));
  auto* q_rope = static_cast<uint8_t*>(device.DeviceMalloc(static_cast<size_t>(heads) * kRope * 2));
  auto* attn_out = static_cast<uint8_t*>(device.DeviceMalloc(static_cast<size_t>(heads) * kLatent * 2));
  auto* lse = static_cast<uint8_t*>(device.DeviceMalloc(static_cast<size_t>(heads) * 4));
  auto* slot_dev = static_cast<uint8_t*>(device.DeviceMalloc(4));
  auto* table_dev = static_cast<uint8_t*>(device.DeviceMalloc(static_cast<size_t>(blocks) * 4));

  struct LayerInput {
    std::vector<uint16_t> latent, rope, new_latent, new_rope, q_latent, q_rope;
  };
  std::vector<LayerInput> inputs(layers);
  for (int64_t l = 0; l < layers; ++l) {
    inputs[l].latent = ReadArray<uint16_t>(in, static_cast<size_t>(rows) * kLatent);
    inputs[l].rope = ReadArray<uint16_t>(in, static_cast<size_t>(rows) * kRope);
    inputs[l].new_latent = ReadArray<uint16_t>(in, kLatent);
    inputs[l].new_rope = ReadArray<uint16_t>(in, kRope);
    inputs[l].q_latent = ReadArray<uint16_t>(in, static_cast<size_t>(heads) * kLatent);
    inputs[l].q_rope = ReadArray<uint16_t>(in, static_cast<size_t>(heads) * kRope);
    device.MemcpySync(latent_pool + latent_layer * l, latent_layer, inputs[l].latent.data(), latent_layer,
                      MemcpyKind::kHostToDevice);
    device.MemcpySync(rope_pool + rope_layer * l, rope_layer, inputs[l].rope.data(), rope_layer, MemcpyKind::kHostToDevice);
  }
  const std::vector<int32_t> block_table = ReadArray<int32_t>(in, static_cast<size_t>(blocks));
  device.MemcpySync(table_dev, blocks * 4, block_table.data(), blocks * 4, MemcpyKind::kHostToDevice);

  // Descriptors with the reference's shapes.
  aclTensor* t_kv_latent = Tensor({1, kLatent}, kBf16, new_latent);
  aclTensor* t_k_rope = Tensor({1, 1, kRope}, kBf16, new_rope);
  aclTensor* t_latent_cache = Tensor({blocks, block_size, 1, kLatent}, kBf16, latent_pool);
  aclTensor* t_rope_cache = Tensor({blocks, block_size, 1, kRope}, kBf16, rope_pool);
  aclTensor* t_slot = Tensor({1}, kInt32, slot_dev);
  aclTensor* t_q_latent = Tensor({1, heads, kLatent}, kBf16, q_latent);
  aclTensor* t_q_rope = Tensor({1, heads, kRope}, kBf16, q_rope);
  aclTensor* t_key = Tensor({blocks, block_size, 1, kLatent}, kBf16, latent_pool);
  aclTensor* t_value = Tensor({blocks, block_size, 1, kLatent}, kBf16, latent_pool);
  aclTensor* t_key_rope = Tensor({blocks, block_size, 1, kRope}, kBf16, rope_pool);
  aclTensor* t_block_table = Tensor({1, blocks}, kInt32, table_dev);
  aclTensor* t_out = Tensor({1, heads, kLatent}, kBf16, attn_out);
  aclTensor* t_lse = Tensor({1, heads, 1}, kFloat, lse);
  const aclTensor* key_items[1] = {t_key};
  const aclTensor* value_items[1] = {t_value};
  aclTensorList* key_list = aclCreateTensorList(key_items, 1);
  aclTensorList* value_list = aclCreateTensorList(value_items, 1);
  const int64_t one = 1;
  aclIntArray* seq_q = aclCreateIntArray(&one, 1);
  aclIntArray* seq_kv = aclCreateIntArray(&context, 1);

  // Plan once (stages 8 and 9 of the reference's Build), keep the executors.
  char cache_mode[] = "Norm";
  char layout[] = "TND";
  StaticOpSlot scatter, attention;
  aclOpExecutor* executor = nullptr;
  uint64_t workspace_bytes = PlanAclnnOp<ScatterPaKvCachePlanFn>(
      table, OpId::kScatterPaKvCache, &executor, t_kv_latent, t_latent_cache, t_slot, t_k_rope, t_rope_cache, nullptr,
      nullptr, nullptr, cache_mode, nullptr, nullptr, nullptr);
  scatter.Adopt(OpId::kScatterPaKvCache, "kv_cache_write", workspace_bytes, executor);
  workspace_bytes = PlanAclnnOp<FusedInferAttentionScoreV5PlanFn>(
      table, OpId::kFusedInferAttentionScoreV5, &executor, t_q_latent, key_list, value_list, nullptr, nullptr, seq_q,
      seq_kv, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, t_block_table, nullptr, nullptr, nullptr,
      nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, t_q_rope, t_key_rope, nullptr, nullptr, nullptr, nullptr,
      nullptr, heads, static_cast<double>(scale), int64_t{65536}, int64_t{0}, layout, int64_t{1}, int64_t{3},
      int64_t{0}, block_size, int64_t{0}, false, int64_t{0}, int64_t{0}, int64_t{0}, int64_t{0}, t_out, t_lse);
  attention.Adopt(OpId::kFusedInferAttentionScoreV5, "attention", workspace_bytes, executor);
  const uint64_t shared_workspace = std::max<uint64_t>(scatter.workspace_size(), attention.workspace_size());
  void* workspace = shared_workspace > 0 ? device.DeviceMalloc(shared_workspace) : nullptr;

  // One decode step: the slot goes to the device once (src/pipeline/pipeline.cpp:515-519), then per layer
  // the address swaps and the two launches.
  const int32_t slot = static_cast<int32_t>(header[6]);
  device.MemcpySync(slot_dev, 4, &slot, 4, MemcpyKind::kHostToDevice);
  std::vector<std::vector<uint16_t>> outs(layers), rows_back(layers);
  for (int64_t l = 0; l < layers; ++l) {
    device.MemcpySync(new_latent, kLatent * 2, inputs[l].new_latent.data(), kLatent * 2, MemcpyKind::kHostToDevice);
    device.MemcpySync(new_rope, kRope * 2, inputs[l].new_rope.data(), kRope * 2, MemcpyKind::kHostToDevice);
    device.MemcpySync(q_latent, heads * kLatent * 2, inputs[l].q_latent.data(), heads * kLatent * 2, MemcpyKind::kHostToDevice);
    device.MemcpySync(q_rope, heads * kRope * 2, inputs[l].q_rope.data(), heads * kRope * 2, MemcpyKind::kHostToDevice);
    uint8_t* latent = latent_pool + latent_layer * l;
    uint8_t* rope = rope_pool + rope_layer * l;
    scatter.SetAddress(kScatterKeyCache, t_latent_cache, latent);
    scatter.SetAddress(kScatterValueCache, t_rope_cache, rope);
    attention.SetTensorListAddress(kFiaKeyList, 0, key_list, latent);
    attention.SetTensorListAddress(kFiaValueList, 0, value_list, latent);
    attention.SetAddress(kFiaKeyRope, t_key_rope, rope);
    scatter.Launch(table, workspace, stream);
    attention.Launch(table, workspace, stream);
    device.SynchronizeStream(stream);
    outs[l].resize(static_cast<size_t>(heads) * kLatent);
    device.MemcpySync(outs[l].data(), outs[l].size() * 2, attn_out, outs[l].size() * 2, MemcpyKind::kDeviceToHost);
    rows_back[l].resize(kLatent + kRope);
    device.MemcpySync(rows_back[l].data(), kLatent * 2, latent + static_cast<size_t>(slot) * kLatent * 2, kLatent * 2,
                      MemcpyKind::kDeviceToHost);
    device.MemcpySync(rows_back[l].data() + kLatent, kRope * 2, rope + static_cast<size_t>(slot) * kRope * 2, kRope * 2,
                      MemcpyKind::kDeviceToHost);
  }

  std::ofstream out(out_path, std::ios::binary);
  for (int64_t l = 0; l < layers; ++l) out.write(reinterpret_cast<const char*>(outs[l].data()), outs[l].size() * 2);
  for (int64_t l = 0; l < layers; ++l) out.write(reinterpret_cast<const char*>(rows_back[l].data()), rows_back[l].size() * 2);
  const std::string inventory = table.DescribeInventory();
  out.write(inventory.data(), static_cast<std::streamsize>(inventory.size()));
  if (!out) throw Dsv4Error("cannot write " + out_path);

  scatter.Reset();
  attention.Reset();
  device.DestroyStream(stream);
  std::cout << "op_slot_probe: " << layers << " layers, context " << context << ", backend " << device.backend_name()
            << ", device allocations " << device.DeviceAllocationCount() << "\n";
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: op_slot_probe <input file> <output file>\n");
    return 2;
  }
  try {
    return Run(argv[1], argv[2]);
  } catch (const std::exception& error) {
    std::fprintf(stderr, "op_slot_probe: %s\n", error.what());
    return 1;
  }
}
