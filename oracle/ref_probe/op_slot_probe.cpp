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
// 567-588), but linked against libb200kv.so instead of the vendor's operator library. Memory and descriptors
// come from the reference's StaticMemoryArena (src/memory/static_arena.cpp): the four KV spans are reserved,
// one Commit allocates them, the descriptors and the key / value lists are made by CreateTensor /
// CreateTensorList / CreateIntArray in CreateDescriptors' order (the list copies go through the operator
// library's shape getters, whose results the arena owns and deletes), the workspace by NoteWorkspace /
// CommitWorkspace, and the arena is sealed before the step. The Python test
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
#include "moe/memory/static_arena.hpp"

using namespace ascend_moe;

namespace {

constexpr int kLatent = 512;
constexpr int kRope = 64;
constexpr int32_t kBf16 = 27;   // ACL_BF16
constexpr int32_t kInt32 = 3;   // ACL_INT32
constexpr int32_t kFloat = 0;   // ACL_FLOAT
// Positions of the repointed tensors in the operators' argument lists (include/moe/pipeline/pipeline.hpp:177-184).
constexpr size_t kScatterKeyCache = 1, kScatterValueCache = 4, kFiaKeyList = 1, kFiaValueList = 2, kFiaKeyRope = 25;

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

  // The KV spans as the reference lays them out: two layer-major caches, the block table and the slot
  // (src/memory/static_arena_manager.cpp:298-300, 315-318), plus the step's activations, all carved from the
  // reference's arena with ONE device allocation.
  StaticMemoryArena arena(device);
  const size_t latent_layer = static_cast<size_t>(rows) * kLatent * 2, rope_layer = static_cast<size_t>(rows) * kRope * 2;
  const ArenaHandle h_table = arena.Reserve("kv.block_table", static_cast<size_t>(blocks) * 4);
  const ArenaHandle h_slot = arena.Reserve("kv.slot_mapping", 4);
  const ArenaHandle h_latent = arena.Reserve("kv.latent_cache", latent_layer * layers);
  const ArenaHandle h_rope = arena.Reserve("kv.rope_cache", rope_layer * layers);
  const ArenaHandle h_new_latent = arena.Reserve("attn.kv_latent_normed", kLatent * 2);
  const ArenaHandle h_new_rope = arena.Reserve("attn.k_rope", kRope * 2);
  const ArenaHandle h_q_latent = arena.Reserve("attn.q_latent", static_cast<size_t>(heads) * kLatent * 2);
  const ArenaHandle h_q_rope = arena.Reserve("attn.q_rope", static_cast<size_t>(heads) * kRope * 2);
  const ArenaHandle h_out = arena.Reserve("attn.out", static_cast<size_t>(heads) * kLatent * 2);
  const ArenaHandle h_lse = arena.Reserve("attn.lse", static_cast<size_t>(heads) * 4);
  const uint64_t allocations_before = device.DeviceAllocationCount();
  arena.Commit();
  if (device.DeviceAllocationCount() != allocations_before + 1) throw Dsv4Error("Commit made more than one allocation");
  auto* latent_pool = arena.AddressAs<uint8_t>(h_latent);
  auto* rope_pool = arena.AddressAs<uint8_t>(h_rope);
  auto* new_latent = arena.AddressAs<uint8_t>(h_new_latent);
  auto* new_rope = arena.AddressAs<uint8_t>(h_new_rope);
  auto* q_latent = arena.AddressAs<uint8_t>(h_q_latent);
  auto* q_rope = arena.AddressAs<uint8_t>(h_q_rope);
  auto* attn_out = arena.AddressAs<uint8_t>(h_out);
  auto* lse = arena.AddressAs<uint8_t>(h_lse);
  auto* slot_dev = arena.AddressAs<uint8_t>(h_slot);
  auto* table_dev = arena.AddressAs<uint8_t>(h_table);

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

  // Descriptors with the reference's shapes and labels, in the order of CreateDescriptors
  // (src/memory/static_arena_manager.cpp:480-497, 567-588).
  aclTensor* t_q_latent = arena.CreateTensor("q_latent", {1, heads, kLatent}, kBf16, q_latent);
  aclTensor* t_q_rope = arena.CreateTensor("q_rope", {1, heads, kRope}, kBf16, q_rope);
  aclTensor* t_kv_latent = arena.CreateTensor("kv_latent_normed", {1, kLatent}, kBf16, new_latent);
  aclTensor* t_k_rope = arena.CreateTensor("k_rope", {1, 1, kRope}, kBf16, new_rope);
  aclTensor* t_out = arena.CreateTensor("attn_out", {1, heads, kLatent}, kBf16, attn_out);
  aclTensor* t_lse = arena.CreateTensor("attn_lse", {1, heads, 1}, kFloat, lse);
  aclTensor* t_latent_cache = arena.CreateTensor("kv_latent_cache", {blocks, block_size, 1, kLatent}, kBf16, latent_pool);
  aclTensor* t_rope_cache = arena.CreateTensor("kv_rope_cache", {blocks, block_size, 1, kRope}, kBf16, rope_pool);
  aclTensor* t_key_rope = arena.CreateTensor("key_rope_cache_view", {blocks, block_size, 1, kRope}, kBf16, rope_pool);
  aclTensorList* key_list = arena.CreateTensorList("fia_key_list", {t_latent_cache});
  aclTensorList* value_list = arena.CreateTensorList("fia_value_list", {t_latent_cache});
  aclTensor* t_block_table = arena.CreateTensor("block_table", {1, blocks}, kInt32, table_dev);
  aclTensor* t_slot = arena.CreateTensor("slot_mapping", {1}, kInt32, slot_dev);
  aclIntArray* seq_q = arena.CreateIntArray("actual_seq_q", {1});
  aclIntArray* seq_kv = arena.CreateIntArray("actual_seq_kv", {context});
  // The getters' results belong to the caller (the arena's list copies above released theirs with delete[]);
  // once more here, directly, for all three.
  {
    int64_t* raw = nullptr;
    uint64_t n = 0;
    if (aclGetViewShape(t_latent_cache, &raw, &n) != 0 || n != 4 || raw[0] != blocks || raw[3] != kLatent) {
      throw Dsv4Error("aclGetViewShape disagrees with the descriptor");
    }
    delete[] raw;
    if (aclGetViewStrides(t_latent_cache, &raw, &n) != 0 || n != 4 || raw[3] != 1 || raw[0] != block_size * kLatent) {
      throw Dsv4Error("aclGetViewStrides disagrees with the descriptor");
    }
    delete[] raw;
    if (aclGetStorageShape(t_latent_cache, &raw, &n) != 0 || n != 4 || raw[1] != block_size) {
      throw Dsv4Error("aclGetStorageShape disagrees with the descriptor");
    }
    delete[] raw;
  }

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
  // One shared workspace at the planned high-water mark, then the latch: from here on the arena refuses
  // every reservation, descriptor and allocation (src/memory/static_arena.cpp:270-304).
  arena.NoteWorkspace(scatter.workspace_size());
  arena.NoteWorkspace(attention.workspace_size());
  arena.CommitWorkspace();
  arena.Seal();
  void* workspace = arena.workspace();
  bool refused = false;
  try {
    arena.CreateTensor("late", {1}, kInt32, slot_dev);
  } catch (const Dsv4Error&) {
    refused = true;
  }
  if (!refused) throw Dsv4Error("a sealed arena built a descriptor");
  const uint64_t allocations_sealed = device.DeviceAllocationCount();

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
    // Zero allocations inside the layer loop, as the reference asserts per step (src/pipeline/pipeline.cpp:502-503).
    if (device.DeviceAllocationCount() != allocations_sealed) throw Dsv4Error("the layer loop allocated device memory");
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
            << ", device allocations " << device.DeviceAllocationCount() << ", arena bytes " << arena.arena_bytes()
            << ", descriptors " << arena.descriptors().size() << "\n";
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
