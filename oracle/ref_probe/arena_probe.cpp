// Drives the reference's own StaticMemoryArena (compiled from the reference tree where it lies) over
// a reservation script, and prints what it did. Used to pin this repository's KV arena to the
// reference's behaviour: offsets, alignment, single allocation, phase refusals, workspace high-water.
//
// TEST INFRASTRUCTURE: built only when the reference tree is present; the product never links it.
//
// stdin:  lines "reserve <name> <bytes> <align>", "commit", "note <bytes>", "commit_workspace",
//         "fits <bytes>", "seal", "address <index>"
// stdout: one line per command: "ok <value...>" or "refused".
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <iostream>
#include <sstream>
#include <string>

#include "moe/memory/static_arena.hpp"

namespace {

class HostAllocator final : public ascend_moe::IDeviceAllocator {
 public:
  void* DeviceMalloc(size_t bytes) override {
    ++allocations_;
    return std::aligned_alloc(4096, (bytes + 4095) / 4096 * 4096);
  }
  void DeviceFree(void* pointer) override { std::free(pointer); }
  void* HostPinnedMalloc(size_t bytes) override { return std::aligned_alloc(4096, (bytes + 4095) / 4096 * 4096); }
  void HostPinnedFree(void* pointer) override { std::free(pointer); }
  void DeviceMemset(void* pointer, size_t, int value, size_t count) override { std::memset(pointer, value, count); }
  uint64_t DeviceAllocationCount() const override { return allocations_; }
  bool QueryDeviceMemory(size_t*, size_t*) override { return false; }
  const char* backend_name() const override { return "probe-host"; }

 private:
  uint64_t allocations_ = 0;
};

}  // namespace

int main() {
  HostAllocator allocator;
  ascend_moe::StaticMemoryArena arena(allocator);
  std::deque<std::string> names;  // Reserve keeps the name by pointer
  std::string line;
  while (std::getline(std::cin, line)) {
    std::istringstream in(line);
    std::string cmd;
    in >> cmd;
    if (cmd.empty()) continue;
    try {
      if (cmd == "reserve") {
        std::string name;
        size_t bytes = 0, align = 0;
        in >> name >> bytes >> align;
        names.push_back(name);
        const auto handle = arena.Reserve(names.back().c_str(), bytes, align);
        std::printf("ok %zu %zu %zu\n", static_cast<size_t>(handle), arena.reservations()[handle].offset,
                    arena.reserved_bytes());
      } else if (cmd == "commit") {
        arena.Commit();
        const unsigned char* base = static_cast<const unsigned char*>(arena.arena_base());
        bool zero = true;
        for (size_t i = 0; i < arena.arena_bytes(); ++i) zero = zero && base[i] == 0;
        std::printf("ok %zu %llu %d\n", arena.arena_bytes(),
                    static_cast<unsigned long long>(allocator.DeviceAllocationCount()), zero ? 1 : 0);
      } else if (cmd == "address") {
        size_t index = 0;
        in >> index;
        const auto* p = static_cast<const unsigned char*>(arena.Address(index));
        std::printf("ok %zu\n", static_cast<size_t>(p - static_cast<const unsigned char*>(arena.arena_base())));
      } else if (cmd == "note") {
        unsigned long long bytes = 0;
        in >> bytes;
        arena.NoteWorkspace(bytes);
        std::printf("ok\n");
      } else if (cmd == "commit_workspace") {
        arena.CommitWorkspace();
        std::printf("ok %llu %llu\n", static_cast<unsigned long long>(arena.workspace_bytes()),
                    static_cast<unsigned long long>(allocator.DeviceAllocationCount()));
      } else if (cmd == "fits") {
        unsigned long long bytes = 0;
        in >> bytes;
        arena.AssertWorkspaceFits(bytes, "probe");
        std::printf("ok\n");
      } else if (cmd == "seal") {
        arena.Seal();
        std::printf("ok %d\n", arena.sealed() ? 1 : 0);
      } else if (cmd == "validate") {
        arena.ValidateAlignment();
        std::printf("ok\n");
      } else {
        std::printf("unknown\n");
      }
    } catch (const std::exception&) {
      std::printf("refused\n");
    }
  }
  return 0;
}
