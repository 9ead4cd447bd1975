// Pinned host memory for bounce buffers whose reuse must wait for the GPU.
//
// A general allocator hands a freed address out again at once; a bounce buffer
// that an asynchronous copy is still reading must not be.  FreeAsync(ptr, n,
// stream) therefore records an event on `stream` and parks the block; a poll
// thread (100 us) returns it to the free list when the event has completed.
// Allocate() takes the smallest free block that fits (blocks are at least 256
// bytes, sizes rounded up to 256), else allocates new pinned memory.
// FreeAsync with a null stream synchronises the device and frees directly;
// FreeCompleted returns a block that is known to be idle.
//
// Re-target of the reference's GPUPinnedMemoryPool (musa_ext/mu/device/
// pinned_memory_pool.h:46-108; pinned_memory_pool.cc:24-25, 84-161, 179-252,
// 277-322): same rules, own structure.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <list>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "device_driver.h"

namespace musa_rt {

struct PinnedPoolStats {
  uint64_t host_allocs = 0;      // new pinned allocations
  uint64_t reuse_hits = 0;       // allocations served from the free list
  uint64_t event_allocs = 0;
  uint64_t event_reuse_hits = 0;
  uint64_t free_blocks = 0;
  uint64_t pending_blocks = 0;
  uint64_t bytes_held = 0;
};

class PinnedMemoryPool {
 public:
  static constexpr size_t kMinBlock = 256;

  PinnedMemoryPool(DeviceDriver* driver, int ordinal, int poll_us = 100);
  ~PinnedMemoryPool();
  PinnedMemoryPool(const PinnedMemoryPool&) = delete;
  PinnedMemoryPool& operator=(const PinnedMemoryPool&) = delete;

  void* Allocate(size_t bytes);  // nullptr on failure
  void FreeAsync(void* ptr, size_t bytes, StreamHandle stream);
  void FreeCompleted(void* ptr, size_t bytes);
  PinnedPoolStats stats() const;

 private:
  struct Pending {
    void* ptr;
    size_t size;
    EventHandle event;
  };
  static size_t RoundUp(size_t bytes);
  void PollLoop();
  void PollLocked();  // mu_ held

  DeviceDriver* const driver_;
  const int ordinal_;
  const int poll_us_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::multimap<size_t, void*> free_;          // size -> block, best fit = lower_bound
  std::map<void*, size_t> block_size_;         // every block this pool owns
  std::list<Pending> pending_;
  std::vector<EventHandle> free_events_;
  PinnedPoolStats stats_;
  bool stop_ = false;
  std::thread poller_;
};

}  // namespace musa_rt
