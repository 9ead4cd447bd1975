#include "pinned_pool.h"

#include <chrono>

namespace musa_rt {

PinnedMemoryPool::PinnedMemoryPool(DeviceDriver* driver, int ordinal, int poll_us)
    : driver_(driver), ordinal_(ordinal), poll_us_(poll_us > 0 ? poll_us : 100) {
  poller_ = std::thread([this] { PollLoop(); });
}

PinnedMemoryPool::~PinnedMemoryPool() {
  {
    std::lock_guard<std::mutex> l(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  poller_.join();
  driver_->SetDevice(ordinal_);
  // Whatever is still pending is waited for, then everything goes back.
  for (auto& p : pending_) {
    driver_->EventSynchronize(p.event);
    driver_->EventDestroy(p.event);
  }
  for (EventHandle e : free_events_) driver_->EventDestroy(e);
  for (auto& kv : block_size_) driver_->HostFree(kv.first);
}

size_t PinnedMemoryPool::RoundUp(size_t bytes) {
  if (bytes < kMinBlock) bytes = kMinBlock;
  return (bytes + kMinBlock - 1) / kMinBlock * kMinBlock;
}

void* PinnedMemoryPool::Allocate(size_t bytes) {
  const size_t want = RoundUp(bytes);
  {
    std::lock_guard<std::mutex> l(mu_);
    PollLocked();  // pick up blocks whose copies have just finished
    auto it = free_.lower_bound(want);
    if (it != free_.end()) {
      void* p = it->second;
      free_.erase(it);
      ++stats_.reuse_hits;
      return p;
    }
  }
  driver_->SetDevice(ordinal_);
  void* p = nullptr;
  if (driver_->HostAlloc(&p, want) != 0 || p == nullptr) return nullptr;
  std::lock_guard<std::mutex> l(mu_);
  block_size_[p] = want;
  ++stats_.host_allocs;
  return p;
}

void PinnedMemoryPool::FreeCompleted(void* ptr, size_t) {
  if (ptr == nullptr) return;
  std::lock_guard<std::mutex> l(mu_);
  const auto it = block_size_.find(ptr);
  if (it == block_size_.end()) return;  // not ours
  free_.emplace(it->second, ptr);
}

void PinnedMemoryPool::FreeAsync(void* ptr, size_t bytes, StreamHandle stream) {
  if (ptr == nullptr) return;
  driver_->SetDevice(ordinal_);
  if (stream == nullptr) {
    // No stream to follow: wait for the device, then the block is idle.
    driver_->DeviceSynchronize();
    FreeCompleted(ptr, bytes);
    return;
  }
  EventHandle e = nullptr;
  {
    std::lock_guard<std::mutex> l(mu_);
    if (!free_events_.empty()) {
      e = free_events_.back();
      free_events_.pop_back();
      ++stats_.event_reuse_hits;
    }
  }
  if (e == nullptr) {
    if (driver_->EventCreate(&e, false) != 0) e = nullptr;
    if (e != nullptr) {
      std::lock_guard<std::mutex> l(mu_);
      ++stats_.event_allocs;
    }
  }
  if (e == nullptr || driver_->EventRecord(e, stream) != 0) {
    if (e != nullptr) {
      std::lock_guard<std::mutex> l(mu_);
      free_events_.push_back(e);
    }
    driver_->StreamSynchronize(stream);
    FreeCompleted(ptr, bytes);
    return;
  }
  {
    std::lock_guard<std::mutex> l(mu_);
    if (block_size_.count(ptr) == 0) {  // not ours: do not track it
      free_events_.push_back(e);
      return;
    }
    pending_.push_back(Pending{ptr, block_size_[ptr], e});
  }
  cv_.notify_all();
}

void PinnedMemoryPool::PollLocked() {
  for (auto it = pending_.begin(); it != pending_.end();) {
    if (driver_->EventQuery(it->event) == kNotReady) {
      ++it;
      continue;
    }
    free_.emplace(it->size, it->ptr);
    free_events_.push_back(it->event);
    it = pending_.erase(it);
  }
}

void PinnedMemoryPool::PollLoop() {
  driver_->SetDevice(ordinal_);
  std::unique_lock<std::mutex> l(mu_);
  while (!stop_) {
    if (pending_.empty()) {
      cv_.wait(l, [this] { return stop_ || !pending_.empty(); });
      continue;
    }
    PollLocked();
    cv_.wait_for(l, std::chrono::microseconds(poll_us_));
  }
}

PinnedPoolStats PinnedMemoryPool::stats() const {
  std::lock_guard<std::mutex> l(mu_);
  PinnedPoolStats s = stats_;
  s.free_blocks = free_.size();
  s.pending_blocks = pending_.size();
  s.bytes_held = 0;
  for (const auto& kv : block_size_) s.bytes_held += kv.second;
  return s;
}

}  // namespace musa_rt
