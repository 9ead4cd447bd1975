// Host-only DeviceDriver: streams are FIFO work queues with a worker thread
// each, events complete when their stream reaches them, "device" and pinned
// memory are tracked heap blocks.  Used by the CPU tests of the runtime.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "device_driver.h"

namespace musa_rt {
namespace {

constexpr int kErrInvalid = 1;  // cudaErrorInvalidValue
constexpr int kErrNoDevice = 100;

struct FakeEvent {
  std::mutex mu;
  std::condition_variable cv;
  uint64_t recorded = 0;   // generation of the latest EventRecord
  uint64_t completed = 0;  // generation that has completed
  std::chrono::steady_clock::time_point when;
};

struct FakeStream {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void()>> queue;
  bool busy = false;
  bool stop = false;
  std::thread worker;

  FakeStream() {
    worker = std::thread([this] { Run(); });
  }
  ~FakeStream() {
    {
      std::lock_guard<std::mutex> l(mu);
      stop = true;
    }
    cv.notify_all();
    worker.join();
  }
  void Run() {
    std::unique_lock<std::mutex> l(mu);
    while (true) {
      cv.wait(l, [this] { return stop || !queue.empty(); });
      if (queue.empty()) {
        if (stop) return;
        continue;
      }
      auto fn = std::move(queue.front());
      queue.pop_front();
      busy = true;
      l.unlock();
      fn();
      l.lock();
      busy = false;
      cv.notify_all();
    }
  }
  void Push(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> l(mu);
      queue.push_back(std::move(fn));
    }
    cv.notify_all();
  }
  void Drain() {
    std::unique_lock<std::mutex> l(mu);
    cv.wait(l, [this] { return queue.empty() && !busy; });
  }
  bool Idle() {
    std::lock_guard<std::mutex> l(mu);
    return queue.empty() && !busy;
  }
};

struct Gate {
  std::mutex mu;
  std::condition_variable cv;
  bool open = false;
};

class FakeDriverImpl : public DeviceDriver {
 public:
  const char* Name() const override { return "fake"; }

  int DeviceCount(int* count) override {
    *count = device_count_.load();
    return *count < 0 ? kErrNoDevice : 0;
  }
  int SetDevice(int ordinal) override {
    const int n = device_count_.load();
    return (ordinal >= 0 && ordinal < (n < 0 ? 0 : n)) ? 0 : kErrInvalid;
  }

  int Malloc(void** ptr, size_t bytes) override { return Alloc(ptr, bytes, PointerKind::kDevice); }
  int HostAlloc(void** ptr, size_t bytes) override {
    return Alloc(ptr, bytes, PointerKind::kPinnedHost);
  }
  int Free(void* ptr) override { return Release(ptr, PointerKind::kDevice); }
  int HostFree(void* ptr) override { return Release(ptr, PointerKind::kPinnedHost); }
  int MemGetInfo(size_t* f, size_t* t) override {
    *t = size_t(1) << 34;
    std::lock_guard<std::mutex> l(mu_);
    size_t used = 0;
    for (const auto& kv : blocks_) used += kv.second.first;
    *f = *t - used;
    return 0;
  }

  int StreamCreate(StreamHandle* s) override {
    auto* st = new FakeStream();
    std::lock_guard<std::mutex> l(mu_);
    streams_[st] = std::unique_ptr<FakeStream>(st);
    *s = st;
    return 0;
  }
  int StreamDestroy(StreamHandle s) override {
    std::unique_ptr<FakeStream> owned;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = streams_.find(s);
      if (it == streams_.end()) return kErrInvalid;
      owned = std::move(it->second);
      streams_.erase(it);
    }
    owned->Drain();
    return 0;
  }
  int StreamSynchronize(StreamHandle s) override {
    FakeStream* st = Stream(s);
    if (st == nullptr) return kErrInvalid;
    st->Drain();
    return 0;
  }
  int StreamQuery(StreamHandle s) override {
    FakeStream* st = Stream(s);
    if (st == nullptr) return kErrInvalid;
    return st->Idle() ? 0 : kNotReady;
  }

  int EventCreate(EventHandle* e, bool) override {
    *e = new FakeEvent();
    ++live_events_;
    return 0;
  }
  int EventDestroy(EventHandle e) override {
    if (e == nullptr) return kErrInvalid;
    delete static_cast<FakeEvent*>(e);
    --live_events_;
    return 0;
  }
  int EventRecord(EventHandle e, StreamHandle s) override {
    FakeStream* st = Stream(s);
    auto* ev = static_cast<FakeEvent*>(e);
    if (st == nullptr || ev == nullptr) return kErrInvalid;
    uint64_t gen;
    {
      std::lock_guard<std::mutex> l(ev->mu);
      gen = ++ev->recorded;
    }
    st->Push([ev, gen] {
      std::lock_guard<std::mutex> l(ev->mu);
      if (gen > ev->completed) ev->completed = gen;
      ev->when = std::chrono::steady_clock::now();
      ev->cv.notify_all();
    });
    return 0;
  }
  int EventQuery(EventHandle e) override {
    auto* ev = static_cast<FakeEvent*>(e);
    if (ev == nullptr) return kErrInvalid;
    std::lock_guard<std::mutex> l(ev->mu);
    return ev->completed >= ev->recorded ? 0 : kNotReady;
  }
  int EventSynchronize(EventHandle e) override {
    auto* ev = static_cast<FakeEvent*>(e);
    if (ev == nullptr) return kErrInvalid;
    std::unique_lock<std::mutex> l(ev->mu);
    const uint64_t want = ev->recorded;
    ev->cv.wait(l, [&] { return ev->completed >= want; });
    return 0;
  }
  int EventElapsedMs(EventHandle a, EventHandle b, float* ms) override {
    auto* ea = static_cast<FakeEvent*>(a);
    auto* eb = static_cast<FakeEvent*>(b);
    if (ea == nullptr || eb == nullptr) return kErrInvalid;
    if (EventQuery(a) != 0 || EventQuery(b) != 0) return kNotReady;
    *ms = std::chrono::duration<float, std::milli>(eb->when - ea->when).count();
    return 0;
  }
  int StreamWaitEvent(StreamHandle s, EventHandle e) override {
    FakeStream* st = Stream(s);
    auto* ev = static_cast<FakeEvent*>(e);
    if (st == nullptr || ev == nullptr) return kErrInvalid;
    uint64_t want;
    {
      std::lock_guard<std::mutex> l(ev->mu);
      want = ev->recorded;  // the wait captures the record that exists now
    }
    st->Push([ev, want] {
      std::unique_lock<std::mutex> l(ev->mu);
      ev->cv.wait(l, [&] { return ev->completed >= want; });
    });
    return 0;
  }

  int MemcpyAsync(void* dst, const void* src, size_t n, CopyKind, StreamHandle s) override {
    FakeStream* st = Stream(s);
    if (st == nullptr || (n > 0 && (dst == nullptr || src == nullptr))) return kErrInvalid;
    st->Push([dst, src, n] { std::memcpy(dst, src, n); });
    return 0;
  }
  int Memcpy(void* dst, const void* src, size_t n, CopyKind k) override {
    const int rc = MemcpyAsync(dst, src, n, k, nullptr);
    return rc != 0 ? rc : StreamSynchronize(nullptr);
  }
  int MemsetAsync(void* dst, int byte, size_t n, StreamHandle s) override {
    FakeStream* st = Stream(s);
    if (st == nullptr || (n > 0 && dst == nullptr)) return kErrInvalid;
    st->Push([dst, byte, n] { std::memset(dst, byte, n); });
    return 0;
  }
  int Memset32Async(void* dst, uint32_t pattern, size_t count, StreamHandle s) override {
    FakeStream* st = Stream(s);
    if (st == nullptr || (count > 0 && dst == nullptr)) return kErrInvalid;
    st->Push([dst, pattern, count] {
      auto* p = static_cast<uint32_t*>(dst);
      for (size_t i = 0; i < count; ++i) p[i] = pattern;
    });
    return 0;
  }
  int LaunchHostFunc(StreamHandle s, void (*fn)(void*), void* arg) override {
    FakeStream* st = Stream(s);
    if (st == nullptr || fn == nullptr) return kErrInvalid;
    st->Push([fn, arg] { fn(arg); });
    return 0;
  }
  int DeviceSynchronize() override {
    std::vector<FakeStream*> all;
    {
      std::lock_guard<std::mutex> l(mu_);
      for (auto& kv : streams_) all.push_back(kv.second.get());
    }
    for (FakeStream* st : all) st->Drain();
    DefaultStream()->Drain();
    return 0;
  }
  PointerKind Classify(const void* ptr) override {
    std::lock_guard<std::mutex> l(mu_);
    auto it = blocks_.upper_bound(reinterpret_cast<uintptr_t>(ptr));
    if (it == blocks_.begin()) return PointerKind::kPageableHost;
    --it;
    const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
    if (p < it->first + (it->second.first ? it->second.first : 1)) return it->second.second;
    return PointerKind::kPageableHost;
  }
  std::string ErrorString(int code) override {
    switch (code) {
      case 0: return "no error";
      case kErrInvalid: return "invalid argument";
      case kErrNoDevice: return "no device is detected";
      case kNotReady: return "device not ready";
      default: return "fake driver error " + std::to_string(code);
    }
  }

  // ---- test controls
  void SetDeviceCount(int n) { device_count_.store(n); }
  uint64_t BlockStream(StreamHandle s) {
    FakeStream* st = Stream(s);
    if (st == nullptr) return 0;
    auto gate = std::make_shared<Gate>();
    uint64_t id;
    {
      std::lock_guard<std::mutex> l(mu_);
      id = ++next_gate_;
      gates_[id] = gate;
    }
    st->Push([gate] {
      std::unique_lock<std::mutex> l(gate->mu);
      gate->cv.wait(l, [&] { return gate->open; });
    });
    return id;
  }
  void ReleaseGate(uint64_t id) {
    std::shared_ptr<Gate> gate;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = gates_.find(id);
      if (it == gates_.end()) return;
      gate = it->second;
      gates_.erase(it);
    }
    {
      std::lock_guard<std::mutex> l(gate->mu);
      gate->open = true;
    }
    gate->cv.notify_all();
  }
  int64_t LiveAllocations() {
    std::lock_guard<std::mutex> l(mu_);
    return static_cast<int64_t>(blocks_.size());
  }
  int64_t LiveEvents() { return live_events_.load(); }

 private:
  int Alloc(void** ptr, size_t bytes, PointerKind kind) {
    void* p = std::malloc(bytes > 0 ? bytes : 1);
    if (p == nullptr) return 2;  // cudaErrorMemoryAllocation
    std::lock_guard<std::mutex> l(mu_);
    blocks_[reinterpret_cast<uintptr_t>(p)] = {bytes, kind};
    *ptr = p;
    return 0;
  }
  int Release(void* ptr, PointerKind kind) {
    if (ptr == nullptr) return 0;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = blocks_.find(reinterpret_cast<uintptr_t>(ptr));
      if (it == blocks_.end() || it->second.second != kind) return kErrInvalid;
      blocks_.erase(it);
    }
    std::free(ptr);
    return 0;
  }
  FakeStream* DefaultStream() {
    static FakeStream* s = new FakeStream();
    return s;
  }
  FakeStream* Stream(StreamHandle s) {
    if (s == nullptr) return DefaultStream();
    std::lock_guard<std::mutex> l(mu_);
    auto it = streams_.find(s);
    return it == streams_.end() ? nullptr : it->second.get();
  }

  std::mutex mu_;
  std::atomic<int> device_count_{1};
  std::atomic<int64_t> live_events_{0};
  std::map<uintptr_t, std::pair<size_t, PointerKind>> blocks_;
  std::unordered_map<void*, std::unique_ptr<FakeStream>> streams_;
  std::unordered_map<uint64_t, std::shared_ptr<Gate>> gates_;
  uint64_t next_gate_ = 0;
};

FakeDriverImpl* Impl() {
  static FakeDriverImpl* impl = new FakeDriverImpl();
  return impl;
}

}  // namespace

DeviceDriver* FakeDriver() { return Impl(); }
void FakeDriverSetDeviceCount(int count) { Impl()->SetDeviceCount(count); }
uint64_t FakeDriverBlockStream(StreamHandle stream) { return Impl()->BlockStream(stream); }
void FakeDriverReleaseGate(uint64_t gate) { Impl()->ReleaseGate(gate); }
int64_t FakeDriverLiveAllocations() { return Impl()->LiveAllocations(); }
int64_t FakeDriverLiveEvents() { return Impl()->LiveEvents(); }

}  // namespace musa_rt
