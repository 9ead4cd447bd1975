#include "event_mgr.h"

#include <chrono>

namespace musa_rt {

EventMgr::EventMgr(DeviceDriver* driver, int ordinal, int poll_us, int num_threads)
    : driver_(driver), ordinal_(ordinal), poll_us_(poll_us > 0 ? poll_us : 100) {
  if (num_threads < 1) num_threads = 1;
  for (int i = 0; i < num_threads; ++i) {
    workers_.emplace_back([this] { WorkerLoop(); });
  }
  poller_ = std::thread([this] { PollLoop(); });
}

EventMgr::~EventMgr() {
  shutting_down_.store(true);
  {
    std::lock_guard<std::mutex> l(mu_);
    stop_ = true;
  }
  pending_cv_.notify_all();
  poller_.join();  // drains what is still in use (see PollLoop)
  {
    std::lock_guard<std::mutex> l(work_mu_);
    work_stop_ = true;
  }
  work_cv_.notify_all();
  for (auto& w : workers_) w.join();
  driver_->SetDevice(ordinal_);
  for (EventHandle e : free_events_) driver_->EventDestroy(e);
}

size_t EventMgr::pending() const {
  std::lock_guard<std::mutex> l(mu_);
  return in_use_.size();
}

EventHandle EventMgr::AcquireEvent() {
  {
    std::lock_guard<std::mutex> l(mu_);
    if (!free_events_.empty()) {
      EventHandle e = free_events_.back();
      free_events_.pop_back();
      return e;
    }
  }
  EventHandle e = nullptr;
  if (driver_->EventCreate(&e, /*with_timing=*/false) != 0) return nullptr;
  ++events_created_;
  return e;
}

bool EventMgr::ThenExecute(StreamHandle stream, std::function<void()> fn) {
  return ThenExecuteWithStatus(stream, [f = std::move(fn)](int) { f(); });
}

bool EventMgr::ThenExecuteWithStatus(StreamHandle stream,
                                     std::function<void(int)> fn) {
  if (shutting_down_.load()) return false;
  driver_->SetDevice(ordinal_);
  EventHandle e = AcquireEvent();
  int rc = e != nullptr ? driver_->EventRecord(e, stream) : 1;
  if (rc != 0) {
    // No event: wait for the stream here and run the callback in line, so the
    // caller's resource is still released.
    if (e != nullptr) {
      std::lock_guard<std::mutex> l(mu_);
      free_events_.push_back(e);
    }
    const int sync_rc = driver_->StreamSynchronize(stream);
    fn(sync_rc);
    ++callbacks_run_;
    return false;
  }
  {
    std::lock_guard<std::mutex> l(mu_);
    in_use_.push_back(InUse{e, std::move(fn)});
  }
  pending_cv_.notify_all();
  return true;
}

void EventMgr::PollLoop() {
  driver_->SetDevice(ordinal_);
  std::unique_lock<std::mutex> l(mu_);
  while (true) {
    if (in_use_.empty()) {
      if (stop_) return;
      pending_cv_.wait(l, [this] { return stop_ || !in_use_.empty(); });
      continue;
    }
    // Any completed event, wherever it sits in the list, is retired now.
    std::vector<std::pair<std::function<void(int)>, int>> ready;
    for (auto it = in_use_.begin(); it != in_use_.end();) {
      const int rc = driver_->EventQuery(it->event);
      if (rc == kNotReady) {
        ++it;
        continue;
      }
      ready.emplace_back(std::move(it->fn), rc);
      free_events_.push_back(it->event);
      it = in_use_.erase(it);
    }
    l.unlock();
    if (!ready.empty()) {
      {
        std::lock_guard<std::mutex> wl(work_mu_);
        for (auto& r : ready) {
          work_.push_back([this, fn = std::move(r.first), rc = r.second] {
            fn(rc);
            ++callbacks_run_;
          });
        }
      }
      work_cv_.notify_all();
    } else {
      std::this_thread::sleep_for(std::chrono::microseconds(poll_us_));
    }
    l.lock();
  }
}

void EventMgr::WorkerLoop() {
  std::unique_lock<std::mutex> l(work_mu_);
  while (true) {
    work_cv_.wait(l, [this] { return work_stop_ || !work_.empty(); });
    if (work_.empty()) {
      if (work_stop_) return;
      continue;
    }
    auto fn = std::move(work_.front());
    work_.pop_front();
    l.unlock();
    fn();
    l.lock();
  }
}

}  // namespace musa_rt
