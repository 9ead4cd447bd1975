// Runs host callbacks once the work queued on a stream has completed, without
// blocking that stream or the caller.
//
// ThenExecute(stream, fn) records an event on `stream`; a dedicated thread
// polls the outstanding events (every `poll_us` microseconds while any are
// pending) and hands the callbacks of completed ones to a small worker pool.
// Completion is out of order: a slow stream does not hold back the callbacks
// of faster ones.  Events are recycled.  After shutdown begins no new callback
// is accepted; the ones already queued still run (their streams are drained).
//
// Re-target of the reference's MusaEventMgr (musa_ext/mu/device/
// musa_event_mgr.h:46-117, musa_event_mgr.cc:106-316): same contract (brief,
// non-blocking callbacks; default 100 us poll, 8 workers), own structure.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <list>
#include <mutex>
#include <thread>
#include <vector>

#include "device_driver.h"

namespace musa_rt {

class EventMgr {
 public:
  EventMgr(DeviceDriver* driver, int ordinal, int poll_us = 100, int num_threads = 8);
  ~EventMgr();
  EventMgr(const EventMgr&) = delete;
  EventMgr& operator=(const EventMgr&) = delete;

  // Returns false (and does not keep `fn`) if the manager is shutting down or
  // the event could not be recorded; in the latter case `fn` runs after a
  // stream synchronise instead, so it is never lost.
  bool ThenExecute(StreamHandle stream, std::function<void()> fn);
  // fn(error_code): 0 when the stream work completed.
  bool ThenExecuteWithStatus(StreamHandle stream, std::function<void(int)> fn);

  uint64_t callbacks_run() const { return callbacks_run_.load(); }
  uint64_t events_created() const { return events_created_.load(); }
  size_t pending() const;

 private:
  struct InUse {
    EventHandle event;
    std::function<void(int)> fn;
  };
  void PollLoop();
  void WorkerLoop();
  EventHandle AcquireEvent();

  DeviceDriver* const driver_;
  const int ordinal_;
  const int poll_us_;
  mutable std::mutex mu_;
  std::condition_variable pending_cv_;
  std::list<InUse> in_use_;
  std::vector<EventHandle> free_events_;
  bool stop_ = false;
  std::thread poller_;

  std::mutex work_mu_;
  std::condition_variable work_cv_;
  std::deque<std::function<void()>> work_;
  bool work_stop_ = false;
  std::vector<std::thread> workers_;

  std::atomic<bool> shutting_down_{false};
  std::atomic<uint64_t> callbacks_run_{0};
  std::atomic<uint64_t> events_created_{0};
};

}  // namespace musa_rt
