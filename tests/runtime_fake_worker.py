"""Cases of the device-runtime tests that run on the host-only driver.  Each
case runs in its own process (the driver choice is process-wide), started by
test_runtime_cpu.py:  python runtime_fake_worker.py <case>"""
import ctypes
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import tensorflow_musa_extension_b200 as pkg  # noqa: E402

c = ctypes
vp, u64, i64 = c.c_void_p, c.c_uint64, c.c_int64
CB = c.CFUNCTYPE(None, vp)


class Stream(c.Structure):
    _fields_ = [("magic", u64), ("stream", vp)]


def load():
    pkg.load_plugin()
    lib = pkg.get_library()
    lib.MusaRtLastError.restype = c.c_char_p
    lib.MusaRtDriverName.restype = c.c_char_p
    lib.MusaRtPlatformName.restype = c.c_char_p
    lib.MusaRtDeviceType.restype = c.c_char_p
    lib.MusaRtRawStream.restype = vp
    lib.MusaRtRawStream.argtypes = [vp]
    lib.MusaRtPinnedAllocate.restype = vp
    lib.MusaRtPinnedAllocate.argtypes = [c.c_int, u64]
    lib.MusaRtPinnedFreeAsync.argtypes = [c.c_int, vp, u64, vp]
    lib.MusaRtFakeBlockStream.restype = u64
    lib.MusaRtFakeBlockStream.argtypes = [vp]
    lib.MusaRtFakeReleaseGate.argtypes = [u64]
    lib.MusaRtFakeLiveAllocations.restype = i64
    lib.MusaRtFakeLiveEvents.restype = i64
    lib.MusaRtTimerNanoseconds.restype = u64
    lib.MusaRtTimerNanoseconds.argtypes = [vp]
    lib.MusaRtEventMgrCallbacksRun.restype = u64
    lib.MUSA_TestSeRegistryLiveOrdinalsForTest.restype = c.c_size_t
    lib.MusaRtInitPluginCheck.argtypes = [c.c_size_t, c.c_size_t]
    for name in ("MusaRtAllocate", "MusaRtHostAllocate"):
        getattr(lib, name).argtypes = [c.c_int, u64, c.POINTER(vp)]
    for name in ("MusaRtDeallocate", "MusaRtHostDeallocate"):
        getattr(lib, name).argtypes = [c.c_int, vp]
    lib.MusaRtCreateStream.argtypes = [c.c_int, c.POINTER(vp)]
    lib.MusaRtDestroyStream.argtypes = [c.c_int, vp]
    lib.MusaRtGetStreamStatus.argtypes = [c.c_int, vp]
    lib.MusaRtCreateStreamDependency.argtypes = [c.c_int, vp, vp]
    lib.MusaRtCreateEvent.argtypes = [c.c_int, c.POINTER(vp)]
    lib.MusaRtDestroyEvent.argtypes = [c.c_int, vp]
    lib.MusaRtRecordEvent.argtypes = [c.c_int, vp, vp]
    lib.MusaRtGetEventStatus.argtypes = [c.c_int, vp]
    lib.MusaRtWaitForEvent.argtypes = [c.c_int, vp, vp]
    lib.MusaRtBlockHostForEvent.argtypes = [c.c_int, vp]
    lib.MusaRtCreateTimer.argtypes = [c.c_int, c.POINTER(vp)]
    lib.MusaRtDestroyTimer.argtypes = [c.c_int, vp]
    lib.MusaRtStartTimer.argtypes = [c.c_int, vp, vp]
    lib.MusaRtStopTimer.argtypes = [c.c_int, vp, vp]
    for name in ("MusaRtMemcpyDtoH", "MusaRtMemcpyHtoD", "MusaRtMemcpyDtoD"):
        getattr(lib, name).argtypes = [c.c_int, vp, vp, vp, u64]
    for name in ("MusaRtSyncMemcpyDtoH", "MusaRtSyncMemcpyHtoD", "MusaRtSyncMemcpyDtoD"):
        getattr(lib, name).argtypes = [c.c_int, vp, vp, u64]
    lib.MusaRtMemZero.argtypes = [c.c_int, vp, vp, u64]
    lib.MusaRtMemset.argtypes = [c.c_int, vp, vp, c.c_uint8, u64]
    lib.MusaRtMemset32.argtypes = [c.c_int, vp, vp, c.c_uint32, u64]
    lib.MusaRtHostCallback.argtypes = [c.c_int, vp, CB, vp]
    lib.MusaRtThenExecute.argtypes = [c.c_int, vp, CB, vp]
    lib.MusaRtBlockHostUntilDone.argtypes = [c.c_int, vp]
    lib.MusaRtPinnedStats.argtypes = [c.c_int, c.POINTER(u64 * 7)]
    lib.MusaRtDeviceMemoryUsage.argtypes = [c.c_int, c.POINTER(i64), c.POINTER(i64)]
    return lib


L = load()


def err():
    return L.MusaRtLastError().decode()


def ok(rc):
    assert rc == 0, (rc, err())


def new_stream():
    s = vp()
    ok(L.MusaRtCreateStream(0, c.byref(s)))
    return s


def dev_alloc(n):
    p = vp()
    ok(L.MusaRtAllocate(0, n, c.byref(p)))
    assert p.value
    return p


def stats():
    out = (u64 * 7)()
    ok(L.MusaRtPinnedStats(0, c.byref(out)))
    return dict(zip(["host_allocs", "reuse_hits", "event_allocs", "event_reuse_hits",
                     "free_blocks", "pending_blocks", "bytes_held"], list(out)))


def wait_for(pred, seconds=5.0):
    t0 = time.time()
    while time.time() - t0 < seconds:
        if pred():
            return True
        time.sleep(0.002)
    return pred()


def nparr(a):
    return a.ctypes.data_as(vp)


# ------------------------------------------------------------------ cases --

def case_identity_and_init():
    assert L.MusaRtDriverName() == b"fake"
    assert L.MusaRtPlatformName() == b"MUSA_PLUGGABLE" and L.MusaRtDeviceType() == b"MUSA"
    assert L.MusaRtInitPluginCheck(0, 64) == 0          # struct_size 0 is accepted
    assert L.MusaRtInitPluginCheck(32, 64) == 3 and "too small" in err()
    assert L.MusaRtInitPluginCheck(128, 64) == 0 and err() == ""
    os.environ["TENSORFLOW_MUSA_USE_LEGACY_DEVICE"] = "1"
    assert L.MusaRtInitPluginCheck(128, 64) == 12       # UNIMPLEMENTED in legacy mode
    del os.environ["TENSORFLOW_MUSA_USE_LEGACY_DEVICE"]


def case_device_enumeration():
    n = c.c_int(-5)
    ok(L.MusaRtGetDeviceCount(c.byref(n)))
    assert n.value == 1
    L.MusaRtFakeSetDeviceCount(4)
    ok(L.MUSA_TestPluginGetDeviceCount(c.byref(n)))
    assert n.value == 4
    L.MusaRtFakeSetDeviceCount(-1)                      # the driver call fails
    ok(L.MusaRtGetDeviceCount(c.byref(n)))              # relaxed: 0 devices, OK
    assert n.value == 0
    assert L.MUSA_TestSeRuntimeSmoke() == 0             # relaxed smoke: skipped
    assert L.MUSA_TestSeRuntimeSmokeStrict() == 9
    os.environ["MUSA_STRICT_DEVICE_ENUM"] = "1"
    assert L.MusaRtGetDeviceCount(c.byref(n)) == 9 and "enumeration failed" in err()
    del os.environ["MUSA_STRICT_DEVICE_ENUM"]
    L.MusaRtFakeSetDeviceCount(0)
    assert L.MUSA_TestSeRuntimeSmoke() == 0 and L.MUSA_TestSeRuntimeSmokeStrict() == 9
    L.MusaRtFakeSetDeviceCount(1)
    assert L.MUSA_TestSeRuntimeSmokeStrict() == 0, err()


def case_registry_lifecycle():
    assert L.MUSA_TestSeRegistryLiveOrdinalsForTest() == 0
    assert L.MUSA_TestRegistryDeviceLifecycle() == 0, err()
    assert L.MUSA_TestSeRegistryLiveOrdinalsForTest() == 0
    ok(L.MusaRtCreateDevice(0))
    ok(L.MusaRtCreateDevice(0))
    assert L.MUSA_TestSeRegistryLiveOrdinalsForTest() == 1
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtPinnedAllocate(0, 100)               # still live: helpers exist
    ok(L.MusaRtDestroyDevice(0))
    assert L.MUSA_TestSeRegistryLiveOrdinalsForTest() == 0
    assert not L.MusaRtPinnedAllocate(0, 100)           # dead ordinal: no pool
    assert L.MusaRtFakeLiveAllocations() == 0           # the pool gave its memory back
    assert L.MusaRtCreateDevice(-1) == 3


def case_streams_and_copies():
    ok(L.MusaRtCreateDevice(0))
    s = new_stream()
    wrapper = c.cast(s, c.POINTER(Stream)).contents
    assert wrapper.magic == 0x4D55534153455053 and wrapper.stream
    assert L.MusaRtRawStream(s) == wrapper.stream
    bogus = Stream(0x1234, 0)
    assert L.MusaRtRawStream(c.byref(bogus)) is None
    assert L.MusaRtGetStreamStatus(0, c.byref(bogus)) == 3
    ok(L.MusaRtGetStreamStatus(0, s))
    n = 1 << 16
    a, b = dev_alloc(n * 4), dev_alloc(n * 4)
    src = np.arange(n, dtype=np.uint32) * 7
    back = np.zeros(n, np.uint32)
    ok(L.MusaRtSyncMemcpyHtoD(0, a, nparr(src), n * 4))
    ok(L.MusaRtMemcpyDtoD(0, s, b, a, n * 4))
    ok(L.MusaRtMemcpyDtoH(0, s, nparr(back), b, n * 4))
    ok(L.MusaRtBlockHostUntilDone(0, s))
    assert np.array_equal(src, back)
    ok(L.MusaRtMemset32(0, s, a, 0xDEADBEEF, n * 4))
    ok(L.MusaRtMemset(0, s, b, 0x5A, 100))
    ok(L.MusaRtMemZero(0, s, vp(b.value + 100), 28))
    ok(L.MusaRtBlockHostUntilDone(0, s))
    ok(L.MusaRtSyncMemcpyDtoH(0, nparr(back), a, n * 4))
    assert (back == 0xDEADBEEF).all()
    raw = np.zeros(128, np.uint8)
    ok(L.MusaRtSyncMemcpyDtoH(0, nparr(raw), b, 128))
    assert (raw[:100] == 0x5A).all() and (raw[100:] == 0).all()
    assert L.MusaRtMemset32(0, s, vp(a.value + 2), 1, 8) == 3
    assert L.MusaRtMemcpyDtoH(0, s, None, a, 4) == 3 and "null host pointer" in err()
    assert L.MusaRtMemcpyDtoD(0, None, a, b, 4) == 3 and "null stream" in err()
    ok(L.MusaRtMemcpyDtoD(0, s, None, None, 0))          # empty copies are fine
    free, total = i64(), i64()
    ok(L.MusaRtDeviceMemoryUsage(0, c.byref(free), c.byref(total)))
    assert 0 < free.value < total.value
    ok(L.MusaRtDeallocate(0, a))
    ok(L.MusaRtDeallocate(0, b))
    ok(L.MusaRtDeallocate(0, None))
    ok(L.MusaRtDestroyStream(0, s))
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveAllocations() == 0 and L.MusaRtFakeLiveEvents() == 0


def case_pageable_bounce():
    ok(L.MusaRtCreateDevice(0))
    n = 10000
    a = dev_alloc(n)
    src = (np.arange(n) % 251).astype(np.uint8)          # pageable host memory
    back = np.zeros(n, np.uint8)
    ok(L.MusaRtSyncMemcpyHtoD(0, a, nparr(src), n))
    st = stats()
    assert st["host_allocs"] == 1 and st["reuse_hits"] == 0 and st["free_blocks"] == 1
    assert st["bytes_held"] == 10240                     # rounded up to 256
    ok(L.MusaRtSyncMemcpyHtoD(0, a, nparr(src), n))
    st = stats()
    assert st["host_allocs"] == 1 and st["reuse_hits"] == 1      # staging block reused
    ok(L.MusaRtSyncMemcpyDtoH(0, nparr(back), a, n))
    assert np.array_equal(src, back)
    # a pinned source needs no staging
    pinned = vp()
    ok(L.MusaRtHostAllocate(0, n, c.byref(pinned)))
    c.memmove(pinned, nparr(src), n)
    ok(L.MusaRtSyncMemcpyHtoD(0, a, pinned, n))
    assert stats()["reuse_hits"] == 1
    for var in ("MUSA_SE_DISABLE_PAGEABLE_H2D_BOUNCE", "MUSA_SE_DISABLE_SYNC_H2D_BOUNCE",
                "MUSA_SE_SYNC_H2D"):
        os.environ[var] = "1"
        ok(L.MusaRtSyncMemcpyHtoD(0, a, nparr(src), n))
        assert stats()["reuse_hits"] == 1, var           # pool untouched
        del os.environ[var]
    # the asynchronous form stages a pageable source too: the call returns with
    # the source fully read, the staging block goes back to the pool only after
    # the stream has passed the copy
    s = new_stream()
    gate = L.MusaRtFakeBlockStream(s)
    src2 = src.copy()
    ok(L.MusaRtMemcpyHtoD(0, s, a, nparr(src2), n))
    src2[:] = 0                                          # caller reuses its buffer at once
    st = stats()
    assert st["reuse_hits"] == 2 and st["pending_blocks"] == 1 and st["free_blocks"] == 0
    L.MusaRtFakeReleaseGate(gate)
    ok(L.MusaRtBlockHostUntilDone(0, s))
    wait_for(lambda: stats()["free_blocks"] == 1)
    back[:] = 0
    ok(L.MusaRtSyncMemcpyDtoH(0, nparr(back), a, n))
    assert np.array_equal(src, back)
    os.environ["MUSA_SE_DISABLE_ASYNC_H2D_BOUNCE"] = "1"   # the reference's blocking copy
    ok(L.MusaRtMemcpyHtoD(0, s, a, nparr(src), n))
    assert stats()["reuse_hits"] == 2
    del os.environ["MUSA_SE_DISABLE_ASYNC_H2D_BOUNCE"]
    ok(L.MusaRtHostDeallocate(0, pinned))
    ok(L.MusaRtDeallocate(0, a))
    ok(L.MusaRtDestroyStream(0, s))
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveAllocations() == 0


def case_pinned_pool_reuse_waits_for_the_stream():
    ok(L.MusaRtCreateDevice(0))
    s = new_stream()
    a = L.MusaRtPinnedAllocate(0, 1000)
    gate = L.MusaRtFakeBlockStream(s)                    # the stream stalls here
    ok(L.MusaRtPinnedFreeAsync(0, a, 1000, s))           # "copy still in flight"
    b = L.MusaRtPinnedAllocate(0, 1000)
    assert b and b != a                                  # a must not come back yet
    st = stats()
    assert st["pending_blocks"] == 1 and st["host_allocs"] == 2
    L.MusaRtFakeReleaseGate(gate)
    assert wait_for(lambda: stats()["pending_blocks"] == 0)
    again = L.MusaRtPinnedAllocate(0, 1000)
    assert again == a and stats()["reuse_hits"] == 1
    # best fit: blocks of 1024 (a), 1024 (b) and 8192 free; sizes round up to 256
    big = L.MusaRtPinnedAllocate(0, 8000)
    for p, n in ((again, 1000), (b, 1000), (big, 8000)):
        ok(L.MusaRtPinnedFreeAsync(0, p, n, None))       # null stream: device sync, then free
    assert stats()["free_blocks"] == 3
    assert L.MusaRtPinnedAllocate(0, 1025) == big        # smallest block that fits
    assert L.MusaRtPinnedAllocate(0, 10) in (a, b)       # at least 256 bytes
    # the second FreeAsync reuses the first one's event
    assert stats()["event_allocs"] == 1
    ok(L.MusaRtDestroyStream(0, s))
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveAllocations() == 0 and L.MusaRtFakeLiveEvents() == 0


def case_event_manager():
    ok(L.MusaRtCreateDevice(0))
    slow, fast = new_stream(), new_stream()
    order = []
    cbs = [CB(lambda _, tag=tag: order.append(tag)) for tag in ("slow", "fast")]
    gate = L.MusaRtFakeBlockStream(slow)
    ok(L.MusaRtThenExecute(0, slow, cbs[0], None))
    ok(L.MusaRtThenExecute(0, fast, cbs[1], None))
    assert wait_for(lambda: order == ["fast"])           # not held back by the slow stream
    time.sleep(0.05)
    assert order == ["fast"]
    L.MusaRtFakeReleaseGate(gate)
    assert wait_for(lambda: order == ["fast", "slow"])
    assert L.MusaRtEventMgrCallbacksRun(0) == 2
    # many callbacks from several threads; events are recycled
    count = [0]
    lock = threading.Lock()

    def bump(_):
        with lock:
            count[0] += 1

    cb = CB(bump)

    def worker():
        for _ in range(200):
            ok(L.MusaRtThenExecute(0, fast, cb, None))

    ts = [threading.Thread(target=worker) for _ in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert wait_for(lambda: count[0] == 1600, 20)
    assert L.MusaRtThenExecute(0, None, cb, None) == 3
    ok(L.MusaRtDestroyStream(0, slow))
    ok(L.MusaRtDestroyStream(0, fast))
    ok(L.MusaRtDestroyDevice(0))                         # joins poller and workers
    assert L.MusaRtFakeLiveEvents() == 0
    assert L.MusaRtThenExecute(0, None, cb, None) == 3


def case_stream_dependency():
    ok(L.MusaRtCreateDevice(0))
    producer, consumer = new_stream(), new_stream()
    seen = []
    cb = CB(lambda _: seen.append(time.time()))
    base_events = L.MusaRtFakeLiveEvents()
    gate = L.MusaRtFakeBlockStream(producer)
    ok(L.MusaRtCreateStreamDependency(0, consumer, producer))
    ok(L.MusaRtHostCallback(0, consumer, cb, None))
    time.sleep(0.05)
    assert not seen                                      # consumer waits for producer
    assert L.MusaRtFakeLiveEvents() > base_events        # the temporary event is alive
    L.MusaRtFakeReleaseGate(gate)
    assert wait_for(lambda: len(seen) == 1)
    ok(L.MusaRtBlockHostUntilDone(0, consumer))
    # the event is destroyed only after the consumer passed the wait; the event
    # manager keeps one recycled event of its own
    assert wait_for(lambda: L.MusaRtFakeLiveEvents() == base_events + 1)
    # synchronous mode: destroyed before the call returns
    os.environ["MUSA_SE_SYNC_STREAM_DEPENDENCY"] = "1"
    before = L.MusaRtFakeLiveEvents()
    ok(L.MusaRtCreateStreamDependency(0, consumer, producer))
    assert L.MusaRtFakeLiveEvents() == before
    del os.environ["MUSA_SE_SYNC_STREAM_DEPENDENCY"]
    assert L.MusaRtCreateStreamDependency(0, consumer, None) == 3
    ok(L.MusaRtDestroyStream(0, producer))
    ok(L.MusaRtDestroyStream(0, consumer))
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveEvents() == 0


def case_events_and_timers():
    ok(L.MusaRtCreateDevice(0))
    s, other = new_stream(), new_stream()
    e = vp()
    ok(L.MusaRtCreateEvent(0, c.byref(e)))
    gate = L.MusaRtFakeBlockStream(s)
    ok(L.MusaRtRecordEvent(0, s, e))
    assert L.MusaRtGetEventStatus(0, e) == 1             # pending
    ok(L.MusaRtWaitForEvent(0, other, e))
    hits = []
    cb = CB(lambda _: hits.append(1))
    ok(L.MusaRtHostCallback(0, other, cb, None))
    time.sleep(0.03)
    assert not hits
    L.MusaRtFakeReleaseGate(gate)
    ok(L.MusaRtBlockHostForEvent(0, e))
    assert L.MusaRtGetEventStatus(0, e) == 0             # complete
    assert wait_for(lambda: hits == [1])
    assert L.MusaRtGetEventStatus(0, None) == 2          # error
    t = vp()
    ok(L.MusaRtCreateTimer(0, c.byref(t)))
    ok(L.MusaRtStartTimer(0, s, t))
    nap = CB(lambda _: time.sleep(0.02))
    ok(L.MusaRtHostCallback(0, s, nap, None))
    ok(L.MusaRtStopTimer(0, s, t))
    ns = L.MusaRtTimerNanoseconds(t)
    assert 15e6 < ns < 5e8, ns
    ok(L.MusaRtDestroyTimer(0, t))
    ok(L.MusaRtDestroyEvent(0, e))
    ok(L.MusaRtDestroyStream(0, s))
    ok(L.MusaRtDestroyStream(0, other))
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveEvents() == 0


def case_concurrent_pool_and_copies():
    """Several threads stage pageable copies and free pinned blocks behind
    streams at once; every copy arrives intact and nothing leaks."""
    ok(L.MusaRtCreateDevice(0))
    errors = []

    def worker(seed):
        try:
            rng = np.random.default_rng(seed)
            s = new_stream()
            dev = dev_alloc(1 << 16)
            for _ in range(60):
                n = int(rng.integers(1, 1 << 16))
                src = rng.integers(0, 255, n, dtype=np.uint8)
                back = np.empty(n, np.uint8)
                ok(L.MusaRtSyncMemcpyHtoD(0, dev, nparr(src), n))
                ok(L.MusaRtMemcpyDtoH(0, s, nparr(back), dev, n))
                p = L.MusaRtPinnedAllocate(0, n)
                ok(L.MusaRtPinnedFreeAsync(0, p, n, s))
                ok(L.MusaRtBlockHostUntilDone(0, s))
                assert np.array_equal(src, back)
            ok(L.MusaRtDeallocate(0, dev))
            ok(L.MusaRtDestroyStream(0, s))
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    ts = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=60)
    assert not errors, errors
    st = stats()
    assert st["pending_blocks"] == 0 or wait_for(lambda: stats()["pending_blocks"] == 0)
    assert st["reuse_hits"] > 0
    ok(L.MusaRtDestroyDevice(0))
    assert L.MusaRtFakeLiveAllocations() == 0 and L.MusaRtFakeLiveEvents() == 0


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}

if __name__ == "__main__":
    L.MusaRtUseFakeDriver(1)
    CASES[sys.argv[1]]()
    print("case ok:", sys.argv[1])
