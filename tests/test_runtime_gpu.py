"""The device runtime on the CUDA driver: the reference's runtime smoke hooks
(test/ops/pluggable_se_api_test.py:188-343) plus the paths that need a real
device - pinned staging, stream dependencies between real streams, timers."""
import ctypes as c
import threading
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

vp, u64, i64 = c.c_void_p, c.c_uint64, c.c_int64
CB = c.CFUNCTYPE(None, vp)


@pytest.fixture(scope="module")
def rt(kernel_lib):
    L = kernel_lib
    L.MusaRtLastError.restype = c.c_char_p
    L.MusaRtDriverName.restype = c.c_char_p
    L.MusaRtRawStream.restype = vp
    L.MusaRtRawStream.argtypes = [vp]
    L.MusaRtTimerNanoseconds.restype = u64
    L.MusaRtTimerNanoseconds.argtypes = [vp]
    L.MusaRtAllocate.argtypes = [c.c_int, u64, c.POINTER(vp)]
    L.MusaRtDeallocate.argtypes = [c.c_int, vp]
    L.MusaRtCreateStream.argtypes = [c.c_int, c.POINTER(vp)]
    L.MusaRtDestroyStream.argtypes = [c.c_int, vp]
    L.MusaRtCreateStreamDependency.argtypes = [c.c_int, vp, vp]
    L.MusaRtCreateTimer.argtypes = [c.c_int, c.POINTER(vp)]
    L.MusaRtDestroyTimer.argtypes = [c.c_int, vp]
    L.MusaRtStartTimer.argtypes = [c.c_int, vp, vp]
    L.MusaRtStopTimer.argtypes = [c.c_int, vp, vp]
    L.MusaRtMemcpyDtoH.argtypes = [c.c_int, vp, vp, vp, u64]
    L.MusaRtMemcpyDtoD.argtypes = [c.c_int, vp, vp, vp, u64]
    L.MusaRtSyncMemcpyHtoD.argtypes = [c.c_int, vp, vp, u64]
    L.MusaRtSyncMemcpyDtoH.argtypes = [c.c_int, vp, vp, u64]
    L.MusaRtMemset32.argtypes = [c.c_int, vp, vp, c.c_uint32, u64]
    L.MusaRtThenExecute.argtypes = [c.c_int, vp, CB, vp]
    L.MusaRtBlockHostUntilDone.argtypes = [c.c_int, vp]
    L.MusaRtPinnedStats.argtypes = [c.c_int, c.POINTER(u64 * 7)]
    L.MUSA_TestDeviceMetadata.argtypes = [c.c_int, c.c_char_p, c.c_size_t,
                                          c.POINTER(c.c_int), c.POINTER(i64)]
    assert L.MusaRtDriverName() == b"cuda"
    return L


def ok(L, rc):
    assert rc == 0, (rc, L.MusaRtLastError())


def test_smoke_hooks_and_metadata(rt):
    n = c.c_int()
    ok(rt, rt.MUSA_TestPluginGetDeviceCount(c.byref(n)))
    assert n.value == torch.cuda.device_count() >= 1
    ok(rt, rt.MUSA_TestSeRuntimeSmoke())
    ok(rt, rt.MUSA_TestSeRuntimeSmokeStrict())
    ok(rt, rt.MUSA_TestRegistryDeviceLifecycle())
    name = c.create_string_buffer(128)
    sms, mem = c.c_int(), i64()
    ok(rt, rt.MUSA_TestDeviceMetadata(0, name, 128, c.byref(sms), c.byref(mem)))
    assert name.value.decode() == torch.cuda.get_device_name(0)
    assert sms.value == torch.cuda.get_device_properties(0).multi_processor_count
    assert mem.value == torch.cuda.get_device_properties(0).total_memory


def test_streams_feed_the_kernel_launchers(rt):
    """A stream made by the runtime is the stream a launcher runs on."""
    ok(rt, rt.MusaRtCreateDevice(0))
    s = vp()
    ok(rt, rt.MusaRtCreateStream(0, c.byref(s)))
    raw = rt.MusaRtRawStream(s)
    assert raw
    n = 1 << 20
    x = torch.randn(n, device="cuda")
    y = torch.empty_like(x)
    torch.cuda.synchronize()
    assert rt.LaunchBiasAct_F32(x.data_ptr(), None, y.data_ptr(), n, 1, 1, 1, raw) == 0
    ok(rt, rt.MusaRtBlockHostUntilDone(0, s))
    assert torch.equal(y, torch.relu(x))
    ok(rt, rt.MusaRtDestroyStream(0, s))
    ok(rt, rt.MusaRtDestroyDevice(0))


def test_pageable_staging_dependency_timer_and_callbacks(rt):
    ok(rt, rt.MusaRtCreateDevice(0))
    producer, consumer = vp(), vp()
    ok(rt, rt.MusaRtCreateStream(0, c.byref(producer)))
    ok(rt, rt.MusaRtCreateStream(0, c.byref(consumer)))
    n = 8 << 20
    a, b = vp(), vp()
    ok(rt, rt.MusaRtAllocate(0, n, c.byref(a)))
    ok(rt, rt.MusaRtAllocate(0, n, c.byref(b)))
    src = np.random.default_rng(0).integers(0, 255, n, dtype=np.uint8)   # pageable
    st0, st = (u64 * 7)(), (u64 * 7)()
    ok(rt, rt.MusaRtPinnedStats(0, c.byref(st0)))      # the pool may have served earlier tests
    ok(rt, rt.MusaRtSyncMemcpyHtoD(0, a, src.ctypes.data_as(vp), n))
    ok(rt, rt.MusaRtPinnedStats(0, c.byref(st)))
    # at most one new staging block, and it is back on the free list
    assert st[0] - st0[0] <= 1 and st[0] + st[1] == st0[0] + st0[1] + 1 and st[4] >= 1
    # the asynchronous form stages a pageable source in chunks and has read all
    # of it by the time it returns
    big = np.random.default_rng(1).integers(0, 255, 3 * n + 12345, dtype=np.uint8)
    keep = big.copy()
    wide = vp()
    ok(rt, rt.MusaRtAllocate(0, big.size, c.byref(wide)))
    rt.MusaRtMemcpyHtoD.argtypes = [c.c_int, vp, vp, vp, u64]
    ok(rt, rt.MusaRtMemcpyHtoD(0, producer, wide, big.ctypes.data_as(vp), big.size))
    big[:] = 0
    ok(rt, rt.MusaRtBlockHostUntilDone(0, producer))
    got = np.empty_like(big)
    ok(rt, rt.MusaRtSyncMemcpyDtoH(0, got.ctypes.data_as(vp), wide, big.size))
    assert np.array_equal(got, keep)
    ok(rt, rt.MusaRtDeallocate(0, wide))
    # producer fills b from a; consumer copies b out only after that
    timer = vp()
    ok(rt, rt.MusaRtCreateTimer(0, c.byref(timer)))
    ok(rt, rt.MusaRtStartTimer(0, producer, timer))
    for _ in range(20):
        ok(rt, rt.MusaRtMemcpyDtoD(0, producer, b, a, n))
    ok(rt, rt.MusaRtStopTimer(0, producer, timer))
    ok(rt, rt.MusaRtCreateStreamDependency(0, consumer, producer))
    back = torch.empty(n, dtype=torch.uint8).pin_memory()
    ok(rt, rt.MusaRtMemcpyDtoH(0, consumer, back.data_ptr(), b, n))
    done = threading.Event()
    cb = CB(lambda _: done.set())
    ok(rt, rt.MusaRtThenExecute(0, consumer, cb, None))
    assert done.wait(10)                        # runs once the consumer has drained
    assert np.array_equal(back.numpy(), src)
    ns = rt.MusaRtTimerNanoseconds(timer)
    assert 1e3 < ns < 1e9
    ok(rt, rt.MusaRtDestroyTimer(0, timer))
    ok(rt, rt.MusaRtMemset32(0, producer, a, 0x01020304, n))
    ok(rt, rt.MusaRtBlockHostUntilDone(0, producer))
    out = np.empty(n // 4, np.uint32)
    ok(rt, rt.MusaRtSyncMemcpyDtoH(0, out.ctypes.data_as(vp), a, n))
    assert (out == 0x01020304).all()
    for p in (a, b):
        ok(rt, rt.MusaRtDeallocate(0, p))
    for s in (producer, consumer):
        ok(rt, rt.MusaRtDestroyStream(0, s))
    ok(rt, rt.MusaRtDestroyDevice(0))
