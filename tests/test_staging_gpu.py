"""The upload / compute / download pipeline: results equal the direct op calls,
whatever the depth, the order of collection, the kind of host memory or the
number of submitting threads."""
import ctypes as c
import random
import threading

import numpy as np
import pytest
import torch

from helpers import NP_BF16, to_numpy, to_torch
from tensorflow_musa_extension_b200 import errors, raw_ops
from tensorflow_musa_extension_b200.staging import StagedPipeline, StagedValue

pytestmark = pytest.mark.gpu

EPS = 1e-3
E = torch.empty(0)


def _bn_inputs(seed, rows, ch, dtype=torch.bfloat16, pinned=True):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, ch, generator=g) * 2 + 0.5).to(dtype)
    dy = (torch.randn(rows, ch, generator=g) * 1e-2).to(dtype)
    s = torch.rand(ch, generator=g) + 0.5
    o = torch.randn(ch, generator=g) * 0.1
    if pinned:
        x, dy, s, o = (t.pin_memory() for t in (x, dy, s, o))
    return x, dy, s, o


def _direct(x, dy, s, o):
    fwd = raw_ops.FusedBatchNormV3(x.cuda(), s.cuda(), o.cuda(), E.cuda(), E.cuda(), epsilon=EPS)
    bwd = raw_ops.FusedBatchNormGradV3(dy.cuda(), x.cuda(), s.cuda(), fwd[3], fwd[4], None,
                                       epsilon=EPS)
    torch.cuda.synchronize()
    return [t.cpu() for t in fwd], [t.cpu() for t in bwd]


def _same(a, b):
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(
        a.contiguous().reshape(-1).view(torch.uint8), b.contiguous().reshape(-1).view(torch.uint8))


def test_forward_and_gradient_through_handles(kernel_lib):
    x, dy, s, o = _bn_inputs(1, 4099, 96)
    want_f, want_b = _direct(x, dy, s, o)
    with StagedPipeline(depth=3) as pipe:
        f = pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, E, E, epsilon=EPS)
        assert isinstance(f.input(0), StagedValue) and f.input(0).shape == (4099, 96)
        b = pipe.submit(raw_ops.FusedBatchNormGradV3, dy, f.input(0), s, f.output(3),
                        f.output(4), None, epsilon=EPS)
        got_b = b.result()            # collected before the forward call's results
        got_f = f.result()
        for g, w in zip(got_f, want_f):
            assert _same(g, w)
        for g, w in zip(got_b, want_b):
            assert _same(g, w)
        assert pipe.stats["h2d_bytes"] >= 2 * x.numel() * 2
        f.release()
        with pytest.raises(errors.InvalidArgumentError, match="released"):
            f.result()


@pytest.mark.parametrize("depth", [1, 2, 5])
def test_many_calls_any_collection_order(kernel_lib, depth):
    shapes = [(257, 8), (1024, 64), (33, 1000), (5000, 24), (64, 2048), (1, 16)]
    cases = [_bn_inputs(i, *shapes[i % len(shapes)], dtype=(torch.float32, torch.float16,
                                                            torch.bfloat16)[i % 3])
             for i in range(18)]
    wants = [_direct(*cs)[0] for cs in cases]
    with StagedPipeline(depth=depth) as pipe:
        calls = [pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, E, E, epsilon=EPS, fetch=(0, 1, 2))
                 for (x, dy, s, o) in cases]
        order = list(range(len(calls)))
        random.Random(depth).shuffle(order)
        for i in order:
            got = calls[i].result()
            assert got[3] is None and got[4] is None       # not fetched
            for g, w in zip(got[:3], wants[i][:3]):
                assert _same(g, w), (i, depth)
            calls[i].release()
        assert pipe.stats["calls"] == len(cases)


def test_pageable_numpy_and_device_arguments(kernel_lib):
    x, dy, s, o = _bn_inputs(7, 3001, 40, dtype=torch.float16, pinned=False)
    assert not x.is_pinned()
    want = _direct(x, dy, s, o)[0]
    with StagedPipeline() as pipe:
        a = pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, E, E, epsilon=EPS)
        x_before = x.clone()
        x.zero_()                      # a pageable source is free again after submit
        b = pipe.submit(raw_ops.FusedBatchNormV3, x_before.numpy(), s.numpy(), o.numpy(),
                        E.numpy(), E.numpy(), epsilon=EPS)
        d = pipe.submit(raw_ops.FusedBatchNormV3, x_before.cuda(), s.cuda(), o, E, E, epsilon=EPS)
        for call in (a, b, d):
            for g, w in zip(call.result(), want):
                assert _same(g, w)
    # bfloat16 arrays (ml_dtypes) go up as they are
    xb = np.random.default_rng(0).standard_normal((100, 8)).astype(NP_BF16)
    with StagedPipeline() as pipe:
        r = pipe.submit(raw_ops.Relu, xb).result()[0]
    assert np.array_equal(to_numpy(r).view(np.uint16), np.maximum(xb, 0).view(np.uint16))


def test_in_place_ops_and_ordering_on_the_compute_stream(kernel_lib):
    """An op without outputs (variable update) followed by a reader of the
    variable: the compute stream keeps their order."""
    var = torch.ones(10000, device="cuda")
    delta = torch.full((10000,), 2.0).pin_memory()
    with StagedPipeline(depth=2) as pipe:
        for _ in range(5):
            u = pipe.submit(raw_ops.ResourceApplyGradientDescent, var, 0.25, delta)
            assert u.result() == ()
        r = pipe.submit(raw_ops.Relu, var)
        assert torch.equal(r.result()[0], torch.full((10000,), 1.0 - 5 * 0.5).clamp(min=0))
        pipe.synchronize()
    assert torch.equal(var.cpu(), torch.full((10000,), -1.5))


def test_threads_submit_concurrently(kernel_lib):
    cases = [_bn_inputs(20 + i, 900 + 37 * i, 32) for i in range(4)]
    wants = [_direct(*cs)[0] for cs in cases]
    failures = []
    with StagedPipeline(depth=3) as pipe:
        def worker(i):
            try:
                x, dy, s, o = cases[i]
                for _ in range(8):
                    got = pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, E, E,
                                      epsilon=EPS).result()
                    if not all(_same(g, w) for g, w in zip(got, wants[i])):
                        failures.append(i)
            except Exception as e:  # pragma: no cover
                failures.append((i, repr(e)))
        threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    assert failures == []


def test_a_failing_op_leaves_the_pipeline_usable(kernel_lib):
    x, dy, s, o = _bn_inputs(3, 500, 16)
    with StagedPipeline() as pipe:
        with pytest.raises(errors.InvalidArgumentError):
            pipe.submit(raw_ops.FusedBatchNormV3, x, s[:5].contiguous(), o, E, E, epsilon=EPS)
        got = pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, E, E, epsilon=EPS).result()
        for g, w in zip(got, _direct(x, dy, s, o)[0]):
            assert _same(g, w)
    with pytest.raises(errors.InvalidArgumentError, match="closed"):
        pipe.submit(raw_ops.Relu, x)


def test_released_blocks_are_reused(kernel_lib):
    lib = raw_ops._lib()
    lib.MusaRtPinnedStats.argtypes = [c.c_int, c.POINTER(c.c_uint64 * 7)]
    x = torch.randn(1 << 20).pin_memory()

    def stats():
        out = (c.c_uint64 * 7)()
        assert lib.MusaRtPinnedStats(torch.cuda.current_device(), c.byref(out)) == 0
        return dict(zip(["host_allocs", "reuse_hits", "event_allocs", "event_reuse_hits",
                         "free_blocks", "pending_blocks", "bytes_held"], list(out)))

    with StagedPipeline() as pipe:
        pipe.submit(raw_ops.Relu, x).release()
        pipe.synchronize()
        before = stats()
        for _ in range(6):
            call = pipe.submit(raw_ops.Relu, x)
            assert torch.equal(call.result()[0], torch.relu(x))
            call.release()
            torch.cuda.synchronize()
        after = stats()
    assert after["host_allocs"] <= before["host_allocs"] + 1
    assert after["reuse_hits"] >= before["reuse_hits"] + 4
