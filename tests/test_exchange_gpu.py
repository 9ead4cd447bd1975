"""The peer-memory exchange protocol on one GPU: the replicas are emulated by
one cooperative launch with a CTA per replica (kernels that wait on one another
must not be separate launches on one GPU), each with its own buffer."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _vectors(world, n, seed):
    rng = np.random.default_rng(seed)
    host = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
    dev = [torch.from_numpy(h).cuda() for h in host]
    table = torch.tensor([d.data_ptr() for d in dev], dtype=torch.int64, device="cuda")
    return host, dev, table


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [1, 129, 4097])
def test_every_replica_gets_the_rank_ordered_sum(kernel_lib, world, n):
    host, dev, table = _vectors(world, n, world * 1000 + n)
    st = torch.cuda.current_stream().cuda_stream
    assert kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), 1, -1, st) == 0
    want = np.zeros(n, np.float32)
    for h in host:                          # rank order, fp32: bit-exact
        want = want + h
    for d in dev:
        assert np.array_equal(d.cpu().numpy(), want)


def test_back_to_back_rounds_reuse_the_two_slots(kernel_lib):
    world, n, rounds = 4, 513, 5
    host, dev, table = _vectors(world, n, 7)
    st = torch.cuda.current_stream().cuda_stream
    assert kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), rounds, -1, st) == 0
    # every round replaces each vector by the sum of all: total * world^(rounds-1)
    total = np.zeros(n, np.float32)
    for h in host:
        total = total + h
    want = total.astype(np.float64) * float(world) ** (rounds - 1)
    for d in dev:
        np.testing.assert_allclose(d.cpu().numpy().astype(np.float64), want, rtol=1e-5)
        assert torch.equal(d, dev[0])       # identical on every replica


def test_a_missing_replica_is_reported_not_waited_for_forever(kernel_lib):
    world, n = 3, 64
    _, dev, table = _vectors(world, n, 9)
    st = torch.cuda.current_stream().cuda_stream
    rc = kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), 1, world - 1, st)
    assert rc == 1000 + world               # 1000 + 1 + q with q = world - 1
    torch.cuda.synchronize()                # the context is still usable
    assert torch.isfinite(dev[0]).all()


def test_single_replica_handle_round_trip(kernel_lib):
    h = kernel_lib.MusaExchangeCreate(0, 1, 1000)
    assert h
    raw = ctypes.create_string_buffer(64)
    assert kernel_lib.MusaExchangeIpcHandle(h, raw) == 0 and any(raw.raw)
    assert kernel_lib.MusaExchangeOpenPeers(h, None) == 0
    v = torch.arange(1000, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        assert kernel_lib.LaunchExchangeSums(h, v.data_ptr(), 1000, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(v, torch.arange(1000, dtype=torch.float32, device="cuda"))
    assert kernel_lib.MusaExchangeStatus(h) == 0
    assert kernel_lib.LaunchExchangeSums(h, v.data_ptr(), 5000, st) == -4
    kernel_lib.MusaExchangeDestroy(h)
    assert kernel_lib.MusaExchangeCreate(3, 2, 10) is None
