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
    assert kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), 1, -1, 0, st) == 0
    want = np.zeros(n, np.float32)
    for h in host:                          # rank order, fp32: bit-exact
        want = want + h
    for d in dev:
        assert np.array_equal(d.cpu().numpy(), want)


def test_back_to_back_rounds_reuse_the_two_slots(kernel_lib):
    world, n, rounds = 4, 513, 5
    host, dev, table = _vectors(world, n, 7)
    st = torch.cuda.current_stream().cuda_stream
    assert kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), rounds, -1, 0, st) == 0
    # every round replaces each vector by the sum of all: total * world^(rounds-1)
    total = np.zeros(n, np.float32)
    for h in host:
        total = total + h
    want = total.astype(np.float64) * float(world) ** (rounds - 1)
    for d in dev:
        np.testing.assert_allclose(d.cpu().numpy().astype(np.float64), want, rtol=1e-5)
        assert torch.equal(d, dev[0])       # identical on every replica


@pytest.mark.parametrize("n", [64, 4097])
def test_a_missing_replica_is_reported_not_waited_for_forever(kernel_lib, n):
    """One wait (about a second) runs out, the kernel reports the replica and
    stops waiting for it: the other cells of that replica cost nothing more."""
    import time
    world = 3
    _, dev, table = _vectors(world, n, 9)
    st = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), 1, world - 1, 0, st)
    torch.cuda.synchronize()                # the context is still usable
    elapsed = time.perf_counter() - t0
    assert rc == 1000 + world               # 1000 + 1 + q with q = world - 1
    assert elapsed < 4.0, elapsed
    assert torch.isfinite(dev[0]).all()


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("channels", [1, 64, 2048])
def test_moments_mode_merges_in_rank_order(kernel_lib, world, channels):
    """Every replica ends with the moments of the union of all replicas' rows:
    count-weighted mean, M2 by Chan's formula (fp64 reference)."""
    rng = np.random.default_rng(world * 100 + channels)
    n = 2 * channels + 1
    host = []
    for q in range(world):
        rows = float(rng.integers(1, 5000))
        v = np.concatenate([rng.normal(1e3, 1.0, channels), rng.uniform(0, 1e4, channels),
                            [rows]]).astype(np.float32)
        host.append(v)
    dev = [torch.from_numpy(h).cuda() for h in host]
    table = torch.tensor([d.data_ptr() for d in dev], dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert kernel_lib.MusaExchangeSelfTest(world, n, table.data_ptr(), 1, -1, 1, st) == 0
    g = np.stack(host).astype(np.float64)
    cnt = g[:, 2 * channels]
    total = cnt.sum()
    mean = (cnt[:, None] * g[:, :channels]).sum(0) / total
    m2 = (g[:, channels:2 * channels] + cnt[:, None] * (g[:, :channels] - mean) ** 2).sum(0)
    for d in dev:
        got = d.cpu().numpy().astype(np.float64)
        assert got[2 * channels] == total
        np.testing.assert_allclose(got[:channels], mean, rtol=1e-6)
        np.testing.assert_allclose(got[channels:2 * channels], m2, rtol=1e-5, atol=1e-3)
        assert torch.equal(d, dev[0])       # bit-identical on every replica


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,c", [(4096, 64), (777, 520), (5000, 2048)])
def test_finalize_kernel_runs_the_exchange_itself(kernel_lib, dtype, rows, c):
    """LaunchBnStatsMomentsExchange / LaunchBnGradStatsSumsExchange with a
    one-replica handle return what the two-step forms return, call after call
    (epoch and ticket advance inside the finalize kernel), and leave the
    handle usable by the stand-alone exchange kernel."""
    h = kernel_lib.MusaExchangeCreate(0, 1, 2 * c + 1)
    assert h and kernel_lib.MusaExchangeOpenPeers(h, None) == 0
    st = torch.cuda.current_stream().cuda_stream
    dt = {torch.float32: 0, torch.bfloat16: 2}[dtype]
    need = kernel_lib.BnWorkspaceBytes(rows, c, 1)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(rows + c)
    for _ in range(3):
        x = (torch.randn(rows, c, device="cuda", generator=gen) * 2 + 5).to(dtype)
        dy = torch.randn(rows, c, device="cuda", generator=gen).to(dtype)
        want = torch.empty(2 * c + 1, device="cuda")
        got = torch.empty(2 * c + 1, device="cuda")
        assert kernel_lib.LaunchBnStatsMoments(dt, x.data_ptr(), want.data_ptr(), rows, c, 1,
                                               ws.data_ptr(), ws.numel(), st) == 0
        assert kernel_lib.LaunchBnStatsMomentsExchange(
            dt, x.data_ptr(), got.data_ptr(), rows, c, 1, ws.data_ptr(), ws.numel(), h, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        mean = want[:c].clone()
        gw, gg = torch.empty(2 * c, device="cuda"), torch.empty(2 * c, device="cuda")
        assert kernel_lib.LaunchBnGradStatsSums(dt, dy.data_ptr(), x.data_ptr(), mean.data_ptr(),
                                                gw.data_ptr(), rows, c, 1, ws.data_ptr(),
                                                ws.numel(), st) == 0
        assert kernel_lib.LaunchBnGradStatsSumsExchange(
            dt, dy.data_ptr(), x.data_ptr(), mean.data_ptr(), gg.data_ptr(), rows, c, 1,
            ws.data_ptr(), ws.numel(), h, st) == 0
        v = torch.arange(7, dtype=torch.float32, device="cuda")
        assert kernel_lib.LaunchExchangeSums(h, v.data_ptr(), 7, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(gg, gw)
        assert torch.equal(v, torch.arange(7, dtype=torch.float32, device="cuda"))
    assert kernel_lib.MusaExchangeStatus(h) == 0
    small = kernel_lib.MusaExchangeCreate(0, 1, 8)
    assert kernel_lib.LaunchBnStatsMomentsExchange(
        dt, x.data_ptr(), got.data_ptr(), rows, c, 1, ws.data_ptr(), ws.numel(), small, st) == -4
    kernel_lib.MusaExchangeDestroy(small)
    kernel_lib.MusaExchangeDestroy(h)
