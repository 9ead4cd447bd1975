"""Worker of the world-size-2 CPU tests (gloo): runs the cross-replica host
logic with CPU stand-ins for the four device stages and checks it against the
oracle on the concatenated batch.  Started by test_cross_replica_cpu.py."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import np_ref  # noqa: E402
from tensorflow_musa_extension_b200 import cross_replica as cr  # noqa: E402


class CpuStages:
    """Torch-CPU stand-ins with the contracts of the C launchers."""

    def workspace_bytes(self, rows, c):
        return 16

    def stats_moments(self, x, moments, ws):
        c = x.shape[1]
        xf = x.double()
        mean = xf.mean(0) if x.shape[0] else torch.zeros(c, dtype=torch.float64)
        moments[:c] = mean.float()
        moments[c:2 * c] = ((xf - mean) ** 2).sum(0).float()
        moments[2 * c] = float(x.shape[0])

    def merge_moments(self, gathered, world, c, merged):
        g = gathered.double().reshape(world, 2 * c + 1)
        n = g[:, 2 * c]
        total = n.sum()
        mean = (n[:, None] * g[:, :c]).sum(0) / total
        m2 = (g[:, c:2 * c] + n[:, None] * (g[:, :c] - mean) ** 2).sum(0)
        merged[:c] = mean.float()
        merged[c:2 * c] = m2.float()
        merged[2 * c] = float(total)

    def apply_from_moments(self, x, scale, offset, moments, count, stats, y, eps):
        self._finalize_moments(moments, count, stats, x.shape[1])
        self.apply(x, scale, offset, stats[2], stats[3], y, eps)

    def _finalize_moments(self, moments, count, stats, c):
        mean = moments[:c].double()
        var = (moments[c:2 * c].double() / count).clamp_min(0)
        stats[0].copy_(mean.float())
        stats[1].copy_((var * (count / (count - 1.0)) if count > 1 else var).float())
        stats[2].copy_(mean.float())
        stats[3].copy_(var.float())

    def apply(self, x, scale, offset, mean, var, y, eps):
        y.copy_(((x.float() - mean) * (scale / torch.sqrt(var + eps)) + offset).to(x.dtype))

    def grad_stats_sums(self, dy, x, mean, sums, ws):
        c = x.shape[1]
        sums[:c] = dy.double().sum(0).float()
        sums[c:] = (dy.double() * (x.double() - mean.double())).sum(0).float()

    def grad_apply(self, dy, x, scale, mean, var, sums, count, dx, dscale, doffset, eps):
        c = x.shape[1]
        inv = 1.0 / torch.sqrt(var + eps)
        doffset.copy_(sums[:c])
        dscale.copy_(sums[c:] * inv)
        dx.copy_((scale * inv * (dy.float() - sums[:c] / count
                                 - (x.float() - mean) * inv * inv * sums[c:] / count)).to(x.dtype))


def cpu_adam(var, m, v, grad, b1p, b2p, lr, b1, b2, eps):
    nv, nm, nvv = np_ref.apply_adam(var.numpy(), m.numpy(), v.numpy(), b1p, b2p, lr, b1, b2,
                                    eps, grad.numpy())
    var.copy_(torch.from_numpy(nv))
    m.copy_(torch.from_numpy(nm))
    v.copy_(torch.from_numpy(nvv))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mode = sys.argv[1]
    rng = np.random.default_rng(123)
    if mode in ("syncbn", "syncbn_ragged", "syncbn_large_mean"):
        c = 24
        rows = [40, 13] if mode == "syncbn_ragged" else [40, 40]
        total = sum(rows)
        # |mean| / std = 1000: raw [sum x, sum x^2] exchanged in fp32 would
        # lose the variance here; the merged moments keep it.
        loc, std = (1e3, 1.0) if mode == "syncbn_large_mean" else (0.5, 2.0)
        x = (rng.standard_normal((total, c)) * std + loc).astype(np.float32)
        dy = rng.standard_normal((total, c)).astype(np.float32)
        s = rng.uniform(0.5, 1.5, c).astype(np.float32)
        o = rng.normal(0, 0.1, c).astype(np.float32)
        lo = sum(rows[:rank])
        hi = lo + rows[rank]
        bn = cr.SyncBatchNorm(c, 1e-3, torch.float32, "cpu", rows[rank], dist.group.WORLD,
                              kernels=CpuStages())
        if mode == "syncbn_ragged":
            bn.set_ragged()
        xl, dyl = torch.from_numpy(x[lo:hi].copy()), torch.from_numpy(dy[lo:hi].copy())
        y, dx = torch.empty_like(xl), torch.empty_like(xl)
        bn.forward(xl, torch.from_numpy(s), torch.from_numpy(o), y)
        bn.backward(dyl, xl, torch.from_numpy(s), dx)
        want = np_ref.fused_batch_norm(x, s, o, epsilon=1e-3)
        wg = np_ref.fused_batch_norm_grad(dy, x, s, want[3], want[4], 1e-3)
        assert bn.global_count == total, (bn.global_count, total)
        # The op's mean output is fp32: at |mean| = 1000 its half-ulp (3e-5) is
        # the floor of x - mean, whoever computes it.
        y_atol = 2e-4 if mode == "syncbn_large_mean" else 1e-5
        np.testing.assert_allclose(y.numpy(), want[0][lo:hi], rtol=1e-4, atol=y_atol)
        np.testing.assert_allclose(bn.batch_mean.numpy(), want[1], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(bn.batch_var.numpy(), want[2], rtol=1e-4)
        np.testing.assert_allclose(bn.saved_var.numpy(), want[4], rtol=1e-4)
        np.testing.assert_allclose(dx.numpy(), wg[0][lo:hi], rtol=1e-3,
                                   atol=2e-4 if mode == "syncbn_large_mean" else 1e-5)
        np.testing.assert_allclose(bn.dscale.numpy(), wg[1], rtol=1e-4,
                                   atol=5e-3 if mode == "syncbn_large_mean" else 1e-4)
        np.testing.assert_allclose(bn.doffset.numpy(), wg[2], rtol=1e-4, atol=1e-4)
    elif mode in ("adam_even", "adam_padded"):
        n = 1000 if mode == "adam_even" else 1001
        var0 = rng.normal(0, 0.05, n).astype(np.float32)
        var = torch.from_numpy(var0.copy())
        opt = cr.ShardedAdam(var, dist.group.WORLD, update_fn=cpu_adam)
        assert (opt.lo, opt.hi) == cr.shard_range(n, world, rank)
        ev, em, evv = var0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for step in range(1, 4):
            g = rng.normal(0, 1e-3, n).astype(np.float32)
            ev, em, evv = np_ref.apply_adam(ev, em, evv, 0.9 ** step, 0.999 ** step, 1e-3,
                                            0.9, 0.999, 1e-7, g)
            # even steps hand over the full gradient, odd steps the local range
            gt = torch.from_numpy(g)
            opt.step(gt if step % 2 == 0 else gt[opt.lo:opt.hi], 1e-3, 0.9 ** step,
                     0.999 ** step)
            np.testing.assert_allclose(var.numpy(), ev, rtol=1e-6, atol=1e-9)
        np.testing.assert_allclose(opt.m.numpy(), em[opt.lo:opt.hi], rtol=1e-6, atol=1e-12)
    else:
        raise SystemExit("unknown mode " + mode)
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
