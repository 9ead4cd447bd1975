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

    def stats_sums(self, x, sums, ws):
        c = x.shape[1]
        xf = x.double()
        sums[:c] = xf.sum(0).float()
        sums[c:2 * c] = (xf * xf).sum(0).float()
        sums[2 * c] = float(x.shape[0])

    def apply_from_sums(self, x, scale, offset, sums, count, stats, y, eps):
        self.finalize(sums, count, stats, x.shape[1])
        self.apply(x, scale, offset, stats[2], stats[3], y, eps)

    def finalize(self, sums, count, stats, c):
        mean = sums[:c].double() / count
        var = (sums[c:2 * c].double() / count - mean * mean).clamp_min(0)
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
    if mode in ("syncbn", "syncbn_ragged"):
        c = 24
        rows = [40, 40] if mode == "syncbn" else [40, 13]
        total = sum(rows)
        x = (rng.standard_normal((total, c)) * 2 + 0.5).astype(np.float32)
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
        np.testing.assert_allclose(y.numpy(), want[0][lo:hi], rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(bn.batch_mean.numpy(), want[1], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(bn.batch_var.numpy(), want[2], rtol=1e-4)
        np.testing.assert_allclose(bn.saved_var.numpy(), want[4], rtol=1e-4)
        np.testing.assert_allclose(dx.numpy(), wg[0][lo:hi], rtol=1e-3, atol=1e-5)
        np.testing.assert_allclose(bn.dscale.numpy(), wg[1], rtol=1e-4, atol=1e-4)
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
