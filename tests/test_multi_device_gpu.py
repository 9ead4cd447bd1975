"""One process, two GPUs: the reference's model is a single TensorFlow process
that owns every device (per-ordinal state in
musa_ext/mu/musa_runtime_registry.cc:41-134, the thread-local device cache of
musa_ext/kernels/musa_kernel_runtime.cc:82-129).  Function attributes (the
statistics kernel's 64 KB of dynamic shared memory) and occupancy figures are
per-device state in CUDA; the launchers must set them up on every device they
run on, not only on the first one the process used.  A wrong state shows as a
returned error code (the launch is refused), not as a fault."""
import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import RTOL, adam_inputs, assert_close, bn_inputs, to_numpy, to_torch
from tensorflow_musa_extension_b200 import raw_ops

pytestmark = pytest.mark.gpu

EPS = 1e-3


def _devices():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _rms(a):
    a = np.asarray(a).astype(np.float64)
    return float(np.sqrt(np.mean(a * a))) if a.size else 0.0


@pytest.mark.skipif(_devices() < 2, reason="needs two visible GPUs")
def test_every_op_family_on_the_second_device_of_one_process(kernel_lib):
    # bf16 NHWC with C % 8 == 0: the cp.async-staged statistics kernel (64 KB of
    # dynamic shared memory) and its in-kernel finalize; fp32 rows of 1024:
    # the row-normalisation kernels with their shared-memory ring.
    x, s, o, dy = bn_inputs(41, (6000, 256), "bfloat16", 1.0, 3.0)
    want = np_ref.fused_batch_norm(x, s, o, epsilon=EPS)
    wg = np_ref.fused_batch_norm_grad(dy, x, s, want[3], want[4], EPS)
    # A wide layer: the element-wise kernel adds the partial rows itself and
    # takes more dynamic shared memory than a kernel may without the per-device
    # function attribute.
    wx, ws_, wo, wdy = bn_inputs(44, (8000, 1024), "bfloat16", 1.0, 3.0)
    wide = np_ref.fused_batch_norm(wx, ws_, wo, epsilon=EPS)
    wide_g = np_ref.fused_batch_norm_grad(wdy, wx, ws_, wide[3], wide[4], EPS)
    rows, n = 512, 1024
    rng = np.random.default_rng(42)
    lx = rng.standard_normal((rows, n)).astype(np.float32)
    gam = rng.uniform(0.5, 1.5, n).astype(np.float32)
    bet = rng.normal(0, 0.1, n).astype(np.float32)
    ln_want = np_ref.layer_norm(lx, gam, bet, 1e-5)
    arng, var, m, v = adam_inputs(43, 100003)
    g = arng.normal(0, 1e-3, var.size).astype(np.float32)
    hp = (0.9 ** 10, 0.999 ** 10, 1e-3, 0.9, 0.999, 1e-7)
    ev, em, evv = np_ref.apply_adam(var, m, v, *hp, g)
    xh = rng.standard_normal((512, 1024)).astype(np.float16)
    bh = rng.normal(0, 0.1, 1024).astype(np.float16)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        with torch.cuda.device(dev):
            tx = to_torch(x, dev)
            fwd = raw_ops.FusedBatchNormV3(tx, to_torch(s, dev), to_torch(o, dev),
                                           torch.empty(0, device=dev),
                                           torch.empty(0, device=dev), epsilon=EPS)
            grad = raw_ops.FusedBatchNormGradV3(to_torch(dy, dev), tx, to_torch(s, dev),
                                                fwd.reserve_space_1, fwd.reserve_space_2,
                                                fwd.reserve_space_3, epsilon=EPS)
            torch.cuda.synchronize()
            assert fwd.y.device == torch.device(dev)
            rt = RTOL["lowp"]
            assert_close(to_numpy(fwd.y), want[0], rt, rt * _rms(want[0]), dev + " y")
            assert_close(to_numpy(fwd.reserve_space_1), want[3], 1e-4, 1e-4 * _rms(want[3]),
                         dev + " mean")
            assert_close(to_numpy(fwd.reserve_space_2), want[4], 1e-4, 1e-4 * _rms(want[4]),
                         dev + " var")
            assert_close(to_numpy(grad.x_backprop), wg[0], rt, rt * _rms(wg[0]), dev + " dx")
            assert_close(to_numpy(grad.scale_backprop), wg[1], 1e-4, 1e-4 * _rms(wg[1]),
                         dev + " dscale")
            twx = to_torch(wx, dev)
            wf = raw_ops.FusedBatchNormV3(twx, to_torch(ws_, dev), to_torch(wo, dev),
                                          torch.empty(0, device=dev),
                                          torch.empty(0, device=dev), epsilon=EPS)
            wgr = raw_ops.FusedBatchNormGradV3(to_torch(wdy, dev), twx, to_torch(ws_, dev),
                                               wf.reserve_space_1, wf.reserve_space_2,
                                               wf.reserve_space_3, epsilon=EPS)
            torch.cuda.synchronize()
            assert_close(to_numpy(wf.y), wide[0], rt, rt * _rms(wide[0]), dev + " wide y")
            assert_close(to_numpy(wf.reserve_space_2), wide[4], 1e-4, 1e-4 * _rms(wide[4]),
                         dev + " wide var")
            assert_close(to_numpy(wgr.x_backprop), wide_g[0], rt, rt * _rms(wide_g[0]),
                         dev + " wide dx")
            assert_close(to_numpy(wgr.scale_backprop), wide_g[1], 1e-4, 1e-4 * _rms(wide_g[1]),
                         dev + " wide dscale")
            ly = raw_ops.MusaLayerNorm(to_torch(lx, dev), to_torch(gam, dev),
                                       to_torch(bet, dev), epsilon=1e-5)
            ly = ly[0] if isinstance(ly, (tuple, list)) else ly
            assert_close(to_numpy(ly), ln_want, 1e-4, 1e-5, dev + " layer norm")
            tv, tm, tvv = to_torch(var, dev), to_torch(m, dev), to_torch(v, dev)
            raw_ops.ResourceApplyAdam(tv, tm, tvv, *hp, to_torch(g, dev))
            assert_close(to_numpy(tv), ev, RTOL["f32_adam"], 1e-8, dev + " adam var")
            got = raw_ops.MusaBiasAddRelu(to_torch(xh, dev), to_torch(bh, dev))
            assert np.array_equal(to_numpy(got), np_ref.bias_add_relu(xh, bh))
            db = raw_ops.BiasAddGrad(to_torch(xh, dev))
            assert_close(to_numpy(db), np_ref.bias_add_grad(xh), 2e-2, 1e-2, dev + " bias grad")
