"""MusaLayerNorm, MusaLayerNormGrad, MusaRmsNorm and MusaRmsNormGradDx on the
GPU (through the C ABI) against the CPU oracle and the PyTorch-CPU golden
vectors."""
import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import NP_BF16, RTOL, assert_close, np_dtype, to_numpy, to_torch
from tensorflow_musa_extension_b200 import errors, raw_ops

pytestmark = pytest.mark.gpu

SHAPES = ["s16x32", "s8x16x32", "s32x128", "s2x4x8x16", "s100x1", "s100x2", "s1x1", "s2x8192",
          "s7x1000"]
# Row lengths that exercise every register layout (groups of 8, 32, 64, 128,
# 256, 512 threads with two, three or four packs per thread), the element-wise
# form (odd lengths, very long rows) and the ragged last group.
ROW_SIZES = [1, 2, 3, 8, 31, 32, 64, 100, 128, 192, 256, 384, 768, 1000, 1024, 1536, 2048, 3072,
             4096, 5000, 6144, 8192, 12288, 16384, 20000]


def _tol(dtype):
    return (RTOL["f32_elementwise"], 2e-6) if dtype == "float32" else (RTOL["lowp"], 2e-2)


def test_golden_vectors(golden, kernel_lib):
    g = golden["row_norm_torch_cpu"]
    for name in SHAPES:
        k = "layer_norm/" + name
        x, dy, gamma, beta = (g[k + "/" + n] for n in ("x", "dy", "gamma", "beta"))
        tx, td, tg, tb = (to_torch(a) for a in (x, dy, gamma, beta))
        assert_close(to_numpy(raw_ops.MusaLayerNorm(tx, tg, tb)), g[k + "/y"], 1e-5, 2e-6, k)
        dx, dgamma, dbeta = raw_ops.MusaLayerNormGrad(td, tx, tg, tb)
        rows = x.size // x.shape[-1]
        # Rows of one or two elements are ill-conditioned (var ~ eps): fp32
        # statistics move dx by more than the usual tolerance.
        dx_rt = 1e-4 if x.shape[-1] > 2 else 1e-2
        assert_close(to_numpy(dx), g[k + "/dx"], dx_rt, 2e-5, k + " dx")
        assert_close(to_numpy(dgamma), g[k + "/dgamma"], 1e-4, 2e-6 * rows, k + " dgamma")
        assert_close(to_numpy(dbeta), g[k + "/dbeta"], 1e-4, 2e-6 * rows, k + " dbeta")
        r = "rms_norm/" + name
        y, normalized, inv = raw_ops.MusaRmsNorm(tx, tg)
        assert tuple(inv.shape) == x.shape[:-1] + (1,)
        assert_close(to_numpy(y), g[r + "/y"], 1e-5, 1e-6, r)
        assert_close(to_numpy(normalized), g[r + "/normalized"], 1e-5, 1e-6, r)
        assert_close(to_numpy(inv), g[r + "/inv_rms"], 1e-5, 0, r)
        assert_close(to_numpy(raw_ops.MusaRmsNormGradDx(tx, inv, tg, td)), g[r + "/dx"],
                     1e-4, 2e-5, r + " dx")


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("n", ROW_SIZES)
def test_layer_norm_row_sizes(kernel_lib, dtype, n):
    rng = np.random.default_rng(n)
    dt = np_dtype(dtype)
    rows = 37 if n < 4096 else 5
    x = rng.uniform(-10, 10, (rows, n)).astype(dt)
    dy = rng.uniform(-1, 1, (rows, n)).astype(dt)
    gamma = rng.uniform(0.5, 1.5, n).astype(dt)
    beta = rng.uniform(-0.5, 0.5, n).astype(dt)
    rt, at = _tol(dtype)
    tx, td, tg, tb = (to_torch(a) for a in (x, dy, gamma, beta))
    y = raw_ops.MusaLayerNorm(tx, tg, tb)
    assert y.dtype == tx.dtype and y.shape == tx.shape
    assert_close(to_numpy(y), np_ref.layer_norm(x, gamma, beta), rt, at, "y")
    dx, dgamma, dbeta = raw_ops.MusaLayerNormGrad(td, tx, tg, tb)
    want = np_ref.layer_norm_grad(dy, x, gamma)
    # x_hat is O(1) and |dy| <= 1: absolute tolerances in units of the output.
    # Rows of one or two elements have var ~ 0, inv_std ~ 316: rounding of the
    # row means is amplified by that factor.
    dx_at = at * 2 + (1e-5 if n > 2 else 1e-3)
    assert_close(to_numpy(dx), want[0], rt * 10, dx_at, "dx")
    assert_close(to_numpy(dgamma), want[1], rt * 10, (at + 1e-5) * np.sqrt(rows), "dgamma")
    assert_close(to_numpy(dbeta), want[2], rt * 10, (at + 1e-5) * np.sqrt(rows), "dbeta")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", ROW_SIZES)
def test_rms_norm_row_sizes(kernel_lib, dtype, n):
    rng = np.random.default_rng(1000 + n)
    dt = np_dtype(dtype)
    rows = 37 if n < 4096 else 5
    x = rng.uniform(-3, 3, (rows, n)).astype(dt)
    dy = rng.uniform(-1, 1, (rows, n)).astype(dt)
    gamma = rng.uniform(0.5, 1.5, n).astype(dt)
    rt, at = _tol(dtype)
    tx, td, tg = (to_torch(a) for a in (x, dy, gamma))
    y, normalized, inv = raw_ops.MusaRmsNorm(tx, tg, epsilon=1e-5)
    wy, wn, wi = np_ref.rms_norm(x, gamma, 1e-5)
    assert_close(to_numpy(y), wy, rt, at, "y")
    assert_close(to_numpy(normalized), wn, rt, at, "normalized")
    assert_close(to_numpy(inv), wi, rt, 0, "inv_rms")
    # The gradient reads inv_rms as the forward stored it (rounded to T).
    got = raw_ops.MusaRmsNormGradDx(tx, inv, tg, td)
    want = np_ref.rms_norm_grad_dx(x, to_numpy(inv), gamma, dy)
    assert_close(to_numpy(got), want, rt * 5, at * 5 + 1e-5, "dx")


def test_many_rows_and_reproducibility(kernel_lib):
    """More row blocks than CTAs (the grid strides), and fixed-order column
    sums: two runs give the same bits."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((70001, 96)).astype(np.float32)
    dy = rng.standard_normal((70001, 96)).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, 96).astype(np.float32)
    beta = np.zeros(96, np.float32)
    tx, td, tg, tb = (to_torch(a) for a in (x, dy, gamma, beta))
    a = raw_ops.MusaLayerNormGrad(td, tx, tg, tb)
    b = raw_ops.MusaLayerNormGrad(td, tx, tg, tb)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    want = np_ref.layer_norm_grad(dy, x, gamma)
    assert_close(to_numpy(a.dx), want[0], 1e-4, 1e-5, "dx")
    assert_close(to_numpy(a.dgamma), want[1], 1e-4, 5e-3, "dgamma")
    assert_close(to_numpy(a.dbeta), want[2], 1e-4, 5e-3, "dbeta")
    assert_close(to_numpy(raw_ops.MusaLayerNorm(tx, tg, tb)), np_ref.layer_norm(x, gamma, beta),
                 1e-5, 2e-6, "y")


def test_large_mean_does_not_cancel(kernel_lib):
    """|mean| >> std: the variance is taken around the mean."""
    rng = np.random.default_rng(6)
    x = (rng.standard_normal((64, 1024)) * 0.01 + 1000.0).astype(np.float32)
    gamma = np.ones(1024, np.float32)
    beta = np.zeros(1024, np.float32)
    got = to_numpy(raw_ops.MusaLayerNorm(to_torch(x), to_torch(gamma), to_torch(beta)))
    assert_close(got, np_ref.layer_norm(x, gamma, beta), 1e-3, 1e-3, "y")
    assert abs(got.std(axis=-1).mean() - 1.0) < 0.05


def test_unaligned_views_take_the_element_form(kernel_lib):
    lib = raw_ops._lib()
    rng = np.random.default_rng(7)
    x = rng.standard_normal((33, 64)).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, 64).astype(np.float32)
    beta = rng.uniform(-0.5, 0.5, 64).astype(np.float32)
    buf = torch.empty(33 * 64 + 1, device="cuda")
    buf[1:].copy_(to_torch(x).reshape(-1))
    y = torch.empty(33, 64, device="cuda")
    tg, tb = to_torch(gamma), to_torch(beta)
    mean = torch.empty(33, device="cuda")
    inv = torch.empty(33, device="cuda")
    rc = lib.LaunchLayerNorm_F32(buf[1:].data_ptr(), tg.data_ptr(), tb.data_ptr(), y.data_ptr(),
                                 mean.data_ptr(), inv.data_ptr(), 33, 64, 1e-5,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert_close(to_numpy(y), np_ref.layer_norm(x, gamma, beta), 1e-5, 2e-6)
    assert_close(to_numpy(mean), x.astype(np.float64).mean(-1), 1e-5, 1e-6)
    assert_close(to_numpy(inv), 1 / np.sqrt(x.astype(np.float64).var(-1) + 1e-5), 1e-5, 0)


def test_edge_cases_and_errors(kernel_lib):
    g = torch.ones(8, device="cuda")
    b = torch.zeros(8, device="cuda")
    empty = torch.empty(0, 8, device="cuda")
    assert tuple(raw_ops.MusaLayerNorm(empty, g, b).shape) == (0, 8)
    dx, dgamma, dbeta = raw_ops.MusaLayerNormGrad(empty, empty, g, b)
    assert tuple(dx.shape) == (0, 8) and not dgamma.any() and not dbeta.any()
    y, normalized, inv = raw_ops.MusaRmsNorm(empty, g)
    assert tuple(inv.shape) == (0, 1)
    x = torch.randn(4, 8, device="cuda")
    with pytest.raises(errors.InvalidArgumentError, match="Gamma size mismatch: expected 8, got 7"):
        raw_ops.MusaLayerNorm(x, torch.ones(7, device="cuda"), b)
    with pytest.raises(errors.InvalidArgumentError, match="Beta size mismatch"):
        raw_ops.MusaLayerNorm(x, g, torch.ones(9, device="cuda"))
    with pytest.raises(errors.InvalidArgumentError, match="dy and x must have the same shape"):
        raw_ops.MusaLayerNormGrad(torch.randn(4, 7, device="cuda"), x, g, b)
    with pytest.raises(errors.InvalidArgumentError, match="float/bfloat16"):
        raw_ops.MusaRmsNorm(x.half(), g.half())
    with pytest.raises(errors.InvalidArgumentError, match="inv size mismatch"):
        raw_ops.MusaRmsNormGradDx(x, torch.ones(3, 1, device="cuda"), g, x)
    with pytest.raises(errors.InvalidArgumentError, match="shape mismatch"):
        raw_ops.MusaRmsNormGradDx(x, torch.ones(4, 1, device="cuda"), g, x[:2])
    # host tensors go through the same ops
    xh = np.random.default_rng(0).standard_normal((5, 8)).astype(np.float32)
    got = raw_ops.MusaLayerNorm(xh, np.ones(8, np.float32), np.zeros(8, np.float32))
    assert isinstance(got, np.ndarray)
    assert_close(got, np_ref.layer_norm(xh, np.ones(8), np.zeros(8)), 1e-5, 2e-6)


def test_full_size_properties(kernel_lib):
    """[65536, 1024] bf16 (the chain configuration's shape): normalised rows
    have zero mean and unit variance; dx is orthogonal to 1 and to x_hat within
    rounding."""
    torch.manual_seed(0)
    x = (torch.randn(65536, 1024, device="cuda") * 3 + 1).to(torch.bfloat16)
    dy = torch.randn(65536, 1024, device="cuda").to(torch.bfloat16)
    g = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(1024, device="cuda", dtype=torch.bfloat16)
    y = raw_ops.MusaLayerNorm(x, g, b).float()
    assert y.mean(-1).abs().max().item() < 2e-2
    assert (y.var(-1, unbiased=False) - 1).abs().max().item() < 3e-2
    dx, dgamma, dbeta = raw_ops.MusaLayerNormGrad(dy, x, g, b)
    assert dx.float().mean(-1).abs().max().item() < 2e-2
    assert_close(to_numpy(dbeta.float()), to_numpy(dy.float().sum(0)), 2e-2, 2.0, "dbeta")
    yr, nr, inv = raw_ops.MusaRmsNorm(x, g)
    assert ((nr.float() ** 2).mean(-1) - 1).abs().max().item() < 3e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keras_layer_norm_route_through_fused_batch_norm(kernel_lib, dtype):
    """Keras runs rank-2 LayerNormalization as FusedBatchNormV3 on the NCHW view
    [1, batch, features, 1] (one "channel" per row) and its gradient through
    FusedBatchNormGradV3 with the population VARIANCE
    (test/ops/fused_batchnorm_op_test.py:218-256: x of std 10, dy of std 1e-3).
    That route and the LayerNorm ops give the same normalisation."""
    rng = np.random.default_rng(42)
    dt = np_dtype(dtype)
    x = (10.0 * rng.normal(size=(128, 1536))).astype(np.float32).astype(dt)
    dy = rng.normal(scale=1e-3, size=x.shape).astype(np.float32).astype(dt)
    ones = np.ones(128, np.float32)
    zeros = np.zeros(128, np.float32)
    x4, dy4 = to_torch(x).reshape(1, 128, 1536, 1), to_torch(dy).reshape(1, 128, 1536, 1)
    e = torch.empty(0, device="cuda")
    fwd = raw_ops.FusedBatchNormV3(x4, to_torch(ones), to_torch(zeros), e, e, epsilon=1e-3,
                                   data_format="NCHW")
    grad = raw_ops.FusedBatchNormGradV3(dy4, x4, to_torch(ones), fwd[3], fwd[4], None,
                                        epsilon=1e-3, data_format="NCHW")
    g1 = np.ones(1536, dt)
    b0 = np.zeros(1536, dt)
    rt, at = (1e-4, 1e-5) if dtype == "float32" else (RTOL["lowp"], 2e-2)
    assert_close(to_numpy(fwd[0]).reshape(128, 1536), np_ref.layer_norm(x, g1, b0, 1e-3), rt, at, "y")
    want_dx = np_ref.layer_norm_grad(dy, x, g1, 1e-3)[0]
    got_dx = to_numpy(grad[0]).reshape(128, 1536)
    # the reference's own bound for this case: rtol 0.15, atol 5e-5
    assert_close(got_dx, want_dx, 0.15 if dtype == "bfloat16" else 1e-3, 5e-5 if dtype == "bfloat16" else 1e-8, "dx")
    assert np.abs(got_dx.astype(np.float64)).max() < 1e-3      # not blown up by the variance
    ln = raw_ops.MusaLayerNorm(to_torch(x), to_torch(g1), to_torch(b0), epsilon=1e-3)
    assert_close(to_numpy(ln), to_numpy(fwd[0]).reshape(128, 1536), rt, at, "layer norm op vs route")
    ln_dx = raw_ops.MusaLayerNormGrad(to_torch(dy), to_torch(x), to_torch(g1), to_torch(b0),
                                      epsilon=1e-3).dx
    assert_close(to_numpy(ln_dx), want_dx, 0.15 if dtype == "bfloat16" else 1e-3,
                 5e-5 if dtype == "bfloat16" else 1e-8, "layer norm grad op")


@pytest.mark.parametrize("packs", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [64, 256, 768, 1024, 2048, 3072, 4096])
def test_every_register_layout_gives_the_same_answers(kernel_lib, packs, n):
    """The packs-per-thread layouts (tuning key 12) differ in how a row is
    spread over threads and warps, not in what they compute."""
    lib = raw_ops._lib()
    rng = np.random.default_rng(n + packs)
    for dtype in ("float32", "bfloat16"):
        dt = np_dtype(dtype)
        x = rng.uniform(-4, 4, (300, n)).astype(dt)
        dy = rng.uniform(-1, 1, (300, n)).astype(dt)
        gamma = rng.uniform(0.5, 1.5, n).astype(dt)
        beta = rng.uniform(-0.5, 0.5, n).astype(dt)
        tx, td, tg, tb = (to_torch(a) for a in (x, dy, gamma, beta))
        lib.MusaKernelsSetTuning(12, packs)
        try:
            y = raw_ops.MusaLayerNorm(tx, tg, tb)
            dx, dgamma, dbeta = raw_ops.MusaLayerNormGrad(td, tx, tg, tb)
            ry, rn, rinv = raw_ops.MusaRmsNorm(tx, tg)
            rdx = raw_ops.MusaRmsNormGradDx(tx, rinv, tg, td)
            torch.cuda.synchronize()
        finally:
            lib.MusaKernelsSetTuning(12, 0)
        rt, at = _tol(dtype)
        assert_close(to_numpy(y), np_ref.layer_norm(x, gamma, beta), rt, at, "y")
        want = np_ref.layer_norm_grad(dy, x, gamma)
        assert_close(to_numpy(dx), want[0], rt * 10, at * 2 + 1e-5, "dx")
        assert_close(to_numpy(dgamma), want[1], rt * 10, (at + 1e-5) * 18, "dgamma")
        assert_close(to_numpy(dbeta), want[2], rt * 10, (at + 1e-5) * 18, "dbeta")
        assert_close(to_numpy(ry), np_ref.rms_norm(x, gamma)[0], rt, at, "rms y")
        assert_close(to_numpy(rdx), np_ref.rms_norm_grad_dx(x, to_numpy(rinv), gamma, dy),
                     rt * 5, at * 5 + 1e-5, "rms dx")
