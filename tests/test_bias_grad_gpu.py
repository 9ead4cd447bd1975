"""ReluGrad, BiasAddGrad and the fused backward of the BiasAdd + Relu chain on
the GPU (through the C ABI) against the CPU oracle and the PyTorch-autograd
golden vectors."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import RTOL, assert_close, np_dtype, to_numpy, to_torch
from tensorflow_musa_extension_b200 import errors, raw_ops

pytestmark = pytest.mark.gpu

FLOATS = ["float32", "float16", "bfloat16"]


def _sum_tol(dtype, rows):
    """Column sums: fp32 accumulation error grows with the row count; 16-bit
    outputs carry one rounding of the result."""
    if dtype == "float32":
        return RTOL["f32_bn"], 1e-6 * np.sqrt(rows)
    return RTOL["lowp"], 1e-2


def _inputs(seed, shape, dtype):
    rng = np.random.default_rng(seed)
    dt = np_dtype(dtype)
    grads = rng.standard_normal(shape).astype(dt)
    feats = np.maximum(rng.standard_normal(shape), 0).astype(dt)  # a Relu output
    return grads, feats


def test_golden_vectors(golden, kernel_lib):
    g = golden["bias_grad_torch_cpu"]
    for name, fmt in (("nhwc", "NHWC"), ("nchw", "NCHW"), ("ragged2d", "NHWC")):
        for short, dtype in (("f32", "float32"), ("f16", "float16"), ("bf16", "bfloat16")):
            key = "%s/%s" % (name, short)
            dt = np_dtype(dtype)
            feats = g[key + "/features"].astype(dt)
            grads = g[key + "/gradients"].astype(dt)
            rows = grads.size // g[key + "/bias_grad"].size
            rt, at = _sum_tol(dtype, rows)
            dx, db = raw_ops.MusaBiasAddReluGrad(to_torch(grads), to_torch(feats),
                                                 data_format=fmt)
            assert np.array_equal(to_numpy(dx).astype(np.float64),
                                  g[key + "/backprops"].astype(np.float64)), key
            assert_close(to_numpy(db), g[key + "/bias_grad"], rt, at, key + " fused")
            plain = raw_ops.BiasAddGrad(to_torch(grads), data_format=fmt)
            assert_close(to_numpy(plain), g[key + "/dy_colsum"], rt, at, key + " plain")
            rg = raw_ops.ReluGrad(to_torch(grads), to_torch(feats))
            assert np.array_equal(to_numpy(rg).astype(np.float64),
                                  g[key + "/backprops"].astype(np.float64)), key


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(1, 1), (2, 3), (31, 64), (33, 65), (5, 7, 16), (4, 6, 5, 24),
                                   (1000, 1024), (257, 1000), (4099, 8), (7, 2056),
                                   (20000, 40)])
def test_fused_and_unfused_channels_last(kernel_lib, dtype, shape):
    grads, feats = _inputs(5, shape, dtype)
    want_dx, want_db = np_ref.bias_add_relu_grad(grads, feats)
    rows = grads.size // shape[-1]
    rt, at = _sum_tol(dtype, rows)
    tg, tf = to_torch(grads), to_torch(feats)
    dx, db = raw_ops.MusaBiasAddReluGrad(tg, tf)
    assert dx.dtype == tg.dtype and db.dtype == tg.dtype and tuple(db.shape) == (shape[-1],)
    assert np.array_equal(to_numpy(dx).view(np.uint8), want_dx.view(np.uint8))
    assert_close(to_numpy(db), want_db, rt, at, "fused bias_grad")
    # The un-fused pair gives the same values as the fused op.
    dx2 = raw_ops.ReluGrad(tg, tf)
    assert torch.equal(dx2.view(torch.uint8), dx.view(torch.uint8))
    db2 = raw_ops.BiasAddGrad(dx2)
    assert_close(to_numpy(db2), want_db, rt, at, "unfused bias_grad")
    assert_close(to_numpy(raw_ops.BiasAddGrad(tg)), np_ref.bias_add_grad(grads), rt, at, "plain")


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (3, 16, 8, 8), (2, 5, 1, 1), (4, 7, 3, 8),
                                   (64, 33, 7, 7), (300, 2, 3), (6, 40, 14, 14), (70, 9, 2, 2),
                                   (3, 1000, 3, 3), (500, 8, 56)])
def test_fused_and_unfused_nchw(kernel_lib, dtype, shape):
    grads, feats = _inputs(6, shape, dtype)
    want_dx, want_db = np_ref.bias_add_relu_grad(grads, feats, "NCHW")
    rows = grads.size // shape[1]
    rt, at = _sum_tol(dtype, rows)
    dx, db = raw_ops.MusaBiasAddReluGrad(to_torch(grads), to_torch(feats), data_format="NCHW")
    assert np.array_equal(to_numpy(dx).view(np.uint8), want_dx.view(np.uint8))
    assert_close(to_numpy(db), want_db, rt, at, "fused bias_grad")
    assert_close(to_numpy(raw_ops.BiasAddGrad(to_torch(grads), data_format="NCHW")),
                 np_ref.bias_add_grad(grads, "NCHW"), rt, at, "plain")


@pytest.mark.parametrize("dtype", ["float64", "int32", "int64"])
def test_bias_add_grad_exact_dtypes(kernel_lib, dtype):
    rng = np.random.default_rng(8)
    dt = np_dtype(dtype)
    for shape, fmt in [((1031, 9), "NHWC"), ((64, 128), "NHWC"), ((5, 4, 6, 3), "NCHW")]:
        g = (rng.standard_normal(shape) * 1000).astype(dt)
        got = to_numpy(raw_ops.BiasAddGrad(to_torch(g), data_format=fmt))
        want = np_ref.bias_add_grad(g, fmt)
        assert got.dtype == dt
        if dtype == "float64":
            assert_close(got, want, 1e-12, 1e-9)
        else:
            assert np.array_equal(got, want)
    # Integer sums wrap in the tensor's own width.
    big = np.full((8, 4), 2 ** 30, np.int32)
    assert np.array_equal(to_numpy(raw_ops.BiasAddGrad(to_torch(big))),
                          np_ref.bias_add_grad(big))


def test_results_are_reproducible(kernel_lib):
    """Fixed-order sums: two runs give the same bits."""
    grads, feats = _inputs(9, (30011, 96), "float32")
    tg, tf = to_torch(grads), to_torch(feats)
    a = raw_ops.MusaBiasAddReluGrad(tg, tf).bias_grad
    b = raw_ops.MusaBiasAddReluGrad(tg, tf).bias_grad
    assert torch.equal(a, b)


def test_edge_cases(kernel_lib):
    # 1-D input is its own gradient (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:52-58).
    v = torch.tensor([1.5, -2.0, 3.0], device="cuda")
    assert torch.equal(raw_ops.BiasAddGrad(v), v)
    # Empty inputs give zeros (test/ops/biasadd_grad_op_test.py:88-127).
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for shape in [(4096, 0, 512), (4096, 0, 128), (0, 16)]:
            out = raw_ops.BiasAddGrad(torch.empty(shape, dtype=dtype, device="cuda"))
            assert out.dtype == dtype and tuple(out.shape) == (shape[-1],)
            assert not out.float().abs().sum().item()
    out = raw_ops.ReluGrad(torch.empty((0, 4), device="cuda"), torch.empty((0, 4), device="cuda"))
    assert tuple(out.shape) == (0, 4)
    # Inactive positions: zero and negative-zero features, NaN features.
    gr = torch.tensor([1.0, 2.0, 3.0, 4.0], device="cuda")
    ft = torch.tensor([0.0, -0.0, float("nan"), 1e-30], device="cuda")
    assert to_numpy(raw_ops.ReluGrad(gr, ft)).tolist() == [0.0, 0.0, 0.0, 4.0]
    with pytest.raises(errors.InvalidArgumentError, match="same shape"):
        raw_ops.ReluGrad(torch.zeros((2, 3), device="cuda"), torch.zeros((3, 2), device="cuda"))
    with pytest.raises(errors.InvalidArgumentError, match="data format"):
        raw_ops.BiasAddGrad(torch.zeros((2, 3), device="cuda"), data_format="NCDHW")
    with pytest.raises(errors.InvalidArgumentError):
        raw_ops.ReluGrad(torch.zeros((2, 3), dtype=torch.float64, device="cuda"),
                         torch.zeros((2, 3), dtype=torch.float64, device="cuda"))


def test_unaligned_views_take_the_element_path(kernel_lib):
    """Pointers off the 16-byte grid and channel counts that are no multiple of
    the pack width."""
    for dtype in FLOATS:
        grads, feats = _inputs(10, (515, 27), dtype)
        want_dx, want_db = np_ref.bias_add_relu_grad(grads, feats)
        # A view that starts one element into a larger buffer.
        def shifted(a):
            t = to_torch(a).reshape(-1)
            buf = torch.empty(t.numel() + 1, dtype=t.dtype, device="cuda")
            buf[1:].copy_(t)
            return buf[1:].view(a.shape)
        tg, tf = shifted(grads), shifted(feats)
        assert tg.data_ptr() % 16 != 0
        lib = raw_ops._lib()
        dx = torch.empty_like(to_torch(grads))
        db = torch.empty(27, dtype=dx.dtype, device="cuda")
        nbytes = lib.BiasGradWorkspaceBytes(515, 27, 1, dx.element_size())
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        fn = getattr(lib, "LaunchBiasAddReluGrad_" + raw_ops._SUFFIX[dx.dtype])
        rc = fn(tg.data_ptr(), tf.data_ptr(), dx.data_ptr(), db.data_ptr(), 515, 27, 1,
                ws.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(to_numpy(dx).view(np.uint8), want_dx.view(np.uint8))
        rt, at = _sum_tol(dtype, 515)
        assert_close(to_numpy(db), want_db, rt, at, dtype)


def test_workspace_is_checked(kernel_lib):
    lib = raw_ops._lib()
    g = torch.randn(1024, 64, device="cuda")
    out = torch.empty(64, device="cuda")
    need = lib.BiasGradWorkspaceBytes(1024, 64, 1, 4)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert lib.LaunchBiasAddGrad_F32(g.data_ptr(), out.data_ptr(), 1024, 64, 1,
                                     ws.data_ptr(), need - 1, s) == -2
    assert lib.LaunchBiasAddGrad_F32(g.data_ptr(), out.data_ptr(), 1024, 64, 1,
                                     None, need, s) == -2
    assert lib.LaunchBiasAddGrad_F32(g.data_ptr(), out.data_ptr(), -1, 64, 1,
                                     ws.data_ptr(), need, s) == -1
    assert lib.LaunchBiasAddGrad_F32(g.data_ptr(), out.data_ptr(), 1024, 64, 1,
                                     ws.data_ptr(), need, s) == 0
    torch.cuda.synchronize()
    assert_close(to_numpy(out), to_numpy(g).astype(np.float64).sum(0), 1e-4, 1e-4)


def test_full_size_properties(kernel_lib):
    """The benchmark's chain shape, f16 [65536, 1024]: the fused op equals the
    un-fused pair bit for bit, and the column sum is linear
    (sum over two row halves = sum over all rows) within fp32 accumulation."""
    torch.manual_seed(0)
    rows, c = 65536, 1024
    g = torch.randn(rows, c, device="cuda", dtype=torch.float16)
    f = torch.relu(torch.randn(rows, c, device="cuda", dtype=torch.float16))
    dx, db = raw_ops.MusaBiasAddReluGrad(g, f)
    dx2 = raw_ops.ReluGrad(g, f)
    assert torch.equal(dx.view(torch.int16), dx2.view(torch.int16))
    assert torch.equal(dx, torch.where(f > 0, g, torch.zeros_like(g)))
    db2 = raw_ops.BiasAddGrad(dx2)
    want = dx.double().sum(0)
    assert_close(to_numpy(db), to_numpy(want), RTOL["lowp"], 0.05, "fused")
    assert_close(to_numpy(db2), to_numpy(want), RTOL["lowp"], 0.05, "unfused")
    top = raw_ops.BiasAddGrad(dx[: rows // 2].contiguous()).float()
    bot = raw_ops.BiasAddGrad(dx[rows // 2:].contiguous()).float()
    assert_close(to_numpy(top + bot), to_numpy(want), RTOL["lowp"], 0.3, "halves")
