"""Tensors of more than 2^31 elements: every index of the path is 64-bit.

The CPU oracle cannot walk 2^31 elements in test time, so each case checks
size-independent properties: an element-wise or row-wise op gives the same
bits on a slice as on the whole tensor (slices are taken at the start, across
element 2^31 and at the ragged end), the oracle is run on those slices, and
column sums are compared with float64 sums accumulated chunk by chunk."""
import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import NP_BF16, RTOL, assert_close, to_numpy
from tensorflow_musa_extension_b200 import raw_ops

pytestmark = pytest.mark.gpu

LIMIT = 1 << 31
EPS = 1e-3


@pytest.fixture(autouse=True)
def _release_device_memory():
    yield
    raw_ops._ws_cache.clear()
    torch.cuda.empty_cache()


def _row_windows(rows, row_elems, span=5):
    """Row ranges at the start, across element 2^31 and at the end."""
    mid = LIMIT // row_elems
    return [(0, span), (mid - span, min(rows, mid + span)), (rows - span, rows)]


def _same_bits(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert torch.equal(a.view(torch.int16) if a.element_size() == 2 else a,
                       b.view(torch.int16) if b.element_size() == 2 else b), what


def _column_sums(t, weight=None, chunk=1 << 17):
    """float64 column sums of a [rows, cols] tensor (times `weight`)."""
    acc = torch.zeros(t.shape[1], dtype=torch.float64, device=t.device)
    for r in range(0, t.shape[0], chunk):
        part = t[r:r + chunk].double()
        if weight is not None:
            part = part * weight[r:r + chunk].double()
        acc += part.sum(0)
    return acc


@pytest.mark.parametrize("chain", ["relu", "swish"])
def test_bias_chain_channels_last(kernel_lib, chain):
    rows, cols = (1 << 21) + 3, 1024
    assert rows * cols > LIMIT
    op, ref = {"relu": (raw_ops.MusaBiasAddRelu, np_ref.bias_add_relu),
               "swish": (raw_ops.MusaBiasAddSwish, np_ref.bias_add_swish)}[chain]
    torch.manual_seed(5)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.float16)
    b = (torch.randn(cols, device="cuda") * 0.1).half()
    y = op(x, b)
    for lo, hi in _row_windows(rows, cols):
        _same_bits(op(x[lo:hi], b), y[lo:hi], "%s rows %d:%d" % (chain, lo, hi))
        assert_close(to_numpy(y[lo:hi]), ref(to_numpy(x[lo:hi]), to_numpy(b)),
                     RTOL["lowp"], 1e-3, chain)


def test_bias_chain_planes(kernel_lib):
    # 7x7 planes: flat packs that cross plane boundaries.
    n, c, h = 684_800, 64, 7
    plane = c * h * h
    assert n * plane > LIMIT
    torch.manual_seed(6)
    x = torch.randn(n, c, h, h, device="cuda", dtype=torch.float16)
    b = (torch.randn(c, device="cuda") * 0.1).half()
    y = raw_ops.MusaBiasAddRelu(x, b, data_format="NCHW")
    for lo, hi in _row_windows(n, plane, span=3):
        _same_bits(raw_ops.MusaBiasAddRelu(x[lo:hi], b, data_format="NCHW"), y[lo:hi],
                   "images %d:%d" % (lo, hi))
        assert_close(to_numpy(y[lo:hi]),
                     np_ref.bias_add_relu(to_numpy(x[lo:hi]), to_numpy(b), "NCHW"),
                     RTOL["lowp"], 1e-3, "planes")


def test_adam_bf16_state(kernel_lib):
    n = LIMIT + 8205  # not a whole number of 128-bit packs
    torch.manual_seed(7)
    dt = torch.bfloat16
    var = torch.randn(n, device="cuda", dtype=dt) * 0.5
    m = torch.randn(n, device="cuda", dtype=dt) * 1e-2
    v = torch.rand(n, device="cuda", dtype=dt) * 1e-3
    g = torch.randn(n, device="cuda", dtype=dt) * 0.1
    windows = [(0, 4096), (LIMIT - 2048, LIMIT + 2048), (n - 4099, n)]
    before = [tuple(t[lo:hi].clone() for t in (var, m, v)) for lo, hi in windows]
    args = (0.9 ** 10, 0.999 ** 10, 1e-2, 0.9, 0.999, 1e-4)
    # The op reads its scalar inputs in the state's type.
    ref_args = [np.asarray(a).astype(NP_BF16) for a in args]
    raw_ops.ResourceApplyAdam(var, m, v, *args, g)
    for (lo, hi), (v0, m0, s0) in zip(windows, before):
        want = np_ref.apply_adam(to_numpy(v0), to_numpy(m0), to_numpy(s0), *ref_args,
                                 to_numpy(g[lo:hi]))
        raw_ops.ResourceApplyAdam(v0, m0, s0, *args, g[lo:hi].clone())
        for name, whole, part, ref in zip(("var", "m", "v"), (var, m, v), (v0, m0, s0), want):
            _same_bits(part, whole[lo:hi], "%s %d:%d" % (name, lo, hi))
            assert_close(to_numpy(part), ref, RTOL["lowp"], 1e-6, name)


def test_adam_fp32(kernel_lib):
    n = LIMIT + 8205
    torch.manual_seed(12)
    var = torch.randn(n, device="cuda").mul_(0.05)
    m = torch.randn(n, device="cuda").mul_(1e-4)
    v = torch.rand(n, device="cuda").mul_(1e-6)
    g = torch.randn(n, device="cuda").mul_(1e-3)
    windows = [(0, 4096), (LIMIT - 2048, LIMIT + 2048), (n - 4099, n)]
    before = [tuple(t[lo:hi].clone() for t in (var, m, v)) for lo, hi in windows]
    args = (0.9 ** 10, 0.999 ** 10, 1e-3, 0.9, 0.999, 1e-7)
    raw_ops.ResourceApplyAdam(var, m, v, *args, g)
    for (lo, hi), (v0, m0, s0) in zip(windows, before):
        want = np_ref.apply_adam(to_numpy(v0), to_numpy(m0), to_numpy(s0), *args,
                                 to_numpy(g[lo:hi]))
        raw_ops.ResourceApplyAdam(v0, m0, s0, *args, g[lo:hi].clone())
        for name, whole, part, ref, atol in zip(("var", "m", "v"), (var, m, v), (v0, m0, s0),
                                                want, (1e-8, 1e-10, 1e-14)):
            assert torch.equal(part, whole[lo:hi]), "%s %d:%d" % (name, lo, hi)
            assert_close(to_numpy(part), ref, RTOL["f32_adam"], atol, name)


def _bn_rows(x, mean, var, scale, offset, lo, hi):
    xs = x[lo:hi].double()
    inv = torch.rsqrt(var.double() + EPS)
    return ((xs - mean.double()) * inv * scale.double() + offset.double()).cpu().numpy()


def test_batchnorm_channels_last(kernel_lib):
    rows, c = (1 << 23) + 5, 256
    assert rows * c > LIMIT
    torch.manual_seed(8)
    x = torch.randn(rows, c, device="cuda", dtype=torch.bfloat16) * 3 + 1
    scale = torch.rand(c, device="cuda") + 0.5
    offset = torch.randn(c, device="cuda") * 0.1
    out = raw_ops.FusedBatchNormV3(x, scale, offset, None, None, epsilon=EPS)
    mean = _column_sums(x) / rows
    ex2 = _column_sums(x, x) / rows
    pop_var = ex2 - mean * mean
    assert_close(to_numpy(out.reserve_space_1), mean.cpu().numpy(), RTOL["f32_bn"], 1e-5, "mean")
    assert_close(to_numpy(out.reserve_space_2), pop_var.cpu().numpy(), RTOL["f32_bn"], 0, "var")
    assert_close(to_numpy(out.batch_variance), (pop_var * rows / (rows - 1)).cpu().numpy(),
                 RTOL["f32_bn"], 0, "batch_variance")
    for lo, hi in _row_windows(rows, c):
        want = _bn_rows(x, out.reserve_space_1, out.reserve_space_2, scale, offset, lo, hi)
        assert_close(to_numpy(out.y[lo:hi]), want, RTOL["lowp"], 1e-2, "y")
    saved_mean, saved_var = out.reserve_space_1, out.reserve_space_2
    del out
    torch.cuda.empty_cache()

    dy = torch.randn(rows, c, device="cuda", dtype=torch.bfloat16) * 1e-2
    grad = raw_ops.FusedBatchNormGradV3(dy, x, scale, saved_mean, saved_var, epsilon=EPS)
    inv = torch.rsqrt(saved_var.double() + EPS)
    doffset = _column_sums(dy)
    dscale = (_column_sums(dy, x) - saved_mean.double() * doffset) * inv
    # Sums of 8 M terms of either sign: the tolerance is relative to their scale.
    scale_of = float(np.sqrt(rows) * 1e-2)
    assert_close(to_numpy(grad.offset_backprop), doffset.cpu().numpy(), 1e-3, 1e-3 * scale_of,
                 "doffset")
    assert_close(to_numpy(grad.scale_backprop), dscale.cpu().numpy(), 1e-3, 1e-3 * scale_of,
                 "dscale")
    for lo, hi in _row_windows(rows, c):
        xh = (x[lo:hi].double() - saved_mean.double()) * inv
        want = scale.double() * inv * (dy[lo:hi].double() - doffset / rows - xh * dscale / rows)
        assert_close(to_numpy(grad.x_backprop[lo:hi]), want.cpu().numpy(), RTOL["lowp"], 1e-4,
                     "dx")


def test_batchnorm_planes(kernel_lib):
    n, c, h = 4097, 512, 32
    assert n * c * h * h > LIMIT
    torch.manual_seed(9)
    x = torch.randn(n, c, h, h, device="cuda", dtype=torch.bfloat16) * 2 + 0.5
    scale = torch.rand(c, device="cuda") + 0.5
    offset = torch.randn(c, device="cuda") * 0.1
    out = raw_ops.FusedBatchNormV3(x, scale, offset, None, None, epsilon=EPS,
                                   data_format="NCHW")
    count = n * h * h
    s1 = torch.zeros(c, dtype=torch.float64, device="cuda")
    s2 = torch.zeros(c, dtype=torch.float64, device="cuda")
    for i in range(0, n, 128):
        part = x[i:i + 128].double()
        s1 += part.sum((0, 2, 3))
        s2 += (part * part).sum((0, 2, 3))
    mean = s1 / count
    pop_var = s2 / count - mean * mean
    assert_close(to_numpy(out.reserve_space_1), mean.cpu().numpy(), RTOL["f32_bn"], 1e-5, "mean")
    assert_close(to_numpy(out.reserve_space_2), pop_var.cpu().numpy(), RTOL["f32_bn"], 0, "var")
    for lo, hi in _row_windows(n, c * h * h, span=2):
        shape = (1, c, 1, 1)
        inv = torch.rsqrt(out.reserve_space_2.double() + EPS).view(shape)
        want = (x[lo:hi].double() - out.reserve_space_1.double().view(shape)) * inv * \
            scale.double().view(shape) + offset.double().view(shape)
        assert_close(to_numpy(out.y[lo:hi]), want.cpu().numpy(), RTOL["lowp"], 1e-2, "y")


def test_bias_relu_grad(kernel_lib):
    rows, cols = (1 << 21) + 3, 1024
    torch.manual_seed(10)
    feat = torch.relu(torch.randn(rows, cols, device="cuda", dtype=torch.float16))
    g = torch.randn(rows, cols, device="cuda", dtype=torch.float16)
    backprops, bias_grad = raw_ops.MusaBiasAddReluGrad(g, feat)
    for lo, hi in _row_windows(rows, cols):
        want = np_ref.relu_grad(to_numpy(g[lo:hi]), to_numpy(feat[lo:hi]))
        assert np.array_equal(to_numpy(backprops[lo:hi]), want)
    want_bias = _column_sums(backprops)
    assert_close(to_numpy(bias_grad), want_bias.cpu().numpy(), 2e-3, 1.0, "bias_grad")
    plain = raw_ops.BiasAddGrad(backprops)
    assert_close(to_numpy(plain), want_bias.cpu().numpy(), 2e-3, 1.0, "BiasAddGrad")


def test_row_norms(kernel_lib):
    from tensorflow_musa_extension_b200 import norm_ops
    rows, cols = (1 << 21) + 3, 1024
    torch.manual_seed(11)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) * 3 + 1
    gamma = (torch.rand(cols, device="cuda") + 0.5).bfloat16()
    beta = (torch.randn(cols, device="cuda") * 0.1).bfloat16()
    y = norm_ops.MusaLayerNorm(x, gamma, beta)
    for lo, hi in _row_windows(rows, cols):
        _same_bits(norm_ops.MusaLayerNorm(x[lo:hi], gamma, beta), y[lo:hi], "LayerNorm rows")
        want = np_ref.layer_norm(to_numpy(x[lo:hi]), to_numpy(gamma), to_numpy(beta))
        assert_close(to_numpy(y[lo:hi]), want, RTOL["lowp"], 1e-2, "LayerNorm")
    del y
    torch.cuda.empty_cache()

    dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    dx, dgamma, dbeta = norm_ops.MusaLayerNormGrad(dy, x, gamma, beta)
    for lo, hi in _row_windows(rows, cols):
        part = norm_ops.MusaLayerNormGrad(dy[lo:hi], x[lo:hi], gamma, beta)[0]
        _same_bits(part, dx[lo:hi], "LayerNormGrad rows")
    assert_close(to_numpy(dbeta), _column_sums(dy).cpu().numpy(), 1e-2, 8.0, "dbeta")
    del dx
    torch.cuda.empty_cache()

    out = norm_ops.MusaRmsNorm(x, gamma)
    for lo, hi in _row_windows(rows, cols):
        part = norm_ops.MusaRmsNorm(x[lo:hi], gamma)
        for whole, piece in zip(out, part):
            _same_bits(piece, whole[lo:hi], "RmsNorm rows")
