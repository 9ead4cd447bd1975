"""BiasAdd + activation chains on the GPU (through the C ABI) against the CPU
oracle of the un-fused TensorFlow ops."""
import numpy as np
import pytest
import torch

from oracle import c_ref, np_ref
from helpers import NP_BF16, RTOL, assert_close, np_dtype, to_numpy, to_torch
from tensorflow_musa_extension_b200 import errors, raw_ops

pytestmark = pytest.mark.gpu

FUSED = {
    "bias_add": (raw_ops.BiasAdd, np_ref.bias_add),
    "relu": (raw_ops.MusaBiasAddRelu, np_ref.bias_add_relu),
    "swish": (raw_ops.MusaBiasAddSwish, np_ref.bias_add_swish),
    "sigmoid": (raw_ops.MusaBiasAddSigmoid, np_ref.bias_add_sigmoid),
}


def _tol(dtype):
    if dtype == "float32":
        return RTOL["f32_elementwise"], 1e-7
    return RTOL["lowp"], 1e-3


def test_reference_literals(golden, kernel_lib):
    g = golden["elementwise_literals"]
    assert_close(to_numpy(raw_ops.Relu(to_torch(g["relu/in"]))), g["relu/out"], 0)
    assert_close(to_numpy(raw_ops.Sigmoid(to_torch(g["sigmoid/in"]))), g["sigmoid/out"],
                 RTOL["f32_elementwise"], 1e-38)
    assert_close(to_numpy(raw_ops.BiasAdd(to_torch(g["biasadd/x"]), to_torch(g["biasadd/b"]))),
                 g["biasadd/out_nhwc"], 0)
    assert_close(to_numpy(raw_ops.BiasAdd(to_torch(g["biasadd/x_nchw"]),
                                          to_torch(g["biasadd/b_nchw"]), data_format="NCHW")),
                 g["biasadd/out_nchw"], 0)
    out = raw_ops.BiasAdd(to_torch(g["biasadd/x_i32"]), to_torch(g["biasadd/b_i32"]))
    assert out.dtype == torch.int32
    assert np.array_equal(to_numpy(out), g["biasadd/out_i32"])


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("chain", sorted(FUSED))
@pytest.mark.parametrize("shape", [(1, 1), (2, 3), (31, 64), (33, 65), (32, 8), (5, 7, 16),
                                   (4, 6, 5, 24), (1000, 1024), (257, 1000)])
def test_chains_channels_last(kernel_lib, dtype, chain, shape):
    rng = np.random.default_rng(2)
    dt = np_dtype(dtype)
    x = rng.standard_normal(shape).astype(dt)
    b = rng.normal(0, 0.1, shape[-1]).astype(dt)
    op, ref = FUSED[chain]
    rt, at = _tol(dtype)
    assert_close(to_numpy(op(to_torch(x), to_torch(b))), ref(x, b), rt, at, chain)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("chain", sorted(FUSED))
@pytest.mark.parametrize("shape", [(2, 3, 4, 5), (3, 16, 8, 8), (2, 5, 1, 1), (4, 7, 3, 8),
                                   (3, 5, 7, 7), (2, 9, 14, 14), (5, 3, 3, 3), (33, 40, 7, 7),
                                   (2, 3, 1, 13)])
def test_chains_nchw(kernel_lib, dtype, chain, shape):
    rng = np.random.default_rng(21)
    dt = np_dtype(dtype)
    x = rng.standard_normal(shape).astype(dt)
    b = rng.normal(0, 0.1, shape[1]).astype(dt)
    op, ref = FUSED[chain]
    rt, at = _tol(dtype)
    got = op(to_torch(x), to_torch(b), data_format="NCHW")
    assert_close(to_numpy(got), ref(x, b, "NCHW"), rt, at, chain)


@pytest.mark.parametrize("dtype", ["float64", "int32", "int64"])
def test_bias_add_exact_dtypes(kernel_lib, dtype):
    rng = np.random.default_rng(3)
    dt = np_dtype(dtype)
    x = (rng.standard_normal((17, 9)) * 100).astype(dt)
    b = (rng.standard_normal(9) * 10).astype(dt)
    got = to_numpy(raw_ops.BiasAdd(to_torch(x), to_torch(b)))
    assert got.dtype == dt and np.array_equal(got, x + b)
    xn = (rng.standard_normal((3, 4, 5)) * 100).astype(dt)
    bn = (rng.standard_normal(4) * 10).astype(dt)
    got = to_numpy(raw_ops.BiasAdd(to_torch(xn), to_torch(bn), data_format="NCHW"))
    assert np.array_equal(got, xn + bn.reshape(1, 4, 1))


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16", "float64"])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 4096, 100003])
def test_standalone_relu(kernel_lib, dtype, n):
    rng = np.random.default_rng(4)
    x = rng.standard_normal(n).astype(np_dtype(dtype))
    assert np.array_equal(to_numpy(raw_ops.Relu(to_torch(x))).astype(np.float64),
                          np_ref.relu(x).astype(np.float64))


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_standalone_sigmoid_wide_range(kernel_lib, dtype):
    x = np.concatenate([np.linspace(-100, 100, 4001),
                        np.random.default_rng(5).standard_normal(5000)]).astype(np_dtype(dtype))
    rt, at = _tol(dtype)
    at = 1e-38 if dtype == "float32" else 1e-7
    assert_close(to_numpy(raw_ops.Sigmoid(to_torch(x))), np_ref.sigmoid(x), rt, at)


def test_misaligned_views(kernel_lib):
    rng = np.random.default_rng(6)
    x = rng.standard_normal(64 * 16 + 1).astype(np.float16)
    b = rng.normal(0, 0.1, 17).astype(np.float16)
    tx = to_torch(x)[1:].view(64, 16)      # 2-byte offset: no 128-bit path
    tb = to_torch(b)[1:]
    got = raw_ops.MusaBiasAddRelu(tx, tb)
    assert_close(to_numpy(got), np_ref.bias_add_relu(x[1:].reshape(64, 16), b[1:]), 0)


def test_errors_and_empty(kernel_lib):
    x = torch.zeros(4, 8, device="cuda")
    with pytest.raises(errors.InvalidArgumentError, match="Dimension mismatch in BiasAdd"):
        raw_ops.BiasAdd(x, torch.zeros(7, device="cuda"))
    with pytest.raises(errors.InvalidArgumentError, match="Biases must be 1D"):
        raw_ops.BiasAdd(x, torch.zeros(1, 8, device="cuda"))
    with pytest.raises(errors.InvalidArgumentError, match="at least 2D"):
        raw_ops.BiasAdd(torch.zeros(8, device="cuda"), torch.zeros(8, device="cuda"))
    with pytest.raises(errors.InvalidArgumentError):
        raw_ops.Sigmoid(torch.zeros(8, device="cuda", dtype=torch.int32))
    assert raw_ops.BiasAdd(torch.zeros(0, 8, device="cuda"),
                           torch.zeros(8, device="cuda")).shape == (0, 8)
    assert raw_ops.BiasAdd(x, torch.zeros(0, device="cuda")).shape == (4, 8)


def test_host_buffers_round_trip(kernel_lib):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((100, 32)).astype(NP_BF16)
    b = rng.normal(0, 0.1, 32).astype(NP_BF16)
    got = raw_ops.MusaBiasAddSwish(x, b)
    assert isinstance(got, np.ndarray) and got.dtype == NP_BF16
    assert_close(got, np_ref.bias_add_swish(x, b), RTOL["lowp"], 1e-3)
    got = raw_ops.MusaBiasAddRelu(torch.from_numpy(x.astype(np.float32)),
                                  torch.from_numpy(b.astype(np.float32)))
    assert isinstance(got, torch.Tensor) and not got.is_cuda


@pytest.mark.parametrize("chain,act", [("relu", 1), ("swish", 2)])
def test_full_size_fp16_chain(kernel_lib, chain, act):
    """The benchmark shape: fp16 [65536, 1024] with a [1024] bias."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((65536, 1024), dtype=np.float32).astype(np.float16)
    b = rng.normal(0, 0.1, 1024).astype(np.float16)
    op, _ = FUSED[chain]
    got = to_numpy(op(to_torch(x), to_torch(b)))
    want = c_ref.bias_act(x, b, act)
    if chain == "relu":
        assert np.array_equal(got, want)        # add + max round identically
    else:
        assert_close(got, want, RTOL["lowp"], 1e-3, chain)
        # and tighter in aggregate: one fp16 ulp at most, rarely
        ulp_off = np.abs(got.view(np.int16).astype(np.int32)
                         - want.view(np.int16).astype(np.int32))
        assert ulp_off.max() <= 4 and (ulp_off > 0).mean() < 0.5


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_sigmoid_quads_with_far_negative_members(kernel_lib, dtype):
    """Far negative and far positive inputs next to ordinary ones: every
    element comes out right to relative precision (no cancellation on the
    negative side, no overflow spilling into neighbours of the same pack)."""
    dt = np_dtype(dtype)
    base = np.array([0.5, -1.0, 2.0, -3.0, 10.0, -10.0, 0.0, 4.0], np.float32)
    rows = []
    for pos in range(8):
        for far in (-20.0, -21.0, -30.0, -60.0, -87.0, -100.0, -1000.0, 25.0, 90.0):
            r = base.copy()
            r[pos] = far
            rows.append(r)
    x = np.stack(rows).astype(dt)
    got = to_numpy(raw_ops.Sigmoid(to_torch(x)))
    want = np_ref.sigmoid(x)
    tiny = 1e-7 if dtype == "float16" else 1e-37      # below these the types flush to zero
    assert_close(got, want, RTOL["lowp"], tiny, "sigmoid")
    b = np.zeros(8, dt)
    sw = to_numpy(raw_ops.MusaBiasAddSwish(to_torch(x), to_torch(b)))
    assert_close(sw, np_ref.bias_add_swish(x, b), RTOL["lowp"], tiny * 1000, "swish")
