"""Shared helpers of the parity tests: seeded inputs of the benchmark
configurations, dtype plumbing between NumPy and torch, tolerances."""
import numpy as np

try:
    import ml_dtypes
    NP_BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    NP_BF16 = None

# Tolerances of the parity contract: fp32 element-wise and Adam 1e-5, fp32
# BatchNorm outputs and statistics 1e-4, 16-bit types 2e-2.
RTOL = {"f32_elementwise": 1e-5, "f32_adam": 1e-5, "f32_bn": 1e-4, "lowp": 2e-2}


def np_dtype(name):
    return {"float32": np.dtype(np.float32), "float16": np.dtype(np.float16),
            "bfloat16": NP_BF16, "float64": np.dtype(np.float64),
            "int32": np.dtype(np.int32), "int64": np.dtype(np.int64)}[name]


def to_torch(a, device="cuda"):
    import torch
    a = np.ascontiguousarray(a)
    if NP_BF16 is not None and a.dtype == NP_BF16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).to(device)
    return torch.from_numpy(a).to(device)


def to_numpy(t):
    import torch
    if isinstance(t, np.ndarray):
        return t
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(NP_BF16)
    return t.numpy()


def f64(a):
    return np.asarray(a).astype(np.float64)


def assert_close(actual, expected, rtol, atol=0.0, what=""):
    a, e = f64(actual), f64(expected)
    assert a.shape == e.shape, "%s: shape %s vs %s" % (what, a.shape, e.shape)
    err = np.abs(a - e)
    tol = atol + rtol * np.abs(e)
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(
            "%s: %d of %d elements outside rtol=%g atol=%g; worst at %s: got %r, "
            "expected %r" % (what, int(bad.sum()), a.size, rtol, atol, i, a[i], e[i]))


def bn_inputs(seed, shape, dtype, mean, std, dy_std=1e-2, channel_axis=-1):
    rng = np.random.default_rng(seed)
    c = shape[channel_axis]
    x = (rng.standard_normal(shape, dtype=np.float32) * std + mean).astype(np_dtype(dtype))
    scale = rng.uniform(0.5, 1.5, c).astype(np.float32)
    offset = rng.normal(0, 0.1, c).astype(np.float32)
    dy = (rng.standard_normal(shape, dtype=np.float32) * dy_std).astype(np_dtype(dtype))
    return x, scale, offset, dy


def adam_inputs(seed, n):
    rng = np.random.default_rng(seed)
    var = rng.normal(0, 0.05, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = rng.uniform(0, 1e-6, n).astype(np.float32)
    return rng, var, m, v


ADAM_HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-7,
                  beta1_power=0.9 ** 10, beta2_power=0.999 ** 10)
