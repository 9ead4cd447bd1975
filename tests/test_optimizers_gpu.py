"""Nadam, RMSProp (plain and centered) and gradient descent (single, mixed,
grouped) on the GPU, through the op front end and the C ABI, against the CPU
oracle and the float64 golden vectors."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import NP_BF16, RTOL, assert_close, np_dtype, to_numpy, to_torch
from tensorflow_musa_extension_b200 import errors, raw_ops
from tensorflow_musa_extension_b200.raw_ops import Variable

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "float16", "bfloat16", "float64"]


def _tol(dtype):
    if dtype == "float32":
        return RTOL["f32_adam"], 1e-7
    if dtype == "float64":
        return 1e-12, 1e-14
    return RTOL["lowp"], 1e-3


def _rand_states(seed, n, dtype, count):
    rng = np.random.default_rng(seed)
    dt = np_dtype(dtype)
    var = rng.standard_normal(n).astype(dt)
    others = [rng.standard_normal(n) * 0.01 for _ in range(count - 1)]
    grad = rng.standard_normal(n).astype(dt)
    return var, others, grad


# ------------------------------------------------------------------ golden --

def test_golden_vectors(golden, kernel_lib):
    g = golden["optimizer_cases"]
    rt, at = 2e-6, 1e-7
    for case in ("basic", "small", "half"):
        key = "nadam/" + case
        t = [to_torch(g["%s/%s" % (key, n)]) for n in ("var", "m", "v")]
        raw_ops.ResourceApplyNadam(*t, *g[key + "/hyper"], to_torch(g[key + "/grad"]))
        for x, name in zip(t, ("var_out", "m_out", "v_out")):
            assert_close(to_numpy(x), g[key + "/" + name], rt, at, key + name)
    for case in ("basic", "dtypes", "zero_grad", "negative_grad"):
        key = "rmsprop/" + case
        t = [to_torch(g["%s/%s" % (key, n)]) for n in ("var", "ms", "mom")]
        raw_ops.ResourceApplyRMSProp(*t, *g[key + "/hyper"], to_torch(g[key + "/grad"]))
        for x, name in zip(t, ("var_out", "ms_out", "mom_out")):
            assert_close(to_numpy(x), g[key + "/" + name], rt, at, key + name)
    for case in ("basic", "dtypes"):
        key = "centered_rmsprop/" + case
        t = [to_torch(g["%s/%s" % (key, n)]) for n in ("var", "mg", "ms", "mom")]
        raw_ops.ResourceApplyCenteredRMSProp(*t, *g[key + "/hyper"],
                                             to_torch(g[key + "/grad"]))
        for x, name in zip(t, ("var_out", "mg_out", "ms_out", "mom_out")):
            assert_close(to_numpy(x), g[key + "/" + name], rt, at, key + name)
    for case in ("vector", "matrix", "locking"):
        key = "sgd/" + case
        var = to_torch(g[key + "/var"])
        raw_ops.ResourceApplyGradientDescent(var, float(g[key + "/alpha"]),
                                             to_torch(g[key + "/grad"]), use_locking=True)
        assert_close(to_numpy(var), g[key + "/var_out"], 2e-7, 1e-7, key)


# ------------------------------------------------------------------- Nadam --

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_nadam_matches_oracle(kernel_lib, dtype, n):
    rng = np.random.default_rng(n)
    dt = np_dtype(dtype)
    var = rng.uniform(-1, 1, n).astype(dt)
    m = rng.uniform(-1, 1, n).astype(dt)
    v = rng.uniform(0.1, 1, n).astype(dt)
    grad = rng.uniform(-1, 1, n).astype(dt)
    hyper = (0.9, 0.99, 0.01, 0.9, 0.99, 1e-8)
    # The op reads every scalar as T first.
    hyper_t = tuple(float(np.asarray(h).astype(dt).astype(np.float64)) for h in hyper)
    want = np_ref.apply_nadam(var, m, v, *hyper_t, grad)
    tv, tm, tvv = Variable(to_torch(var), "var"), Variable(to_torch(m), "m"), Variable(to_torch(v), "v")
    assert raw_ops.ResourceApplyNadam(tv, tm, tvv, *hyper, to_torch(grad)) is None
    rt, at = _tol(dtype)
    if dtype == "float64":
        rt, at = 1e-6, 1e-7       # the scalars travel as float (the reference's launcher)
    for got, w, name in zip((tv, tm, tvv), want, ("var", "m", "v")):
        assert_close(to_numpy(got.tensor()), w, rt, at, "%s %s" % (dtype, name))


def test_nadam_errors(kernel_lib):
    ok = torch.zeros(4, device="cuda")
    with pytest.raises(errors.FailedPreconditionError, match="Nadam variables"):
        raw_ops.ResourceApplyNadam(Variable(ok.clone()), Variable(None), Variable(ok.clone()),
                                   0.9, 0.99, 0.01, 0.9, 0.99, 1e-8, ok)
    with pytest.raises(errors.InvalidArgumentError, match="same shape"):
        raw_ops.ResourceApplyNadam(ok.clone(), ok.clone(), ok.clone(), 0.9, 0.99, 0.01, 0.9,
                                   0.99, 1e-8, torch.zeros(5, device="cuda"))
    # Empty tensors launch nothing.
    e = torch.zeros(0, device="cuda")
    raw_ops.ResourceApplyNadam(e, e.clone(), e.clone(), 0.9, 0.99, 0.01, 0.9, 0.99, 1e-8, e)


# ----------------------------------------------------------------- RMSProp --

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1,), (7,), (33, 9), (1000, 129), (2, 3, 4, 5)])
def test_rms_prop_matches_oracle(kernel_lib, dtype, shape):
    rng = np.random.RandomState(sum(shape))   # as the reference's shape test seeds it
    dt = np_dtype(dtype)
    var = rng.randn(*shape).astype(np.float32).astype(dt)
    ms = (np.abs(rng.randn(*shape).astype(np.float32)) * 0.1).astype(dt)
    mom = (rng.randn(*shape).astype(np.float32) * 0.01).astype(dt)
    grad = rng.randn(*shape).astype(np.float32).astype(dt)
    hyper = (0.01, 0.9, 0.9, 1e-7)
    hyper_t = tuple(float(np.asarray(h).astype(dt).astype(np.float64)) for h in hyper)
    want = np_ref.apply_rms_prop(var, ms, mom, *hyper_t, grad)
    t = [to_torch(a) for a in (var, ms, mom)]
    out = raw_ops.ApplyRMSProp(*t, *hyper, to_torch(grad), use_locking=True)
    assert out.data_ptr() == t[0].data_ptr()            # output 0 forwards var
    rt, at = _tol(dtype)
    for got, w, name in zip(t, want, ("var", "ms", "mom")):
        assert_close(to_numpy(got), w, rt, at, "%s %s" % (dtype, name))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(6,), (33, 9), (1000, 129)])
def test_centered_rms_prop_matches_oracle(kernel_lib, dtype, shape):
    rng = np.random.RandomState(sum(shape))
    dt = np_dtype(dtype)
    var = rng.randn(*shape).astype(np.float32).astype(dt)
    mg = (rng.randn(*shape).astype(np.float32) * 0.01).astype(dt)
    ms = (np.abs(rng.randn(*shape).astype(np.float32)) * 0.1 + 0.01).astype(dt)
    mom = (rng.randn(*shape).astype(np.float32) * 0.01).astype(dt)
    grad = rng.randn(*shape).astype(np.float32).astype(dt)
    hyper = (0.01, 0.9, 0.9, 1e-5)
    hyper_t = tuple(float(np.asarray(h).astype(dt).astype(np.float64)) for h in hyper)
    want = np_ref.apply_centered_rms_prop(var, mg, ms, mom, *hyper_t, grad)
    vs = [Variable(to_torch(a), n) for a, n in zip((var, mg, ms, mom), ("var", "mg", "ms", "mom"))]
    assert raw_ops.ResourceApplyCenteredRMSProp(*vs, *hyper, to_torch(grad)) is None
    rt, at = _tol(dtype)
    for got, w, name in zip(vs, want, ("var", "mg", "ms", "mom")):
        assert_close(to_numpy(got.tensor()), w, rt, at, "%s %s" % (dtype, name))


def test_rms_prop_errors_and_copy_on_write(kernel_lib):
    ok = torch.ones(4, device="cuda")
    with pytest.raises(errors.InvalidArgumentError, match="var and ms must have the same shape"):
        raw_ops.ResourceApplyRMSProp(ok.clone(), torch.ones(5, device="cuda"), ok.clone(),
                                     0.01, 0.9, 0.9, 1e-7, ok)
    with pytest.raises(errors.InvalidArgumentError, match="rho must be a scalar, got 2"):
        raw_ops.ResourceApplyRMSProp(ok.clone(), ok.clone(), ok.clone(), 0.01, [0.9, 0.9], 0.9,
                                     1e-7, ok)
    with pytest.raises(errors.FailedPreconditionError, match="Fused RMSProp variables"):
        raw_ops.ResourceApplyRMSProp(Variable(None), Variable(ok.clone()), Variable(ok.clone()),
                                     0.01, 0.9, 0.9, 1e-7, ok)
    # A reader holding the old value keeps it: the update works on a copy.
    var = Variable(ok.clone(), "var")
    seen = var.value()
    raw_ops.ResourceApplyRMSProp(var, Variable(ok.clone()), Variable(ok.clone()), 0.01, 0.9, 0.9,
                                 1e-7, ok)
    assert torch.equal(seen, ok) and not torch.equal(var.tensor(), ok)


def test_vector_and_element_paths_agree_bit_for_bit(kernel_lib):
    """The same update through 128-bit packs and through an unaligned view."""
    n = 10007
    rng = np.random.default_rng(3)
    base = [rng.standard_normal(n).astype(np.float32) for _ in range(4)]
    base[1] = np.abs(base[1]) * 0.1

    def run(shift):
        ts = []
        for a in base:
            buf = torch.empty(n + 1, device="cuda")
            view = buf[shift:shift + n]
            view.copy_(to_torch(a))
            ts.append(view)
        raw_ops.ResourceApplyRMSProp(ts[0], ts[1], ts[2], 0.01, 0.9, 0.9, 1e-7, ts[3])
        return [to_numpy(t) for t in ts[:3]]

    for a, b in zip(run(0), run(1)):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


# -------------------------------------------------------- gradient descent --

@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("n", [1, 5, 4096, 70001])
def test_gradient_descent_is_exact(kernel_lib, dtype, n):
    """One multiply and one subtract, each rounded once: the CPU restatement is
    reproduced bit for bit."""
    rng = np.random.default_rng(n)
    dt = np_dtype(dtype)
    var = rng.standard_normal(n).astype(dt)
    delta = rng.standard_normal(n).astype(dt)
    want = np_ref.apply_gradient_descent(var, 0.1, delta)
    t = Variable(to_torch(var))
    raw_ops.ResourceApplyGradientDescent(t, 0.1, to_torch(delta))
    got = to_numpy(t.tensor())
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_mixed_gradient_descent(kernel_lib):
    rng = np.random.default_rng(1)
    var = rng.standard_normal(5003).astype(np.float32)
    delta = rng.standard_normal(5003).astype(NP_BF16)
    want = np_ref.apply_gradient_descent(var, 0.05, delta)
    t = to_torch(var)
    raw_ops.MusaResourceApplyGradientDescentMixed(t, 0.05, to_torch(delta))
    assert np.array_equal(to_numpy(t).view(np.uint32), want.view(np.uint32))
    with pytest.raises(errors.InvalidArgumentError, match="float variables"):
        raw_ops.MusaResourceApplyGradientDescentMixed(t.half(), 0.05, to_torch(delta))
    with pytest.raises(errors.InvalidArgumentError, match="same shape"):
        raw_ops.ResourceApplyGradientDescent(t, 0.05, t[:5])
    with pytest.raises(errors.FailedPreconditionError, match="not initialized"):
        raw_ops.ResourceApplyGradientDescent(Variable(None), 0.05, t)


@pytest.mark.parametrize("delta_dtype", ["float32", "bfloat16"])
def test_grouped_gradient_descent(kernel_lib, delta_dtype):
    """300 tensors of ragged sizes (more than one launch's worth of
    descriptors), including empty ones and unaligned views."""
    rng = np.random.default_rng(9)
    sizes = [int(s) for s in rng.integers(0, 6000, 300)]
    sizes[0], sizes[1], sizes[2] = 0, 1, 2049
    vars_np, deltas_np, alphas, vars_t, deltas_t = [], [], [], [], []
    for i, n in enumerate(sizes):
        v = rng.standard_normal(n).astype(np.float32)
        d = rng.standard_normal(n).astype(np_dtype(delta_dtype))
        a = float(np.float32(rng.uniform(0.001, 0.5)))
        vars_np.append(v)
        deltas_np.append(d)
        alphas.append(a)
        if i % 7 == 3 and n > 0:       # a view one element into its buffer
            buf = torch.empty(n + 1, device="cuda")
            buf[1:].copy_(to_torch(v))
            vars_t.append(buf[1:])
        else:
            vars_t.append(to_torch(v))
        deltas_t.append(to_torch(d))
    raw_ops.MusaGroupedResourceApplyGradientDescentMixed(vars_t, alphas, deltas_t)
    for v, d, a, t in zip(vars_np, deltas_np, alphas, vars_t):
        want = np_ref.apply_gradient_descent(v, a, d)
        assert np.array_equal(to_numpy(t).view(np.uint32), want.view(np.uint32))
    with pytest.raises(errors.InvalidArgumentError, match="float variables"):
        raw_ops.MusaGroupedResourceApplyGradientDescentMixed(
            [torch.zeros(3, device="cuda", dtype=torch.float16)], [0.1],
            [torch.zeros(3, device="cuda")])
    with pytest.raises(errors.InvalidArgumentError, match="alpha must be a scalar"):
        raw_ops.MusaGroupedResourceApplyGradientDescentMixed(
            [torch.zeros(3, device="cuda")], [[0.1, 0.2]], [torch.zeros(3, device="cuda")])


@pytest.mark.parametrize("delta_dtype", ["float32", "bfloat16"])
def test_grouped_table_form_matches_host_table_form(kernel_lib, delta_dtype):
    """The reference's five-device-table interface, with its own way of
    assigning CTAs to tensors (ceil(n / 256) capped at 4096 per tensor)."""
    lib = raw_ops._lib()
    rng = np.random.default_rng(11)
    sizes = [5, 256, 257, 100000, 3, 40000]
    dt = torch.float32 if delta_dtype == "float32" else torch.bfloat16
    vars_a = [torch.randn(n, device="cuda") for n in sizes]
    deltas = [torch.randn(n, device="cuda").to(dt) for n in sizes]
    alphas = [float(np.float32(a)) for a in rng.uniform(0.01, 0.3, len(sizes))]
    vars_b = [v.clone() for v in vars_a]
    raw_ops.MusaGroupedResourceApplyGradientDescentMixed(vars_b, alphas, deltas)

    offs = [0]
    for n in sizes:
        offs.append(offs[-1] + min(max((n + 255) // 256, 1), 4096))
    dev = lambda a, t: torch.tensor(a, dtype=t, device="cuda")
    var_ptrs = dev([v.data_ptr() for v in vars_a], torch.int64)
    grad_ptrs = dev([d.data_ptr() for d in deltas], torch.int64)
    al = dev(alphas, torch.float32)
    sz = dev(sizes, torch.int64)
    bo = dev(offs, torch.int64)
    fn = (lib.LaunchGroupedResourceApplyGradientDescentFloat if delta_dtype == "float32"
          else lib.LaunchGroupedResourceApplyGradientDescentFloatBFloat16)
    fn(var_ptrs.data_ptr(), grad_ptrs.data_ptr(), al.data_ptr(), sz.data_ptr(), bo.data_ptr(),
       len(sizes), offs[-1], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for a, b in zip(vars_a, vars_b):
        assert torch.equal(a, b)


def test_full_size_rms_prop_range_sharding_is_bit_identical(kernel_lib):
    """25.6 M parameters (the Adam configuration's size): updating two halves
    separately gives the bits of the whole-vector update."""
    n = 25_557_032
    torch.manual_seed(1)
    var = torch.randn(n, device="cuda") * 0.05
    ms = torch.rand(n, device="cuda") * 1e-4
    mom = torch.randn(n, device="cuda") * 1e-4
    grad = torch.randn(n, device="cuda") * 1e-3
    whole = [t.clone() for t in (var, ms, mom)]
    raw_ops.ResourceApplyRMSProp(*whole, 1e-3, 0.9, 0.9, 1e-7, grad)
    cut = n // 2 + 3                                        # an unaligned cut
    parts = [t.clone() for t in (var, ms, mom)]
    raw_ops.ResourceApplyRMSProp(*[t[:cut] for t in parts], 1e-3, 0.9, 0.9, 1e-7, grad[:cut])
    raw_ops.ResourceApplyRMSProp(*[t[cut:] for t in parts], 1e-3, 0.9, 0.9, 1e-7, grad[cut:])
    for a, b in zip(whole, parts):
        assert torch.equal(a, b)
    # Spot check against the oracle on a slice.
    sl = slice(1_000_000, 1_004_096)
    want = np_ref.apply_rms_prop(to_numpy(var[sl]), to_numpy(ms[sl]), to_numpy(mom[sl]),
                                 float(np.float32(1e-3)), float(np.float32(0.9)),
                                 float(np.float32(0.9)), float(np.float32(1e-7)),
                                 to_numpy(grad[sl]))
    for got, w in zip(whole, want):
        assert_close(to_numpy(got[sl]), w, RTOL["f32_adam"], 1e-9)


# ---------------------------------------------------------------- Adagrad --

def test_adagrad_golden_vectors(golden, kernel_lib):
    g = golden["adagrad_reference_numpy"]
    for name in sorted({k.split("/")[1] for k in g.files}):
        k = "adagrad/" + name
        lr, eps = g[k + "/hyper"]
        var, accum = to_torch(g[k + "/var"]), to_torch(g[k + "/accum"])
        raw_ops.ResourceApplyAdagradV2(var, accum, lr, eps, to_torch(g[k + "/grad"]))
        assert_close(to_numpy(var), g[k + "/var_out"], 2e-6, 1e-7, k)
        assert_close(to_numpy(accum), g[k + "/accum_out"], 3e-7, 1e-8, k)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("update_slots", [True, False])
@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_adagrad_matches_oracle(kernel_lib, dtype, update_slots, n):
    rng = np.random.default_rng(n)
    dt = np_dtype(dtype)
    var = rng.random(n).astype(dt)
    accum = (rng.random(n) + 0.01).astype(dt)
    grad = (rng.random(n) * 0.1).astype(dt)
    lr, eps = (float(np.asarray(h).astype(dt).astype(np.float64)) for h in (0.01, 1e-7))
    want = np_ref.apply_adagrad_v2(var, accum, lr, eps, grad, update_slots)
    tv, ta = Variable(to_torch(var), "var"), Variable(to_torch(accum), "accum")
    assert raw_ops.ResourceApplyAdagradV2(tv, ta, 0.01, 1e-7, to_torch(grad),
                                          update_slots=update_slots) is None
    rt, at = _tol(dtype)
    assert_close(to_numpy(tv.tensor()), want[0], rt, at, "var")
    assert_close(to_numpy(ta.tensor()), want[1], rt, at, "accum")
    if not update_slots:
        assert np.array_equal(to_numpy(ta.tensor()).view(np.uint8), accum.view(np.uint8))


def test_adagrad_errors_and_ref_variable_form(kernel_lib):
    ok = torch.ones(4, device="cuda")
    with pytest.raises(errors.FailedPreconditionError, match="Fused AdagradV2 variables"):
        raw_ops.ResourceApplyAdagradV2(Variable(None), Variable(ok.clone()), 0.1, 1e-7, ok)
    with pytest.raises(errors.InvalidArgumentError, match="var and accum must have the same shape"):
        raw_ops.ResourceApplyAdagradV2(ok.clone(), torch.ones(5, device="cuda"), 0.1, 1e-7, ok)
    with pytest.raises(errors.InvalidArgumentError, match="epsilon must be a scalar"):
        raw_ops.ResourceApplyAdagradV2(ok.clone(), ok.clone(), 0.1, [1e-7, 1e-7], ok)
    var = ok.clone()
    out = raw_ops.ApplyAdagradV2(var, ok.clone(), 0.1, 0.0, ok, use_locking=True)
    assert out.data_ptr() == var.data_ptr()
    assert_close(to_numpy(var), np.full(4, 1 - 0.1 / np.sqrt(2.0)), 1e-6)
