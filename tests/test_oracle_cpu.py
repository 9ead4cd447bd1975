"""The CPU oracle against the committed golden vectors, and the C restatement
against the NumPy one.  No GPU."""
import numpy as np
import pytest

from oracle import c_ref, np_ref
from helpers import NP_BF16, RTOL, assert_close


@pytest.mark.parametrize("case", ["step10", "first_step_guard", "step1"])
def test_adam_matches_reference_numpy_statement(golden, case):
    g = golden["adam_reference_numpy"]
    s = g[case + "/scalars"]
    var, m, v = np_ref.apply_adam(g[case + "/var"], g[case + "/m"], g[case + "/v"],
                                  s[0], s[1], s[2], s[3], s[4], s[5], g[case + "/grad"])
    assert_close(m, g[case + "/expected_m"], 1e-7, what="m")
    assert_close(v, g[case + "/expected_v"], 1e-7, what="v")
    assert_close(var, g[case + "/expected_var"], 1e-6, what="var")


@pytest.mark.parametrize("case", ["step10", "first_step_guard", "step1"])
def test_adam_double_op_chain_matches_reference_numpy_statement(golden, case):
    """The float64 restatement of the reference's op chain (T = double) against
    the reference's own NumPy statement of the update: the same inputs widened
    to double agree with its float32 answers to float32 rounding."""
    g = golden["adam_reference_numpy"]
    s = [float(x) for x in g[case + "/scalars"]]
    var, m, v = np_ref.apply_adam_op_chain(g[case + "/var"], g[case + "/m"], g[case + "/v"],
                                           s[0], s[1], s[2], s[3], s[4], s[5],
                                           g[case + "/grad"])
    assert var.dtype == np.float64
    # (absolute floors: the float32 roundings of the golden's own terms)
    assert_close(m, g[case + "/expected_m"], 2e-7, 1e-10, what="m")
    assert_close(v, g[case + "/expected_v"], 2e-7, 1e-14, what="v")
    assert_close(var, g[case + "/expected_var"], 1e-6, 1e-8, what="var")
    # Nesterov numerator: m * beta1 + g * (1 - beta1) (TensorFlow's CPU kernel).
    nv, nm, _ = np_ref.apply_adam_op_chain(g[case + "/var"], g[case + "/m"], g[case + "/v"],
                                           s[0], s[1], s[2], s[3], s[4], s[5],
                                           g[case + "/grad"], use_nesterov=True)
    assert np.array_equal(nm, m) and not np.array_equal(nv, var)


def test_adam_first_step_guard_uses_lr():
    assert np_ref.adam_alpha(1e-3, 1.0, 1.0) == np.float32(1e-3)
    a = np_ref.adam_alpha(1e-3, 0.9, 0.999)
    assert abs(float(a) - 1e-3 * np.sqrt(1 - 0.999) / 0.1) < 1e-9


def test_adam_c_matches_numpy():
    rng = np.random.default_rng(5)
    n = 10007
    var = rng.normal(0, 0.05, n).astype(np.float32)
    m = rng.normal(0, 1e-4, n).astype(np.float32)
    v = rng.uniform(0, 1e-6, n).astype(np.float32)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    ev, em, evv = np_ref.apply_adam(var, m, v, 0.9 ** 10, 0.999 ** 10, 1e-3, 0.9,
                                    0.999, 1e-7, g)
    alpha = np_ref.adam_alpha(1e-3, np.float32(0.9 ** 10), np.float32(0.999 ** 10))
    c_ref.adam_f32(var, m, v, g, 0.9, 0.999, 1e-7, alpha)
    assert_close(m, em, 0, what="m")
    assert_close(v, evv, 0, what="v")
    assert_close(var, ev, 1e-6, what="var")


def _bn_names(g):
    return sorted({k.split("/")[0] for k in g.files})


def test_bn_oracle_matches_independent_implementation(golden):
    g = golden["bn_torch_cpu"]
    for n in _bn_names(g):
        fmt = str(g[n + "/format"])
        out = np_ref.fused_batch_norm(g[n + "/x"], g[n + "/scale"], g[n + "/offset"],
                                      epsilon=1e-3, data_format=fmt)
        scale_y = np.abs(g[n + "/y"]).max()
        assert_close(out[0], g[n + "/y"], 1e-5, 1e-5 * scale_y, n + " y")
        assert_close(out[1], g[n + "/mean"], 1e-6, 1e-7, n + " batch_mean")
        assert_close(out[2], g[n + "/var_unbiased"], 1e-6, 0, n + " batch_var")
        assert_close(out[3], g[n + "/mean"], 1e-6, 1e-7, n + " reserve_1")
        assert_close(out[4], g[n + "/var_pop"], 1e-6, 0, n + " reserve_2")
        assert out[5].shape == () and out[5] == 0
        gr = np_ref.fused_batch_norm_grad(g[n + "/dy"], g[n + "/x"], g[n + "/scale"],
                                          out[3], out[4], 1e-3, fmt)
        s = np.abs(g[n + "/dx"]).max()
        assert_close(gr[0], g[n + "/dx"], 1e-4, 1e-5 * s, n + " dx")
        s = np.abs(g[n + "/dscale"]).max()
        assert_close(gr[1], g[n + "/dscale"], 1e-4, 1e-4 * s, n + " dscale")
        assert_close(gr[2], g[n + "/doffset"], 1e-5, 1e-6, n + " doffset")
        assert gr[3].shape == gr[1].shape and not gr[3].any() and not gr[4].any()


def test_bn_single_value_per_channel_skips_bessel():
    x = np.array([[[[1.0, 2.0, 3.0]]]], np.float32)
    out = np_ref.fused_batch_norm(x, np.ones(3, np.float32), np.zeros(3, np.float32))
    assert np.all(out[2] == 0) and np.all(out[4] == 0)
    assert np.all(np.isfinite(out[0]))


def test_bn_exponential_avg_factor_blends():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((4, 3, 3, 5)).astype(np.float32)
    s, o = np.ones(5, np.float32), np.zeros(5, np.float32)
    rm, rv = np.full(5, 2.0, np.float32), np.full(5, 3.0, np.float32)
    full = np_ref.fused_batch_norm(x, s, o)
    half = np_ref.fused_batch_norm(x, s, o, rm, rv, exponential_avg_factor=0.5)
    assert_close(half[1], 0.5 * rm + 0.5 * full[1], 1e-6)
    assert_close(half[2], 0.5 * rv + 0.5 * full[2], 1e-6)
    assert_close(half[3], full[3], 0)


def test_bn_inference_uses_given_statistics():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 3, 4)).astype(np.float32)
    s = rng.uniform(0.5, 1.5, 4).astype(np.float32)
    o = rng.normal(0, 0.1, 4).astype(np.float32)
    mean = rng.normal(0, 1, 4).astype(np.float32)
    var = rng.uniform(0.5, 2, 4).astype(np.float32)
    y = np_ref.fused_batch_norm(x, s, o, mean, var, is_training=False)[0]
    assert_close(y, (x - mean) / np.sqrt(var + 1e-3) * s + o, 1e-5, 1e-6)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    dx = np_ref.fused_batch_norm_grad(dy, x, s, mean, var, is_training=False)[0]
    assert_close(dx, dy * s / np.sqrt(var + 1e-3), 1e-5, 1e-7)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_bn_c_matches_numpy(dtype):
    rng = np.random.default_rng(7)
    dt = {"float32": np.float32, "float16": np.float16, "bfloat16": NP_BF16}[dtype]
    x = (rng.standard_normal((3000, 24)) * 3 + 1).astype(dt)
    dy = (rng.standard_normal((3000, 24)) * 1e-2).astype(dt)
    s = rng.uniform(0.5, 1.5, 24).astype(np.float32)
    o = rng.normal(0, 0.1, 24).astype(np.float32)
    rt = RTOL["f32_bn"] if dtype == "float32" else RTOL["lowp"]
    c = c_ref.bn_fwd_train(x, s, o, 1e-3)
    e = np_ref.fused_batch_norm(x, s, o, epsilon=1e-3)
    assert_close(c[0], e[0], rt, rt, "y")
    for i in range(1, 5):
        assert_close(c[i], e[i], 1e-5, 1e-6, "stat %d" % i)
    cg = c_ref.bn_grad(dy, x, s, e[3], e[4], 1e-3)
    eg = np_ref.fused_batch_norm_grad(dy, x, s, e[3], e[4], 1e-3)
    assert_close(cg[0], eg[0], rt, rt * np.abs(eg[0].astype(np.float64)).max(), "dx")
    assert_close(cg[1], eg[1], 1e-4, 1e-5, "dscale")
    assert_close(cg[2], eg[2], 1e-4, 1e-6, "doffset")


def test_elementwise_literals(golden):
    g = golden["elementwise_literals"]
    assert_close(np_ref.relu(g["relu/in"]), g["relu/out"], 0)
    assert_close(np_ref.sigmoid(g["sigmoid/in"]), g["sigmoid/out"], 1e-6, 1e-45)
    assert_close(np_ref.bias_add(g["biasadd/x"], g["biasadd/b"]), g["biasadd/out_nhwc"], 0)
    assert_close(np_ref.bias_add(g["biasadd/x_nchw"], g["biasadd/b_nchw"], "NCHW"),
                 g["biasadd/out_nchw"], 0)
    out = np_ref.bias_add(g["biasadd/x_i32"], g["biasadd/b_i32"])
    assert out.dtype == np.int32 and np.array_equal(out, g["biasadd/out_i32"])


def test_bias_add_edge_cases():
    with pytest.raises(ValueError, match="Dimension mismatch in BiasAdd"):
        np_ref.bias_add(np.zeros((2, 3), np.float32), np.zeros(4, np.float32))
    assert np_ref.bias_add(np.zeros((0, 3), np.float32), np.zeros(3, np.float32)).shape == (0, 3)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("act,fn", [(0, np_ref.bias_add), (1, np_ref.bias_add_relu),
                                    (2, np_ref.bias_add_swish),
                                    (3, np_ref.bias_add_sigmoid)])
def test_bias_act_c_matches_numpy(dtype, act, fn):
    rng = np.random.default_rng(9)
    dt = {"float32": np.float32, "float16": np.float16, "bfloat16": NP_BF16}[dtype]
    x = rng.standard_normal((257, 40)).astype(dt)
    b = rng.normal(0, 0.1, 40).astype(dt)
    rt = 1e-6 if dtype == "float32" else 0.0
    assert_close(c_ref.bias_act(x, b, act), fn(x, b), rt, 0, "act %d" % act)


def _bias_grad_cases(g):
    for name, fmt in (("nhwc", "NHWC"), ("nchw", "NCHW"), ("ragged2d", "NHWC")):
        for dt in ("f32", "f16", "bf16"):
            yield "%s/%s" % (name, dt), fmt, {"f32": "float32", "f16": "float16",
                                              "bf16": "bfloat16"}[dt]


def test_bias_grad_oracle_matches_independent_implementation(golden):
    """ReluGrad / BiasAddGrad of the oracle against PyTorch's CPU autograd of
    relu(x + b) at the shapes of the reference's BiasAddGrad test."""
    from helpers import np_dtype
    g = golden["bias_grad_torch_cpu"]
    for key, fmt, dtype in _bias_grad_cases(g):
        dt = np_dtype(dtype)
        feats = g[key + "/features"].astype(dt)
        grads = g[key + "/gradients"].astype(dt)
        dx, db = np_ref.bias_add_relu_grad(grads, feats, fmt)
        assert dx.dtype == dt and db.dtype == dt
        # backprops is a selection of the gradients: exact in every type.
        assert np.array_equal(dx.astype(np.float64), g[key + "/backprops"].astype(np.float64)), key
        assert np.array_equal(db.astype(np.float64),
                              g[key + "/bias_grad"].astype(dt).astype(np.float64)), key
        plain = np_ref.bias_add_grad(grads, fmt)
        assert np.array_equal(plain.astype(np.float64),
                              g[key + "/dy_colsum"].astype(dt).astype(np.float64)), key


def test_bias_grad_oracle_edge_cases():
    # 1-D input: nothing to reduce, the input is the result
    # (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:52-58).
    v = np.array([1.5, -2.0, 3.0], np.float32)
    assert np.array_equal(np_ref.bias_add_grad(v), v)
    # Empty inputs give zeros of the channel count (test/ops/biasadd_grad_op_test.py:88-127).
    for shape in [(4096, 0, 512), (4096, 0, 128), (0, 16)]:
        out = np_ref.bias_add_grad(np.zeros(shape, np.float16))
        assert out.shape == (shape[-1],) and out.dtype == np.float16 and not out.any()
    # Integer sums wrap in the tensor's own width.
    big = np.full((4, 2), 2 ** 30, np.int32)
    assert np.array_equal(np_ref.bias_add_grad(big), np.array([0, 0], np.int32))
    # features == 0 is inactive; a NaN feature is inactive as well.
    gr = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    ft = np.array([0.0, -0.0, np.nan, 1e-30], np.float32)
    assert np.array_equal(np_ref.relu_grad(gr, ft), np.array([0, 0, 0, 4], np.float32))
    with pytest.raises(ValueError):
        np_ref.relu_grad(np.zeros((2, 3), np.float32), np.zeros((3, 2), np.float32))


# ------------------------------------------- Nadam, RMSProp, gradient descent --

def _states(g, key, names):
    return [g["%s/%s" % (key, n)] for n in names]


def test_optimizer_oracle_matches_float64_statements(golden):
    """fp32 restatements against the float64 evaluation of the formulas at the
    reference tests' inputs: the difference is fp32 rounding only."""
    g = golden["optimizer_cases"]
    for case in ("basic", "small", "half"):
        key = "nadam/" + case
        var, m, v, grad = _states(g, key, ("var", "m", "v", "grad"))
        got = np_ref.apply_nadam(var, m, v, *g[key + "/hyper"], grad)
        for out, name in zip(got, ("var_out", "m_out", "v_out")):
            np.testing.assert_allclose(out, g[key + "/" + name], rtol=2e-6, atol=1e-7)
    for case in ("basic", "dtypes", "zero_grad", "negative_grad"):
        key = "rmsprop/" + case
        var, ms, mom, grad = _states(g, key, ("var", "ms", "mom", "grad"))
        got = np_ref.apply_rms_prop(var, ms, mom, *g[key + "/hyper"], grad)
        for out, name in zip(got, ("var_out", "ms_out", "mom_out")):
            np.testing.assert_allclose(out, g[key + "/" + name], rtol=2e-6, atol=1e-7)
    for case in ("basic", "dtypes"):
        key = "centered_rmsprop/" + case
        var, mg, ms, mom, grad = _states(g, key, ("var", "mg", "ms", "mom", "grad"))
        got = np_ref.apply_centered_rms_prop(var, mg, ms, mom, *g[key + "/hyper"], grad)
        for out, name in zip(got, ("var_out", "mg_out", "ms_out", "mom_out")):
            np.testing.assert_allclose(out, g[key + "/" + name], rtol=2e-6, atol=1e-7)
    for case in ("vector", "matrix", "locking"):
        key = "sgd/" + case
        got = np_ref.apply_gradient_descent(g[key + "/var"], float(g[key + "/alpha"]),
                                            g[key + "/grad"])
        np.testing.assert_allclose(got, g[key + "/var_out"], rtol=2e-7, atol=1e-7)


def test_optimizer_oracle_low_precision_and_double():
    from helpers import NP_BF16
    rng = np.random.default_rng(4)
    var = rng.standard_normal(64)
    ms = np.abs(rng.standard_normal(64)) * 0.1
    mom = rng.standard_normal(64) * 0.01
    grad = rng.standard_normal(64)
    want = np_ref.apply_rms_prop(*(a.astype(np.float64) for a in (var, ms, mom)),
                                 0.01, 0.9, 0.9, 1e-7, grad.astype(np.float64))
    for dt, tol in ((np.float16, 2e-3), (NP_BF16, 2e-2)):
        got = np_ref.apply_rms_prop(*(a.astype(dt) for a in (var, ms, mom)),
                                    0.01, 0.9, 0.9, 1e-7, grad.astype(dt))
        for a, b in zip(got, want):
            assert a.dtype == dt
            np.testing.assert_allclose(a.astype(np.float64), b, rtol=tol * 4, atol=tol)
    # 16-bit gradient descent rounds the product before the subtraction.
    v16 = np.array([1.0], np.float16)
    d16 = np.array([0.3333], np.float16)
    step = np.float16(np.float16(0.1).astype(np.float32) * d16.astype(np.float32))
    assert np_ref.apply_gradient_descent(v16, 0.1, d16)[0] == np.float16(
        np.float32(1.0) - np.float32(step[0]))


# ------------------------------------------------------ LayerNorm, RMSNorm --

ROW_NORM_SHAPES = ["s16x32", "s8x16x32", "s32x128", "s2x4x8x16", "s100x1", "s100x2", "s1x1",
                   "s2x8192", "s7x1000"]


def test_row_norm_oracle_matches_independent_implementation(golden):
    """LayerNorm / RMSNorm restatements against PyTorch's CPU layer_norm /
    rms_norm (float64) and its autograd."""
    g = golden["row_norm_torch_cpu"]
    for name in ROW_NORM_SHAPES:
        k = "layer_norm/" + name
        x, dy, gamma, beta = (g[k + "/" + n] for n in ("x", "dy", "gamma", "beta"))
        x64, dy64 = x.astype(np.float64), dy.astype(np.float64)
        np.testing.assert_allclose(np_ref.layer_norm(x64, gamma, beta), g[k + "/y"],
                                   rtol=1e-9, atol=1e-9)
        dx, dgamma, dbeta = np_ref.layer_norm_grad(dy64, x64, gamma)
        np.testing.assert_allclose(dx, g[k + "/dx"], rtol=1e-8, atol=1e-9)
        np.testing.assert_allclose(dgamma, g[k + "/dgamma"], rtol=1e-9, atol=1e-9)
        np.testing.assert_allclose(dbeta, g[k + "/dbeta"], rtol=1e-9, atol=1e-9)
        r = "rms_norm/" + name
        y, normalized, inv = np_ref.rms_norm(x64, gamma)
        np.testing.assert_allclose(y, g[r + "/y"], rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(normalized, g[r + "/normalized"], rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(inv, g[r + "/inv_rms"], rtol=1e-12)
        np.testing.assert_allclose(np_ref.rms_norm_grad_dx(x64, inv, gamma, dy64),
                                   g[r + "/dx"], rtol=1e-8, atol=1e-10)
        assert np_ref.layer_norm(x, gamma, beta).dtype == np.float32


def test_adagrad_oracle_matches_reference_numpy_statement(golden):
    """AdagradV2 restatement against the reference test's own NumPy helper
    (evaluated in float64 when the vectors were made)."""
    g = golden["adagrad_reference_numpy"]
    names = sorted({k.split("/")[1] for k in g.files})
    assert "vector" in names and "matrix" in names and len(names) == 5
    for name in names:
        k = "adagrad/" + name
        lr, eps = g[k + "/hyper"]
        var, accum = np_ref.apply_adagrad_v2(g[k + "/var"], g[k + "/accum"], lr, eps,
                                             g[k + "/grad"])
        np.testing.assert_allclose(var, g[k + "/var_out"], rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(accum, g[k + "/accum_out"], rtol=2e-7, atol=1e-8)
        v64, a64 = np_ref.apply_adagrad_v2(*(g[k + "/" + n].astype(np.float64)
                                             for n in ("var", "accum")), lr, eps,
                                           g[k + "/grad"].astype(np.float64))
        np.testing.assert_allclose(v64, g[k + "/var_out"], rtol=1e-13)
        np.testing.assert_allclose(a64, g[k + "/accum_out"], rtol=1e-13)
    # without update_slots the accumulator stays and is used as it is
    v = np.array([1.0, 2.0], np.float32)
    a = np.array([4.0, 9.0], np.float32)
    gr = np.array([1.0, 1.0], np.float32)
    nv, na = np_ref.apply_adagrad_v2(v, a, 0.5, 0.0, gr, update_slots=False)
    assert np.array_equal(na, a) and np.allclose(nv, [1 - 0.25, 2 - 0.5 / 3])
