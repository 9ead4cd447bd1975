"""CPU oracle (NumPy) for the BatchNorm / ApplyAdam / BiasAdd+activation path.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the results that
TensorFlow's CPU kernels give for the ops of this path, following the
conventions that the reference plugin documents and tests against.  It is
imported by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark; the product (the CUDA library and its Python front end) never
imports it.

Pinning status.  The stated target oracle is TensorFlow 2.6.1's CPU kernels.
TensorFlow is not installable next to this code (no wheel for the interpreter,
no network), and the reference's own arithmetic for BatchNorm / BiasAdd / Relu /
Sigmoid sits in a closed vendor library, so:
  * ApplyAdam is pinned to the reference's own NumPy restatement of the update
    rule (test/ops/musa_resource_sparse_apply_adam_op_test.py:35-69), run from
    the reference file by tests/golden/make_golden.py, and to the in-repo
    device kernels it mirrors line by line;
  * Relu / Sigmoid / BiasAdd are pinned to the literal cases of the reference
    tests (test/ops/relu_op_test.py:58-96, test/ops/sigmoid_op_test.py:58-93,
    test/ops/biasadd_op_test.py:74-116) whose answers are closed-form;
  * FusedBatchNorm forward/gradient: PARITY UNPINNED against TensorFlow itself.
    The restatement follows the output conventions the reference documents
    (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:126-170, 265-277) and is
    cross-checked against an independent implementation (PyTorch's CPU
    batch_norm and its autograd) in tests/golden/make_golden.py.

Every function accumulates in float64 and rounds once to the output dtype,
except where the op's own arithmetic type matters (Adam: float32 throughout;
16-bit element-wise chains: one rounding per un-fused op).
"""
import numpy as np

try:  # bfloat16 as a NumPy dtype
    import ml_dtypes

    bfloat16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    bfloat16 = None


# --------------------------------------------------------------------------
# FusedBatchNorm{,V2,V3}
# --------------------------------------------------------------------------

def _channel_axis(ndim, data_format):
    if data_format == "NHWC":
        return ndim - 1
    if data_format == "NCHW":
        return 1
    raise ValueError("data_format must be NHWC or NCHW, got %r" % (data_format,))


def fused_batch_norm(x, scale, offset, mean=None, variance=None, epsilon=1e-3,
                     exponential_avg_factor=1.0, data_format="NHWC",
                     is_training=True):
    """FusedBatchNormV3 forward.

    Returns (y, batch_mean, batch_var, reserve_space_1, reserve_space_2,
    reserve_space_3) with the conventions of
    musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:
      :141-150  batch_var is the Bessel-corrected (1/(R-1)) variance,
      :158-170  reserve_space_2 is the population (1/R) variance and the
                correction is skipped when there is one value per channel,
      :59-62    reserve_space_3 is a zero-filled 0-D tensor,
      :173-178  inference uses the given mean/variance.
    With exponential_avg_factor != 1 the first two statistics outputs are
    blended with the incoming running values, as TensorFlow's CPU kernel does.
    """
    x = np.asarray(x)
    out_dtype = x.dtype
    ax = _channel_axis(x.ndim, data_format)
    red = tuple(i for i in range(x.ndim) if i != ax)
    shape = [1] * x.ndim
    shape[ax] = x.shape[ax]
    x64 = x.astype(np.float64)
    scale64 = np.asarray(scale, np.float64).reshape(shape)
    offset64 = np.asarray(offset, np.float64).reshape(shape)
    eps = float(np.float32(epsilon))
    if is_training:
        count = x64.size // max(x.shape[ax], 1)
        mu = x64.mean(axis=red)
        var = ((x64 - mu.reshape(shape)) ** 2).mean(axis=red)
        unbiased = var * (count / (count - 1.0)) if count > 1 else var
        f = float(np.float32(exponential_avg_factor))
        if f == 1.0:
            bm, bv = mu, unbiased
        else:
            bm = (1.0 - f) * np.asarray(mean, np.float64) + f * mu
            bv = (1.0 - f) * np.asarray(variance, np.float64) + f * unbiased
        # The normalisation uses the float32 statistics that the op emits.
        mu32 = mu.astype(np.float32).astype(np.float64)
        var32 = var.astype(np.float32).astype(np.float64)
        inv = 1.0 / np.sqrt(var32 + eps)
        y = (x64 - mu32.reshape(shape)) * (inv.reshape(shape) * scale64) + offset64
        return (y.astype(out_dtype), bm.astype(np.float32), bv.astype(np.float32),
                mu.astype(np.float32), var.astype(np.float32),
                np.zeros((), np.float32))
    mu = np.asarray(mean, np.float64)
    var = np.asarray(variance, np.float64)
    inv = 1.0 / np.sqrt(var + eps)
    y = (x64 - mu.reshape(shape)) * (inv.reshape(shape) * scale64) + offset64
    return (y.astype(out_dtype), mu.astype(np.float32), var.astype(np.float32),
            mu.astype(np.float32), var.astype(np.float32), np.zeros((), np.float32))


def fused_batch_norm_grad(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                          epsilon=1e-3, data_format="NHWC", is_training=True):
    """FusedBatchNormGradV3.

    reserve_space_1 is the batch mean and reserve_space_2 the POPULATION
    variance; the op converts the latter with rsqrt(var + eps)
    (musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:265-277,
    musa_ext/kernels/nn/musa_fused_batchnorm_kernel.mu:23-29).
    Returns (dx, dscale, doffset, out3, out4); the last two are the zero-filled
    [C] placeholders that the reference emits (:220-242).
    """
    dy = np.asarray(y_backprop)
    x = np.asarray(x)
    ax = _channel_axis(x.ndim, data_format)
    red = tuple(i for i in range(x.ndim) if i != ax)
    shape = [1] * x.ndim
    shape[ax] = x.shape[ax]
    c = x.shape[ax]
    count = x.size // max(c, 1)
    dy64 = dy.astype(np.float64)
    x64 = x.astype(np.float64)
    mu = np.asarray(reserve_space_1, np.float64).reshape(shape)
    var = np.asarray(reserve_space_2, np.float64).reshape(shape)
    s = np.asarray(scale, np.float64).reshape(shape)
    inv = 1.0 / np.sqrt(var + float(np.float32(epsilon)))
    xc = x64 - mu
    doffset = dy64.sum(axis=red)
    dscale = (dy64 * xc).sum(axis=red) * inv.reshape(-1)
    if is_training:
        dx = s * inv * (dy64 - doffset.reshape(shape) / count
                        - xc * inv * dscale.reshape(shape) / count)
    else:
        dx = dy64 * s * inv
    zeros = np.zeros((c,), np.float32)
    return (dx.astype(x.dtype), dscale.astype(np.float32),
            doffset.astype(np.float32), zeros, zeros.copy())


# --------------------------------------------------------------------------
# ApplyAdam / ResourceApplyAdam / MusaResourceApplyAdamMixed
# --------------------------------------------------------------------------

def adam_alpha(lr, beta1_power, beta2_power):
    """Bias-corrected step size, computed in float64 then narrowed, including
    the reference-only first-step guard
    (musa_ext/kernels/training/musa_applyadam_op.cc:236-246)."""
    one_minus = 1.0 - float(beta1_power)
    if abs(one_minus) < 1e-10:
        return np.float32(lr)
    return np.float32(float(lr) * np.sqrt(1.0 - float(beta2_power)) / one_minus)


def adam_alpha64(lr, beta1_power, beta2_power):
    """The same step size kept in float64 (T = double: `static_cast<T>(alpha_val)`,
    musa_ext/kernels/training/musa_applyadam_op.cc:317)."""
    one_minus = 1.0 - float(beta1_power)
    if abs(one_minus) < 1e-10:
        return np.float64(lr)
    return np.float64(float(lr) * np.sqrt(1.0 - float(beta2_power)) / one_minus)


def apply_adam(var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon,
               grad, use_nesterov=False):
    """One Adam step.  State arrays of float32, float16 or bfloat16; grad of
    any of those.  float32 arithmetic in the order of the device kernels
    (musa_ext/kernels/training/musa_apply_sparse_adam_kernel.mu:150-156,
    musa_ext/kernels/training/musa_applyadam_bf16_kernel.mu:92-111), one
    round-to-nearest-even on store.  Returns new (var, m, v); inputs are not
    modified."""
    dt = np.asarray(var).dtype
    f32 = np.float32
    alpha = adam_alpha(f32(lr), f32(beta1_power), f32(beta2_power))
    b1, b2, eps = f32(beta1), f32(beta2), f32(epsilon)
    omb1, omb2 = f32(1.0) - b1, f32(1.0) - b2
    g = np.asarray(grad).astype(f32)
    m32 = np.asarray(m).astype(f32)
    v32 = np.asarray(v).astype(f32)
    var32 = np.asarray(var).astype(f32)
    m_new = b1 * m32 + omb1 * g
    v_new = b2 * v32 + omb2 * g * g
    numer = (b1 * m_new + omb1 * g) if use_nesterov else m_new
    var_new = var32 - alpha * numer / (np.sqrt(v_new) + eps)
    return var_new.astype(dt), m_new.astype(dt), v_new.astype(dt)


def apply_adam_op_chain(var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon,
                        grad, use_nesterov=False):
    """One Adam step for float64 tensors the way the reference serves that
    dtype: a chain of element-wise ops that each store a tensor of type T
    (musa_ext/kernels/training/musa_applyadam_op.cc:297-415): MUL, MUL, ADD for
    m; MUL, MUL, MUL, ADD for v; SQRT, ADD epsilon, DIV, MUL alpha, SUB.  NumPy
    rounds every one of these float64 operations once, as the chain does.  The
    scalars are read as T, alpha comes from `adam_alpha` in float64 (:236-246),
    1 - beta is formed in T (:309-314).  With use_nesterov the numerator is
    TensorFlow's m * beta1 + g * (1 - beta1) (the chain ignores the attr).
    Returns new (var, m, v)."""
    f64 = np.float64
    var = np.asarray(var, f64)
    m = np.asarray(m, f64)
    v = np.asarray(v, f64)
    g = np.asarray(grad, f64)
    b1, b2, eps = f64(beta1), f64(beta2), f64(epsilon)
    alpha = adam_alpha64(f64(lr), f64(beta1_power), f64(beta2_power))
    omb1, omb2 = f64(1.0) - b1, f64(1.0) - b2
    m_new = m * b1 + g * omb1
    v_new = v * b2 + (g * g) * omb2
    numer = (m_new * b1 + g * omb1) if use_nesterov else m_new
    var_new = var - (numer / (np.sqrt(v_new) + eps)) * alpha
    return var_new, m_new, v_new


# --------------------------------------------------------------------------
# BiasAdd, Relu, Sigmoid and the fused chains
# --------------------------------------------------------------------------

def _compute_dtype(dt):
    # TensorFlow's CPU functors for half/bfloat16 widen to float per op.
    if dt == np.float16 or (bfloat16 is not None and dt == bfloat16):
        return np.float32
    return dt


def bias_add(x, bias, data_format="NHWC"):
    """BiasAdd: bias along the last axis (NHWC / 2-D) or axis 1 (NCHW)
    (musa_ext/kernels/nn/musa_biasadd_op.cc:33-57); the add is done in the
    tensor's own type."""
    x = np.asarray(x)
    bias = np.asarray(bias)
    ax = 1 if data_format == "NCHW" else x.ndim - 1
    if x.size and bias.size and bias.shape[0] != x.shape[ax]:
        raise ValueError("Dimension mismatch in BiasAdd")
    if x.size == 0 or bias.size == 0:
        return np.empty(x.shape, x.dtype)
    shape = [1] * x.ndim
    shape[ax] = x.shape[ax]
    ct = _compute_dtype(x.dtype)
    return (x.astype(ct) + bias.astype(ct).reshape(shape)).astype(x.dtype)


def relu(x):
    """Relu: max(x, 0) (musa_ext/kernels/nn/musa_relu_op.cc:19-57)."""
    x = np.asarray(x)
    return np.maximum(x, np.zeros((), x.dtype)).astype(x.dtype)


def sigmoid(x):
    """Sigmoid: 1 / (1 + exp(-x)) (musa_ext/kernels/nn/musa_sigmoid_op.cc:18-35);
    float64 evaluation, one rounding."""
    x = np.asarray(x)
    x64 = x.astype(np.float64)
    with np.errstate(over="ignore"):
        return (1.0 / (1.0 + np.exp(-x64))).astype(x.dtype)


def bias_add_relu(x, bias, data_format="NHWC"):
    """The un-fused chain Relu(BiasAdd(x, b))."""
    return relu(bias_add(x, bias, data_format))


def bias_add_swish(x, bias, data_format="NHWC"):
    """The un-fused chain Mul(x, Sigmoid(BiasAdd(x, b))), each op rounding to
    the tensor's type as separate TensorFlow ops do."""
    x = np.asarray(x)
    ct = _compute_dtype(x.dtype)
    s = sigmoid(bias_add(x, bias, data_format))
    return (x.astype(ct) * s.astype(ct)).astype(x.dtype)


def bias_add_sigmoid(x, bias, data_format="NHWC"):
    """The un-fused chain Sigmoid(BiasAdd(x, b))."""
    return sigmoid(bias_add(x, bias, data_format))


def bias_add_grad(out_backprop, data_format="NHWC"):
    """BiasAddGrad: the sum of `out_backprop` over every axis but the channel
    axis (last for NHWC, 1 for NCHW), returned in the tensor's type.  A 1-D
    input is its own result; an input with no elements gives zeros
    (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:23-70).  Floating types are
    added in fp64 and rounded once; integer types wrap in their own width."""
    g = np.asarray(out_backprop)
    if g.ndim < 1:
        raise ValueError("Input tensor must be at least 1D")
    if g.ndim == 1:
        return g.copy()
    ax = 1 if data_format == "NCHW" else g.ndim - 1
    axes = tuple(i for i in range(g.ndim) if i != ax)
    if np.issubdtype(g.dtype, np.integer):
        return g.sum(axis=axes, dtype=g.dtype)
    return g.astype(np.float64).sum(axis=axes).astype(g.dtype)


def relu_grad(gradients, features):
    """ReluGrad: gradients * (features > 0)
    (musa_ext/kernels/nn/musa_relu_grad_op.cc:19-48)."""
    g = np.asarray(gradients)
    f = np.asarray(features)
    if g.shape != f.shape:
        raise ValueError("Inputs to ReluGrad must have the same shape")
    ct = _compute_dtype(g.dtype)
    with np.errstate(invalid="ignore"):
        mask = (f.astype(ct) > 0).astype(ct)
        return (g.astype(ct) * mask).astype(g.dtype)


def bias_add_relu_grad(gradients, features, data_format="NHWC"):
    """The un-fused pair: backprops = ReluGrad(gradients, features) and
    bias_grad = BiasAddGrad(backprops)."""
    dx = relu_grad(gradients, features)
    return dx, bias_add_grad(dx, data_format)


# --------------------------------------------------------------------------
# Nadam, RMSProp, gradient descent
# --------------------------------------------------------------------------

def _update_dtype(dt):
    """Arithmetic type of the optimizer kernels: fp32 for float and the
    16-bit types, fp64 for double."""
    return np.float64 if dt == np.float64 else np.float32


def apply_nadam(var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon,
                grad):
    """ResourceApplyNadam as the reference states it
    (musa_ext/kernels/training/musa_resource_apply_nadam_kernel.mu:64-76 and the
    formula in test/ops/resource_apply_nadam_op_test.py:57-67):
      m' = b1*m + (1-b1)*g;  v' = b2*v + (1-b2)*g^2
      var' = var - lr * ((b1*m' + (1-b1)*g) / (1-b1^t)) / (sqrt(v' / (1-b2^t)) + eps)
    The scalars are narrowed to float and 1-x is taken in float, as the
    launcher does; the state is rounded once to the tensor's type.  Returns
    (var', m', v')."""
    var, m, v, grad = (np.asarray(a) for a in (var, m, v, grad))
    ct = _update_dtype(var.dtype)
    f = np.float32
    b1, b2 = f(beta1), f(beta2)
    omb1, omb2 = ct(f(1) - b1), ct(f(1) - b2)
    omb1p, omb2p = ct(f(1) - f(beta1_power)), ct(f(1) - f(beta2_power))
    b1, b2, lr_, eps = ct(b1), ct(b2), ct(f(lr)), ct(f(epsilon))
    g = grad.astype(ct)
    m_new = b1 * m.astype(ct) + omb1 * g
    v_new = b2 * v.astype(ct) + omb2 * g * g
    m_hat = (b1 * m_new + omb1 * g) / omb1p
    v_hat = v_new / omb2p
    var_new = var.astype(ct) - lr_ * m_hat / (np.sqrt(v_hat) + eps)
    return (var_new.astype(var.dtype), m_new.astype(var.dtype),
            v_new.astype(var.dtype))


def apply_rms_prop(var, ms, mom, lr, rho, momentum, epsilon, grad):
    """ResourceApplyRMSProp / ApplyRMSProp
    (musa_ext/kernels/training/musa_applyrmsprop_kernel.mu:84-98):
      ms' = rho*ms + (1-rho)*g^2;  mom' = momentum*mom + lr*g / sqrt(ms' + eps)
      var' = var - mom'
    Returns (var', ms', mom')."""
    var, ms, mom, grad = (np.asarray(a) for a in (var, ms, mom, grad))
    ct = _update_dtype(var.dtype)
    lr_, rho_, mo_, eps = ct(lr), ct(rho), ct(momentum), ct(epsilon)
    omr = ct(1) - rho_
    g = grad.astype(ct)
    ms_new = rho_ * ms.astype(ct) + omr * g * g
    mom_new = mo_ * mom.astype(ct) + lr_ * g / np.sqrt(ms_new + eps)
    var_new = var.astype(ct) - mom_new
    return (var_new.astype(var.dtype), ms_new.astype(var.dtype),
            mom_new.astype(var.dtype))


def apply_centered_rms_prop(var, mg, ms, mom, lr, rho, momentum, epsilon, grad):
    """ResourceApplyCenteredRMSProp / ApplyCenteredRMSProp
    (musa_ext/kernels/training/musa_applyrmsprop_kernel.mu:112-132):
      mg' = rho*mg + (1-rho)*g;  ms' = rho*ms + (1-rho)*g^2
      mom' = momentum*mom + lr*g / sqrt(ms' - mg'^2 + eps);  var' = var - mom'
    Returns (var', mg', ms', mom')."""
    var, mg, ms, mom, grad = (np.asarray(a) for a in (var, mg, ms, mom, grad))
    ct = _update_dtype(var.dtype)
    lr_, rho_, mo_, eps = ct(lr), ct(rho), ct(momentum), ct(epsilon)
    omr = ct(1) - rho_
    g = grad.astype(ct)
    mg_new = rho_ * mg.astype(ct) + omr * g
    ms_new = rho_ * ms.astype(ct) + omr * g * g
    denom = ms_new - mg_new * mg_new + eps
    mom_new = mo_ * mom.astype(ct) + lr_ * g / np.sqrt(denom)
    var_new = var.astype(ct) - mom_new
    return (var_new.astype(var.dtype), mg_new.astype(var.dtype),
            ms_new.astype(var.dtype), mom_new.astype(var.dtype))


def apply_gradient_descent(var, alpha, delta):
    """ResourceApplyGradientDescent and its mixed form: var' = var - alpha*delta
    (musa_ext/kernels/training/musa_applygradientdescent_kernel.mu:14-36).  A
    float variable takes a float or bfloat16 delta; a 16-bit variable rounds
    alpha*delta to its own type before the subtraction, like the separately
    stored product of musa_applygradientdescent_op.cc:186-199."""
    var, delta = np.asarray(var), np.asarray(delta)
    if var.dtype == np.float32:
        step = np.float32(alpha) * delta.astype(np.float32)
        return (var - step).astype(np.float32)
    ct = _compute_dtype(var.dtype)
    a = np.asarray(alpha).astype(var.dtype).astype(ct)
    step = (a * delta.astype(ct)).astype(var.dtype).astype(ct)
    return (var.astype(ct) - step).astype(var.dtype)


# --------------------------------------------------------------------------
# LayerNorm and RMSNorm over the last axis
# --------------------------------------------------------------------------

def layer_norm(x, gamma, beta, epsilon=1e-5):
    """MusaLayerNorm: y = (x - mean) / sqrt(var + eps) * gamma + beta over the
    last axis, population variance, statistics in fp64, one rounding to the
    tensor's type (musa_ext/kernels/fusion/musa_layernorm_op.cc:26-100; the
    reference test compares with Keras LayerNormalization,
    test/ops/layernorm_op_test.py:32-70)."""
    x = np.asarray(x)
    xf = x.astype(np.float64)
    mean = xf.mean(axis=-1, keepdims=True)
    var = np.square(xf - mean).mean(axis=-1, keepdims=True)
    y = (xf - mean) / np.sqrt(var + epsilon) * np.asarray(gamma).astype(np.float64) \
        + np.asarray(beta).astype(np.float64)
    return y.astype(x.dtype)


def layer_norm_grad(dy, x, gamma, epsilon=1e-5):
    """MusaLayerNormGrad: (dx, dgamma, dbeta)
    (musa_ext/kernels/fusion/musa_layernorm_grad_op.cc:23-141)."""
    x = np.asarray(x)
    xf, d = x.astype(np.float64), np.asarray(dy).astype(np.float64)
    g = np.asarray(gamma).astype(np.float64)
    mean = xf.mean(axis=-1, keepdims=True)
    var = np.square(xf - mean).mean(axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(var + epsilon)
    xh = (xf - mean) * inv
    gd = d * g
    dx = inv * (gd - gd.mean(axis=-1, keepdims=True)
                - xh * (gd * xh).mean(axis=-1, keepdims=True))
    red = tuple(range(x.ndim - 1))
    return (dx.astype(x.dtype), (d * xh).sum(axis=red).astype(x.dtype),
            d.sum(axis=red).astype(x.dtype))


def rms_norm(x, gamma, epsilon=1e-5):
    """MusaRmsNorm: inv = 1/sqrt(mean(x^2) + eps); normalized = x * inv;
    y = normalized * gamma; returns (y, normalized, inv_rms[..., 1])
    (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:58-92).  y is computed from the
    unrounded normalized value, as the kernel does."""
    x = np.asarray(x)
    xf = x.astype(np.float64)
    inv = 1.0 / np.sqrt(np.square(xf).mean(axis=-1, keepdims=True) + epsilon)
    norm = xf * inv
    return ((norm * np.asarray(gamma).astype(np.float64)).astype(x.dtype),
            norm.astype(x.dtype), inv.astype(x.dtype))


def rms_norm_grad_dx(x, inv_rms, gamma, dy):
    """MusaRmsNormGradDx: dx = dy*gamma*inv - x * (sum(x*dy*gamma) * inv^3 / n)
    with inv read in the tensor's type
    (musa_ext/kernels/nn/musa_rmsnorm_kernel.mu:171-204)."""
    x = np.asarray(x)
    xf, d = x.astype(np.float64), np.asarray(dy).astype(np.float64)
    g = np.asarray(gamma).astype(np.float64)
    inv = np.asarray(inv_rms).astype(np.float64).reshape(x.shape[:-1] + (1,))
    dot = (xf * d * g).sum(axis=-1, keepdims=True)
    coeff = dot * inv ** 3 / x.shape[-1]
    return (d * g * inv - xf * coeff).astype(x.dtype)


def apply_adagrad_v2(var, accum, lr, epsilon, grad, update_slots=True):
    """ResourceApplyAdagradV2 / ApplyAdagradV2: accum' = accum + g^2 (with
    update_slots); var' = var - lr * g / (sqrt(accum') + epsilon)
    (musa_ext/kernels/training/musa_applyadagrad_kernel.mu:65-77; the same
    statement as the reference test's NumPy helper,
    test/ops/apply_adagrad_op_test.py:53-62).  Returns (var', accum')."""
    var, accum, grad = (np.asarray(a) for a in (var, accum, grad))
    ct = _update_dtype(var.dtype)
    g = grad.astype(ct)
    acc = accum.astype(ct) + g * g if update_slots else accum.astype(ct)
    var_new = var.astype(ct) - ct(lr) * g / (np.sqrt(acc) + ct(epsilon))
    return var_new.astype(var.dtype), acc.astype(var.dtype)
