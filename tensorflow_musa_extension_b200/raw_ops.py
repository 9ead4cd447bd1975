"""Op front end: the TensorFlow op names of the BatchNorm / Adam / BiasAdd +
activation path, with their attrs, dtype sets and error behaviour, executed by
the sm_100a kernel library.

This is the host-side mirror of the reference's OpKernel layer: each function
does what the matching `Compute()` does around its device call (shape and dtype
checks, output allocation, host-scalar handling) and then calls the C launcher.

Tensors are torch CUDA tensors.  Host buffers (NumPy arrays or CPU torch
tensors) are accepted too: they are copied to the current device on the current
stream, the op runs, and the outputs come back in the same host form; that is
the end-to-end path a TensorFlow feed/fetch takes.  There is no CPU
implementation behind these functions: without a device or without the kernel
library they raise.
"""
import collections
import threading

import numpy as np
import torch

from . import _capi
from . import _loader
from .errors import (FailedPreconditionError, InternalError,
                     InvalidArgumentError, UnimplementedError)

try:
    import ml_dtypes
    _NP_BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _NP_BF16 = None

ACT_IDENTITY, ACT_RELU, ACT_SWISH, ACT_SIGMOID = 0, 1, 2, 3

_SUFFIX = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
           torch.float64: "F64", torch.int32: "I32", torch.int64: "I64"}
_DT_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_bound = None
_bind_lock = threading.Lock()


def _lib():
    global _bound
    if _bound is None:
        with _bind_lock:
            if _bound is None:
                _bound = _capi.bind(_loader.get_library())
    return _bound


def _require_cuda():
    if not torch.cuda.is_available():
        raise InternalError(
            "no CUDA device is visible: the MUSA ops have no CPU implementation")


# ---------------------------------------------------------------- tensors --

class _HostForm:
    """Remembers how host inputs arrived so that outputs go back the same way."""

    def __init__(self):
        self.kind = None  # None (device) | "numpy" | "torch_cpu"

    def to_device(self, t, dtype=None):
        if t is None:
            return None
        if isinstance(t, torch.Tensor):
            if t.is_cuda:
                out = t
            else:
                self.kind = self.kind or "torch_cpu"
                out = t.to("cuda", non_blocking=True)
        else:
            a = np.asarray(t)
            self.kind = self.kind or "numpy"
            if _NP_BF16 is not None and a.dtype == _NP_BF16:
                ht = torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(
                    torch.bfloat16)
            else:
                ht = torch.from_numpy(np.ascontiguousarray(a))
            out = ht.to("cuda", non_blocking=True)
        if dtype is not None and out.dtype != dtype:
            out = out.to(dtype)
        return out

    def back(self, t):
        """Device result -> host, through pinned memory (torch's caching host
        allocator stands where the reference keeps a pinned bounce-buffer pool,
        musa_ext/mu/device/pinned_memory_pool.h:46-108)."""
        return self.back_many((t,))[0]

    def back_many(self, tensors):
        """All results to the host with one stream synchronisation."""
        if self.kind is None:
            return list(tensors)
        hs = []
        for t in tensors:
            if t is None:
                hs.append(None)
                continue
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            h.copy_(t, non_blocking=True)
            hs.append(h)
        torch.cuda.current_stream().synchronize()
        if self.kind == "torch_cpu":
            return hs
        out = []
        for h in hs:
            if h is None:
                out.append(None)
            elif h.dtype == torch.bfloat16:
                out.append(h.view(torch.int16).numpy().view(_NP_BF16))
            else:
                out.append(h.numpy())
        return out


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(rc, what):
    if rc == 0:
        return
    if rc < 0:
        raise InvalidArgumentError("%s: %s" % (what, _capi.ERROR_NAMES.get(rc, rc)))
    raise InternalError("%s: CUDA error %d" % (what, rc))


_ws_cache = {}


def _workspace(nbytes, device):
    """Scratch for the BatchNorm launchers (TensorFlow: allocate_temp).  One
    growing buffer per (device, stream); reuse on one stream is ordered."""
    key = (device.index, _stream())
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _geometry(shape, data_format):
    """[outer, channels, inner] view of a tensor shape."""
    if data_format == "NHWC":
        c = shape[-1]
        outer = 1
        for d in shape[:-1]:
            outer *= d
        return outer, c, 1
    if data_format == "NCHW":
        inner = 1
        for d in shape[2:]:
            inner *= d
        return shape[0], shape[1], inner
    raise InvalidArgumentError("Invalid data format: %r" % (data_format,))


# ------------------------------------------------------- FusedBatchNorm ----

FusedBatchNormV3Output = collections.namedtuple(
    "FusedBatchNormV3",
    ["y", "batch_mean", "batch_variance", "reserve_space_1", "reserve_space_2",
     "reserve_space_3"])
FusedBatchNormOutput = collections.namedtuple(
    "FusedBatchNorm",
    ["y", "batch_mean", "batch_variance", "reserve_space_1", "reserve_space_2"])
FusedBatchNormGradV3Output = collections.namedtuple(
    "FusedBatchNormGradV3",
    ["x_backprop", "scale_backprop", "offset_backprop", "reserve_space_4",
     "reserve_space_5"])

_BN_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def _bn_check_inputs(x, vecs, data_format, opname):
    if x.dtype not in _BN_DTYPES:
        raise InvalidArgumentError(
            "%s: T must be one of float, half, bfloat16; got %s" % (opname, x.dtype))
    if x.dim() < 2:
        raise InvalidArgumentError("%s: input must be at least 2-D" % opname)
    outer, c, inner = _geometry(tuple(x.shape), data_format)
    for name, v in vecs:
        if v is None:
            continue
        if v.dim() != 1:
            raise InvalidArgumentError("%s: %s must be 1-dimensional" % (opname, name))
        if v.numel() != c and not (name in ("mean", "variance") and v.numel() == 0):
            raise InvalidArgumentError(
                "%s: %s must have %d elements, got %d" % (opname, name, c, v.numel()))
    return outer, c, inner


def FusedBatchNormV3(x, scale, offset, mean, variance, epsilon=0.0001,
                     exponential_avg_factor=1.0, data_format="NHWC",
                     is_training=True, name=None):
    """FusedBatchNormV3 on T in {float, half, bfloat16} with float statistics
    (registration: musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:303-325;
    Compute: :42-182).  Returns the op's six outputs."""
    _require_cuda()
    hf = _HostForm()
    x = hf.to_device(x)
    scale = hf.to_device(scale, torch.float32)
    offset = hf.to_device(offset, torch.float32)
    mean = hf.to_device(mean, torch.float32)
    variance = hf.to_device(variance, torch.float32)
    outer, c, inner = _bn_check_inputs(
        x, (("scale", scale), ("offset", offset), ("mean", mean),
            ("variance", variance)), data_format, "FusedBatchNormV3")
    have_est = mean is not None and mean.numel() == c and \
        variance is not None and variance.numel() == c
    if not is_training and not have_est:
        raise InvalidArgumentError(
            "FusedBatchNormV3: mean and variance must be given when is_training=False")
    if is_training and float(exponential_avg_factor) != 1.0 and not have_est:
        raise InvalidArgumentError(
            "FusedBatchNormV3: mean and variance must be given when "
            "exponential_avg_factor != 1")
    x = x.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        y = torch.empty_like(x)
        stats = [torch.empty(c, dtype=torch.float32, device=dev) for _ in range(4)]
        reserve_3 = torch.zeros((), dtype=torch.float32, device=dev)
        sfx = _SUFFIX[x.dtype]
        if x.numel() == 0:
            for s in stats:
                s.zero_()
        elif is_training:
            nbytes = _lib().BnWorkspaceBytes(outer, c, inner)
            ws = _workspace(nbytes, dev)
            fn = getattr(_lib(), "LaunchBnFwdTrain_" + sfx)
            rc = fn(_ptr(x), _ptr(scale), _ptr(offset),
                    _ptr(mean) if have_est else None,
                    _ptr(variance) if have_est else None, _ptr(y),
                    _ptr(stats[0]), _ptr(stats[1]), _ptr(stats[2]), _ptr(stats[3]),
                    outer, c, inner, float(epsilon), float(exponential_avg_factor),
                    _ptr(ws), ws.numel(), _stream())
            _check(rc, "FusedBatchNormV3")
        else:
            fn = getattr(_lib(), "LaunchBnFwdInfer_" + sfx)
            rc = fn(_ptr(x), _ptr(scale), _ptr(offset), _ptr(mean), _ptr(variance),
                    _ptr(y), outer, c, inner, float(epsilon), _stream())
            _check(rc, "FusedBatchNormV3")
            # The op passes the given statistics through in inference mode.
            stats[0].copy_(mean)
            stats[1].copy_(variance)
            stats[2].copy_(mean)
            stats[3].copy_(variance)
    return FusedBatchNormV3Output(*hf.back_many((y, *stats, reserve_3)))


def FusedBatchNormV2(x, scale, offset, mean, variance, epsilon=0.0001,
                     exponential_avg_factor=1.0, data_format="NHWC",
                     is_training=True, name=None):
    """FusedBatchNormV2: the V3 kernel without reserve_space_3."""
    out = FusedBatchNormV3(x, scale, offset, mean, variance, epsilon,
                           exponential_avg_factor, data_format, is_training)
    return FusedBatchNormOutput(*out[:5])


def FusedBatchNorm(x, scale, offset, mean, variance, epsilon=0.0001,
                   exponential_avg_factor=1.0, data_format="NHWC",
                   is_training=True, name=None):
    """FusedBatchNorm (V1): the same kernel class serves all three versions."""
    out = FusedBatchNormV3(x, scale, offset, mean, variance, epsilon,
                           exponential_avg_factor, data_format, is_training)
    return FusedBatchNormOutput(*out[:5])


def FusedBatchNormGradV3(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                         reserve_space_3=None, epsilon=0.0001, data_format="NHWC",
                         is_training=True, name=None):
    """FusedBatchNormGradV3 (Compute:
    musa_ext/kernels/nn/musa_fused_batchnorm_op.cc:206-295).  reserve_space_1
    is the mean, reserve_space_2 the population variance; reserve_space_3 is
    accepted and ignored.  Outputs 3 and 4 are zero-filled [C], as the
    reference emits them (:220-242)."""
    _require_cuda()
    hf = _HostForm()
    dy = hf.to_device(y_backprop)
    x = hf.to_device(x)
    scale = hf.to_device(scale, torch.float32)
    mean = hf.to_device(reserve_space_1, torch.float32)
    var = hf.to_device(reserve_space_2, torch.float32)
    outer, c, inner = _bn_check_inputs(
        x, (("scale", scale), ("reserve_space_1", mean), ("reserve_space_2", var)),
        data_format, "FusedBatchNormGradV3")
    if dy.shape != x.shape:
        raise InvalidArgumentError(
            "FusedBatchNormGradV3: x and y_backprop must have same shape, but x has "
            "shape %s and y_backprop has shape %s" % (tuple(x.shape), tuple(dy.shape)))
    if dy.dtype != x.dtype:
        raise InvalidArgumentError(
            "FusedBatchNormGradV3: x and y_backprop must have the same dtype")
    x = x.contiguous()
    dy = dy.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        dx = torch.empty_like(x)
        dscale = torch.empty(c, dtype=torch.float32, device=dev)
        doffset = torch.empty(c, dtype=torch.float32, device=dev)
        r4 = torch.zeros(c, dtype=torch.float32, device=dev)
        r5 = torch.zeros(c, dtype=torch.float32, device=dev)
        if x.numel() == 0:
            dscale.zero_()
            doffset.zero_()
        else:
            nbytes = _lib().BnWorkspaceBytes(outer, c, inner)
            ws = _workspace(nbytes, dev)
            fn = getattr(_lib(), "LaunchBnGrad_" + _SUFFIX[x.dtype])
            rc = fn(_ptr(dy), _ptr(x), _ptr(scale), _ptr(mean), _ptr(var), _ptr(dx),
                    _ptr(dscale), _ptr(doffset), outer, c, inner, float(epsilon),
                    bool(is_training), _ptr(ws), ws.numel(), _stream())
            _check(rc, "FusedBatchNormGradV3")
    return FusedBatchNormGradV3Output(*hf.back_many((dx, dscale, doffset, r4, r5)))


def FusedBatchNormGradV2(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                         epsilon=0.0001, data_format="NHWC", is_training=True,
                         name=None):
    return FusedBatchNormGradV3(y_backprop, x, scale, reserve_space_1,
                                reserve_space_2, None, epsilon, data_format,
                                is_training)


def FusedBatchNormGrad(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                       epsilon=0.0001, data_format="NHWC", is_training=True,
                       name=None):
    return FusedBatchNormGradV3(y_backprop, x, scale, reserve_space_1,
                                reserve_space_2, None, epsilon, data_format,
                                is_training)


# ------------------------------------------------------------- ApplyAdam ---

class Variable:
    """A resource variable as the Adam ops see it: a tensor, a mutex, and the
    copy-on-read flag (the fields of tensorflow::Var that
    musa_ext/kernels/training/musa_applyadam_op.cc:74-156 uses).

    `value()` hands out an alias of the tensor; while aliases are alive the
    next in-place update first copies the tensor (copy-on-write,
    PrepareTensorForMusaUpdate :97-106), so a reader never sees a half-updated
    buffer."""

    def __init__(self, tensor=None, name="Variable"):
        self.name = name
        self.mu = threading.Lock()
        self.copy_on_read_mode = False
        self._tensor = tensor
        self._aliases = 0

    @property
    def is_initialized(self):
        return self._tensor is not None

    def tensor(self):
        return self._tensor

    def assign(self, tensor):
        self._tensor = tensor
        self._aliases = 0

    def value(self):
        self._aliases += 1
        return self._tensor

    def release(self):
        """Drop one alias handed out by value()."""
        if self._aliases > 0:
            self._aliases -= 1

    def prepare_for_update(self):
        if self._tensor is None:
            return
        if self.copy_on_read_mode or self._aliases > 0:
            self._tensor = self._tensor.clone()
            self._aliases = 0


def _as_variable(v):
    return v if isinstance(v, Variable) else None


def _np_dtype_of(t):
    if t == torch.bfloat16:
        return _NP_BF16
    return {torch.float32: np.float32, torch.float16: np.float16,
            torch.float64: np.float64}[t]


def _scalar_in(value, torch_dtype):
    """A host scalar input read as the op's T and widened to double (the
    kernel reads `scalar<T>()`; musa_applyadam_op.cc:224-229)."""
    if isinstance(value, torch.Tensor):
        value = value.detach().cpu().to(torch.float64).item()
    arr = np.asarray(value)
    if arr.size != 1:
        raise InvalidArgumentError("scalar input expected, got shape %s" % (arr.shape,))
    return float(np.asarray(arr.reshape(()).astype(np.float64)).astype(
        _np_dtype_of(torch_dtype)).astype(np.float64))


def _adam_alpha(lr, beta1_power, beta2_power):
    """alpha = lr * sqrt(1 - beta2^t) / (1 - beta1^t) in float64, with the
    first-step guard (musa_applyadam_op.cc:236-246)."""
    one_minus = 1.0 - beta1_power
    if abs(one_minus) < 1e-10:
        return lr
    return lr * float(np.sqrt(1.0 - beta2_power)) / one_minus


def _adam_lock(variables, tensors_only):
    """De-duplicated, address-ordered locking of the var/m/v mutexes, always
    taken whatever use_locking says (musa_applyadam_op.cc:138-156)."""
    if tensors_only:
        return []
    uniq = sorted({id(v): v for v in variables}.values(), key=id)
    for v in uniq:
        v.mu.acquire()
    return uniq


def _adam_impl(opname, var, m, v, beta1_power, beta2_power, lr, beta1, beta2,
               epsilon, grad, use_nesterov, mixed):
    _require_cuda()
    vs = [_as_variable(t) for t in (var, m, v)]
    all_vars = all(x is not None for x in vs)
    if not all_vars and any(x is not None for x in vs):
        raise InvalidArgumentError(
            "%s: var, m and v must all be Variables or all be tensors" % opname)
    locked = _adam_lock(vs, not all_vars)
    try:
        if all_vars:
            for label, x in zip(("var", "m", "v"), vs):
                if not x.is_initialized:
                    raise FailedPreconditionError(
                        "Attempting to use uninitialized variables: %s (%s)"
                        % (x.name, label))
            for x in vs:
                x.prepare_for_update()
            var_t, m_t, v_t = (x.tensor() for x in vs)
        else:
            var_t, m_t, v_t = var, m, v
        hf = _HostForm()
        grad = hf.to_device(grad)
        for label, t in (("var", var_t), ("m", m_t), ("v", v_t)):
            if not (isinstance(t, torch.Tensor) and t.is_cuda):
                raise InvalidArgumentError(
                    "%s: %s must be a device tensor (it is updated in place)"
                    % (opname, label))
            if not t.is_contiguous():
                raise InvalidArgumentError("%s: %s must be contiguous" % (opname, label))
        if var_t.shape != m_t.shape:
            raise InvalidArgumentError(
                "var and m do not have the same shape %s %s"
                % (tuple(var_t.shape), tuple(m_t.shape)))
        if var_t.shape != v_t.shape:
            raise InvalidArgumentError(
                "var and v do not have the same shape %s %s"
                % (tuple(var_t.shape), tuple(v_t.shape)))
        if var_t.shape != grad.shape:
            raise InvalidArgumentError(
                "var and grad do not have the same shape %s %s"
                % (tuple(var_t.shape), tuple(grad.shape)))
        T = var_t.dtype
        if m_t.dtype != T or v_t.dtype != T:
            raise InvalidArgumentError("%s: var, m and v must share a dtype" % opname)
        if mixed:
            if T != torch.float32:
                raise InvalidArgumentError(
                    "%s: var, m and v must be float, got %s" % (opname, T))
            if grad.dtype not in _BN_DTYPES:
                raise InvalidArgumentError(
                    "%s: T must be one of float, half, bfloat16; got %s"
                    % (opname, grad.dtype))
            scalar_t = torch.float32
        else:
            if grad.dtype != T:
                raise InvalidArgumentError(
                    "%s: grad dtype %s does not match var dtype %s"
                    % (opname, grad.dtype, T))
            if T in (torch.int32, torch.int64):
                # Registered by the reference for ResourceApplyAdam only
                # (musa_applyadam_op.cc:676-677) and served by its op chain
                # (:297-415), whose integer results hang on what a closed
                # library does for integer sqrt and divide (beta1 = beta2 = 0
                # after the cast to T, a divide by sqrt(g*g) + 0); TensorFlow's
                # own CPU kernel, the parity oracle of this op, is not
                # registered for integer T at all.  There is nothing to match.
                raise UnimplementedError(
                    "%s: T=%s is not supported: TensorFlow's CPU kernel has no integer "
                    "ApplyAdam to compare with, and the reference's element-wise op chain "
                    "for it (musa_applyadam_op.cc:297-415) is defined only by a closed "
                    "library's integer sqrt/divide; float, double, half and bfloat16 are "
                    "served" % (opname, T))
            if T not in _BN_DTYPES and T != torch.float64:
                raise InvalidArgumentError(
                    "%s: T must be one of float, double, half, bfloat16; got %s"
                    % (opname, T))
            scalar_t = T
        b1p = _scalar_in(beta1_power, scalar_t)
        b2p = _scalar_in(beta2_power, scalar_t)
        lr_ = _scalar_in(lr, scalar_t)
        b1 = _scalar_in(beta1, scalar_t)
        b2 = _scalar_in(beta2, scalar_t)
        eps = _scalar_in(epsilon, scalar_t)
        alpha = _adam_alpha(lr_, b1p, b2p)
        n = var_t.numel()
        if n > 0:
            grad = grad.contiguous()
            L = _lib()
            with torch.cuda.device(var_t.device):
                st = _stream()
                if T == torch.float64:
                    # One pass with the operations, order and roundings of the
                    # reference's op chain for this dtype (:297-415).
                    L.LaunchApplyAdam_F64(_ptr(var_t), _ptr(m_t), _ptr(v_t), _ptr(grad),
                                          alpha, b1, b2, eps, n, bool(use_nesterov), st)
                elif mixed or (T == torch.float32 and use_nesterov):
                    fn = {torch.float32: L.LaunchApplyAdamMixed_Float,
                          torch.float16: L.LaunchApplyAdamMixed_Half,
                          torch.bfloat16: L.LaunchApplyAdamMixed_BFloat16}[grad.dtype]
                    fn(_ptr(var_t), _ptr(m_t), _ptr(v_t), _ptr(grad), alpha, b1, b2,
                       eps, n, bool(use_nesterov), st)
                elif T == torch.float32:
                    L.LaunchResourceApplyAdamFloat(
                        _ptr(var_t), _ptr(m_t), _ptr(v_t), _ptr(grad), b1, b2, eps,
                        alpha, n, st)
                else:
                    fn = (L.LaunchApplyAdamSameType_BFloat16 if T == torch.bfloat16
                          else L.LaunchApplyAdamSameType_Half)
                    fn(_ptr(var_t), _ptr(m_t), _ptr(v_t), _ptr(grad), alpha, b1, b2,
                       eps, n, bool(use_nesterov), st)
        return var_t
    finally:
        for x in reversed(locked):
            x.mu.release()


def ResourceApplyAdam(var, m, v, beta1_power, beta2_power, lr, beta1, beta2,
                      epsilon, grad, use_locking=False, use_nesterov=False,
                      name=None):
    """ResourceApplyAdam: in-place Adam step on var, m, v
    (musa_ext/kernels/training/musa_applyadam_op.cc:130-416; registered for
    float, double, half, bfloat16, int64 and int32, :672-677; the two integer
    types raise Unimplemented here, with the reason in the message).  var/m/v are `Variable`s or
    device tensors.  The six scalars are host values read as T; alpha is taken
    in float64.  float + use_nesterov runs the Nesterov numerator (TensorFlow's
    CPU kernel honours the attr; the reference's float fast path is taken only
    without it, :248-265).  Returns None, as the op has no outputs."""
    _adam_impl("ResourceApplyAdam", var, m, v, beta1_power, beta2_power, lr, beta1,
               beta2, epsilon, grad, use_nesterov, mixed=False)
    return None


def ApplyAdam(var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon,
              grad, use_locking=False, use_nesterov=False, name=None):
    """ApplyAdam (ref variables): same update; output 0 forwards var
    (musa_ext/kernels/training/musa_applyadam_op.cc:423-643, :531-537)."""
    return _adam_impl("ApplyAdam", var, m, v, beta1_power, beta2_power, lr, beta1,
                      beta2, epsilon, grad, use_nesterov, mixed=False)


def MusaResourceApplyAdamMixed(var, m, v, beta1_power, beta2_power, lr, beta1,
                               beta2, epsilon, grad, use_locking=False,
                               use_nesterov=False, name=None):
    """MusaResourceApplyAdamMixed: float var/m/v, grad T in {float, half,
    bfloat16}, float scalars, use_nesterov honoured (op definition
    musa_ext/kernels/training/musa_applyadam_mixed_op.cc:265-281; Compute
    :125-258)."""
    _adam_impl("MusaResourceApplyAdamMixed", var, m, v, beta1_power, beta2_power,
               lr, beta1, beta2, epsilon, grad, use_nesterov, mixed=True)
    return None


# --------------------------------------------- BiasAdd, Relu, Sigmoid, fused --

_BIAS_DTYPES = (torch.float32, torch.float64, torch.float16, torch.bfloat16,
                torch.int32, torch.int64)
_ACT_FLOAT = (torch.float32, torch.float16, torch.bfloat16)


def _bias_act(opname, value, bias, data_format, act, dtypes):
    _require_cuda()
    hf = _HostForm()
    x = hf.to_device(value)
    b = hf.to_device(bias)
    if x.dtype not in dtypes:
        raise InvalidArgumentError("%s: unsupported dtype %s" % (opname, x.dtype))
    if b is not None:
        if b.dtype != x.dtype:
            raise InvalidArgumentError(
                "%s: bias dtype %s does not match value dtype %s"
                % (opname, b.dtype, x.dtype))
        if x.dim() < 2:
            raise InvalidArgumentError(
                "Input tensor must be at least 2D: %s" % (tuple(x.shape),))
        if b.dim() != 1:
            raise InvalidArgumentError(
                "Biases must be 1D: %s" % (tuple(b.shape),))
    x = x.contiguous()
    with torch.cuda.device(x.device):
        y = torch.empty_like(x)
        # Empty input or bias: allocate the output and return
        # (musa_ext/kernels/nn/musa_biasadd_op.cc:27-31).
        if x.numel() == 0 or (b is not None and b.numel() == 0):
            return hf.back(y)
        if b is not None:
            outer, c, inner = _geometry(tuple(x.shape), data_format)
            if b.shape[0] != c:
                raise InvalidArgumentError("Dimension mismatch in BiasAdd")
            b = b.contiguous()
        else:
            outer, c, inner = x.numel(), 1, 1
        fn = getattr(_lib(), "LaunchBiasAct_" + _SUFFIX[x.dtype])
        rc = fn(_ptr(x), _ptr(b), _ptr(y), outer, c, inner, act, _stream())
        _check(rc, opname)
    return hf.back(y)


def BiasAdd(value, bias, data_format="NHWC", name=None):
    """BiasAdd for T in {float, double, half, bfloat16, int32, int64}
    (musa_ext/kernels/nn/musa_biasadd_op.cc:23-61, :67-80)."""
    return _bias_act("BiasAdd", value, bias, data_format, ACT_IDENTITY, _BIAS_DTYPES)


def BiasAddV1(value, bias, name=None):
    """BiasAddV1: BiasAdd with the channel on the last axis."""
    return _bias_act("BiasAddV1", value, bias, "NHWC", ACT_IDENTITY, _BIAS_DTYPES)


def Relu(features, name=None):
    """Relu for T in {float, half, bfloat16, double}
    (musa_ext/kernels/nn/musa_relu_op.cc:19-57)."""
    return _bias_act("Relu", features, None, "NHWC", ACT_RELU,
                     _ACT_FLOAT + (torch.float64,))


def Sigmoid(x, name=None):
    """Sigmoid for T in {float, half, bfloat16}
    (musa_ext/kernels/nn/musa_sigmoid_op.cc:18-35, :68-78)."""
    return _bias_act("Sigmoid", x, None, "NHWC", ACT_SIGMOID, _ACT_FLOAT)


def MusaBiasAddRelu(value, bias, data_format="NHWC", name=None):
    """Fused Relu(BiasAdd(value, bias)): the op that the BiasAdd->Relu fusion
    pattern emits.  New here: the reference fuses this chain only behind a
    MatMul (musa_ext/graph/fusion/linear_activation_fusion.cc:100-117)."""
    return _bias_act("MusaBiasAddRelu", value, bias, data_format, ACT_RELU, _ACT_FLOAT)


def MusaBiasAddSwish(value, bias, data_format="NHWC", name=None):
    """Fused Mul(value, Sigmoid(BiasAdd(value, bias)))."""
    return _bias_act("MusaBiasAddSwish", value, bias, data_format, ACT_SWISH,
                     _ACT_FLOAT)


def MusaBiasAddSigmoid(value, bias, data_format="NHWC", name=None):
    """Fused Sigmoid(BiasAdd(value, bias))."""
    return _bias_act("MusaBiasAddSigmoid", value, bias, data_format, ACT_SIGMOID,
                     _ACT_FLOAT)


# ------------------------------------ BiasAddGrad, ReluGrad, fused backward --

MusaBiasAddReluGradOutput = collections.namedtuple(
    "MusaBiasAddReluGrad", ["backprops", "bias_grad"])


def _bias_grad_geometry(shape, data_format, opname):
    if data_format not in ("NHWC", "NCHW"):
        raise InvalidArgumentError("Invalid data format")
    if len(shape) < 1:
        raise InvalidArgumentError(
            "Input tensor must be at least 1D: %s" % (tuple(shape),))
    if len(shape) == 1:
        return 1, shape[0], 1
    if data_format == "NCHW":
        inner = 1
        for d in shape[2:]:
            inner *= d
        return shape[0], shape[1], inner
    outer = 1
    for d in shape[:-1]:
        outer *= d
    return outer, shape[-1], 1


def BiasAddGrad(out_backprop, data_format="NHWC", name=None):
    """BiasAddGrad for T in {float, double, half, bfloat16, int32, int64}: the
    sum of `out_backprop` over every axis but the channel axis (last for NHWC,
    1 for NCHW), in the tensor's type.  A 1-D input is returned as it is; an
    input with no elements gives zeros
    (musa_ext/kernels/nn/musa_biasadd_grad_op.cc:23-106, :113-118)."""
    _require_cuda()
    hf = _HostForm()
    g = hf.to_device(out_backprop)
    if g.dtype not in _BIAS_DTYPES:
        raise InvalidArgumentError("BiasAddGrad: unsupported dtype %s" % (g.dtype,))
    outer, c, inner = _bias_grad_geometry(tuple(g.shape), data_format, "BiasAddGrad")
    if g.dim() == 1:
        return hf.back(g)
    g = g.contiguous()
    with torch.cuda.device(g.device):
        out = torch.empty((c,), dtype=g.dtype, device=g.device)
        lib = _lib()
        nbytes = lib.BiasGradWorkspaceBytes(outer, c, inner, g.element_size())
        ws = _workspace(nbytes, g.device)
        fn = getattr(lib, "LaunchBiasAddGrad_" + _SUFFIX[g.dtype])
        rc = fn(_ptr(g), _ptr(out), outer, c, inner, _ptr(ws), ws.numel(),
                _stream())
        _check(rc, "BiasAddGrad")
    return hf.back(out)


def _relu_grad_inputs(opname, gradients, features, hf):
    g = hf.to_device(gradients)
    f = hf.to_device(features)
    if g.dtype not in _ACT_FLOAT:
        raise InvalidArgumentError("%s: unsupported dtype %s" % (opname, g.dtype))
    if f.dtype != g.dtype:
        raise InvalidArgumentError(
            "%s: features dtype %s does not match gradients dtype %s"
            % (opname, f.dtype, g.dtype))
    if tuple(g.shape) != tuple(f.shape):
        raise InvalidArgumentError(
            "Inputs to ReluGrad must have the same shape. gradients: %s, "
            "features: %s" % (tuple(g.shape), tuple(f.shape)))
    return g.contiguous(), f.contiguous()


def ReluGrad(gradients, features, name=None):
    """ReluGrad for T in {float, half, bfloat16}: gradients * (features > 0)
    (musa_ext/kernels/nn/musa_relu_grad_op.cc:19-48, :56-58)."""
    _require_cuda()
    hf = _HostForm()
    g, f = _relu_grad_inputs("ReluGrad", gradients, features, hf)
    with torch.cuda.device(g.device):
        out = torch.empty_like(g)
        if g.numel():
            fn = getattr(_lib(), "LaunchReluGrad_" + _SUFFIX[g.dtype])
            _check(fn(_ptr(g), _ptr(f), _ptr(out), g.numel(), _stream()),
                   "ReluGrad")
    return hf.back(out)


def MusaBiasAddReluGrad(gradients, features, data_format="NHWC", name=None):
    """Fused BiasAddGrad(ReluGrad(gradients, features)): returns (backprops,
    bias_grad) from one pass over the two inputs.  The op that the
    ReluGrad->BiasAddGrad fusion pattern emits; the reference runs the two ops
    separately (musa_ext/kernels/nn/musa_relu_grad_op.cc,
    musa_ext/kernels/nn/musa_biasadd_grad_op.cc)."""
    _require_cuda()
    hf = _HostForm()
    g, f = _relu_grad_inputs("MusaBiasAddReluGrad", gradients, features, hf)
    outer, c, inner = _bias_grad_geometry(tuple(g.shape), data_format,
                                          "MusaBiasAddReluGrad")
    with torch.cuda.device(g.device):
        dx = torch.empty_like(g)
        db = torch.empty((c,), dtype=g.dtype, device=g.device)
        lib = _lib()
        nbytes = lib.BiasGradWorkspaceBytes(outer, c, inner, g.element_size())
        ws = _workspace(nbytes, g.device)
        fn = getattr(lib, "LaunchBiasAddReluGrad_" + _SUFFIX[g.dtype])
        rc = fn(_ptr(g), _ptr(f), _ptr(dx), _ptr(db), outer, c, inner, _ptr(ws),
                ws.numel(), _stream())
        _check(rc, "MusaBiasAddReluGrad")
    dx, db = hf.back_many([dx, db])
    return MusaBiasAddReluGradOutput(dx, db)


# ------------------------------ Nadam, RMSProp, gradient descent (re-export) --
# Defined in training_ops.py; imported last because that module uses the
# helpers above.
from .training_ops import (  # noqa: E402,F401
    ApplyAdagradV2, ApplyCenteredRMSProp, ApplyRMSProp, ResourceApplyAdagradV2, MusaGroupedResourceApplyGradientDescentMixed,
    MusaResourceApplyGradientDescentMixed, ResourceApplyCenteredRMSProp,
    ResourceApplyGradientDescent, ResourceApplyNadam, ResourceApplyRMSProp)
from .norm_ops import (  # noqa: E402,F401
    MusaLayerNorm, MusaLayerNormGrad, MusaRmsNorm, MusaRmsNormGradDx)
