"""Op front end of the streaming optimizers next to Adam: Nadam, RMSProp
(plain and centered), Adagrad and gradient descent (single, mixed, grouped).

Each function mirrors one registered op of the reference: same name, argument
meaning, checks and error text; the update itself is one launch through the C
ABI of the kernel library.  State tensors are `raw_ops.Variable`s (resource
variables: mutex, initialised flag, copy-on-write) or plain device tensors."""
import ctypes

import numpy as np
import torch

from .errors import (FailedPreconditionError, InvalidArgumentError)
from . import raw_ops as _r

_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_LONG = {torch.float32: "Float", torch.float16: "Half", torch.bfloat16: "BFloat16",
         torch.float64: "Double"}


def _lock(variables):
    """De-duplicated, address-ordered locking, as every one of these ops does
    (e.g. musa_ext/kernels/training/musa_resource_apply_nadam_op.cc:64-82)."""
    uniq = sorted({id(v): v for v in variables if v is not None}.values(), key=id)
    for v in uniq:
        v.mu.acquire()
    return uniq


def _unlock(locked):
    for v in reversed(locked):
        v.mu.release()


def _resolve_states(opname, labels, states, uninit_message):
    """Variables -> their tensors (after the initialised check and the
    copy-on-write step); plain tensors pass through."""
    vs = [_r._as_variable(s) for s in states]
    if any(v is not None for v in vs) and not all(v is not None for v in vs):
        raise InvalidArgumentError(
            "%s: %s must all be Variables or all be tensors"
            % (opname, ", ".join(labels)))
    if vs[0] is None:
        return list(states)
    if not all(v.is_initialized for v in vs):
        raise FailedPreconditionError(uninit_message)
    for v in vs:
        v.prepare_for_update()
    return [v.tensor() for v in vs]


def _check_state_tensors(opname, labels, tensors, grad, dtypes):
    var_t = tensors[0]
    for label, t in zip(labels, tensors):
        if not (isinstance(t, torch.Tensor) and t.is_cuda):
            raise InvalidArgumentError(
                "%s: %s must be a device tensor (it is updated in place)" % (opname, label))
        if not t.is_contiguous():
            raise InvalidArgumentError("%s: %s must be contiguous" % (opname, label))
    if var_t.dtype not in dtypes:
        raise InvalidArgumentError("%s: unsupported dtype %s" % (opname, var_t.dtype))
    for label, t in list(zip(labels, tensors))[1:] + [("grad", grad)]:
        if tuple(t.shape) != tuple(var_t.shape):
            # CheckSameShape (musa_ext/kernels/training/musa_applyrmsprop_op.cc:150-160)
            raise InvalidArgumentError(
                "var and %s must have the same shape. var shape: %s, %s shape: %s"
                % (label, tuple(var_t.shape), label, tuple(t.shape)))
    for label, t in list(zip(labels, tensors))[1:]:
        if t.dtype != var_t.dtype:
            raise InvalidArgumentError(
                "%s: %s dtype %s does not match var dtype %s"
                % (opname, label, t.dtype, var_t.dtype))


def _scalar(value, name, dtype):
    """A scalar input read as T (`scalar<T>()`), widened to double."""
    arr = value.detach().cpu().numpy() if isinstance(value, torch.Tensor) else np.asarray(value)
    if arr.size != 1:
        # CheckScalar (musa_ext/kernels/training/musa_applyrmsprop_op.cc:162-168)
        raise InvalidArgumentError(
            "%s must be a scalar, got %d elements." % (name, arr.size))
    return _r._scalar_in(float(arr.reshape(())), dtype)


def _stateful(opname, labels, states, grad, uninit_message, lock, launch):
    _r._require_cuda()
    locked = _lock([_r._as_variable(s) for s in states]) if lock else []
    try:
        tensors = _resolve_states(opname, labels, states, uninit_message)
        hf = _r._HostForm()
        g = hf.to_device(grad)
        _check_state_tensors(opname, labels, tensors, g, _FLOATS)
        if g.dtype != tensors[0].dtype:
            raise InvalidArgumentError(
                "%s: grad dtype %s does not match var dtype %s"
                % (opname, g.dtype, tensors[0].dtype))
        n = tensors[0].numel()
        if n > 0:
            g = g.contiguous()
            with torch.cuda.device(tensors[0].device):
                launch(_r._lib(), tensors, g, n, _r._stream())
        return tensors[0]
    finally:
        _unlock(locked)


# ------------------------------------------------------------------ Nadam --

def ResourceApplyNadam(var, m, v, beta1_power, beta2_power, lr, beta1, beta2,
                       epsilon, grad, use_locking=False, name=None):
    """ResourceApplyNadam for T in {float, double, half, bfloat16}: in-place
    Nadam step on var, m, v; the six scalars are read as T and handed to the
    kernel as float (musa_ext/kernels/training/musa_resource_apply_nadam_op.cc:
    56-131, op definition :154-167).  Returns None."""
    def launch(lib, t, g, n, st):
        T = t[0].dtype
        sc = [_scalar(x, nm, T) for x, nm in (
            (beta1_power, "beta1_power"), (beta2_power, "beta2_power"), (lr, "lr"),
            (beta1, "beta1"), (beta2, "beta2"), (epsilon, "epsilon"))]
        fn = getattr(lib, "LaunchResourceApplyNadam_" + _LONG[T])
        fn(_r._ptr(t[0]), _r._ptr(t[1]), _r._ptr(t[2]), _r._ptr(g), *sc, n, st)

    _stateful("ResourceApplyNadam", ("var", "m", "v"), (var, m, v), grad,
              "Nadam variables (var/m/v) not initialized.", True, launch)
    return None


# ---------------------------------------------------------------- RMSProp --

def _rms_prop(opname, var, ms, mom, lr, rho, momentum, epsilon, grad, lock):
    def launch(lib, t, g, n, st):
        T = t[0].dtype
        sc = [_scalar(x, nm, T) for x, nm in (
            (lr, "lr"), (rho, "rho"), (momentum, "momentum"), (epsilon, "epsilon"))]
        fn = getattr(lib, "LaunchFusedResourceApplyRMSProp_" + _LONG[T])
        fn(_r._ptr(t[0]), _r._ptr(t[1]), _r._ptr(t[2]), _r._ptr(g), *sc, n, st)

    return _stateful(opname, ("var", "ms", "mom"), (var, ms, mom), grad,
                     "Fused RMSProp variables (var/ms/mom) not initialized.", lock, launch)


def _centered_rms_prop(opname, var, mg, ms, mom, lr, rho, momentum, epsilon, grad, lock):
    def launch(lib, t, g, n, st):
        T = t[0].dtype
        sc = [_scalar(x, nm, T) for x, nm in (
            (lr, "lr"), (rho, "rho"), (momentum, "momentum"), (epsilon, "epsilon"))]
        fn = getattr(lib, "LaunchFusedResourceApplyCenteredRMSProp_" + _LONG[T])
        fn(_r._ptr(t[0]), _r._ptr(t[1]), _r._ptr(t[2]), _r._ptr(t[3]), _r._ptr(g), *sc, n, st)

    return _stateful(opname, ("var", "mg", "ms", "mom"), (var, mg, ms, mom), grad,
                     "Fused CenteredRMSProp variables (var/mg/ms/mom) not initialized.",
                     lock, launch)


def ResourceApplyRMSProp(var, ms, mom, lr, rho, momentum, epsilon, grad,
                         use_locking=False, name=None):
    """ResourceApplyRMSProp for T in {float, double, half, bfloat16}
    (musa_ext/kernels/training/musa_applyrmsprop_op.cc:186-246, :493-496).  The
    variables are locked whatever `use_locking` says; the launch is not followed
    by a stream synchronisation (the reference's CheckLaunchAndSync, :170-182,
    waits for the kernel on every call).  Returns None."""
    _rms_prop("ResourceApplyRMSProp", var, ms, mom, lr, rho, momentum, epsilon, grad, True)
    return None


def ApplyRMSProp(var, ms, mom, lr, rho, momentum, epsilon, grad, use_locking=False,
                 name=None):
    """ApplyRMSProp (ref variables): same update, locks only with
    `use_locking`, output 0 forwards var
    (musa_ext/kernels/training/musa_applyrmsprop_op.cc:251-318)."""
    return _rms_prop("ApplyRMSProp", var, ms, mom, lr, rho, momentum, epsilon, grad,
                     bool(use_locking))


def ResourceApplyCenteredRMSProp(var, mg, ms, mom, lr, rho, momentum, epsilon, grad,
                                 use_locking=False, name=None):
    """ResourceApplyCenteredRMSProp
    (musa_ext/kernels/training/musa_applyrmsprop_op.cc:320-385, :503-506)."""
    _centered_rms_prop("ResourceApplyCenteredRMSProp", var, mg, ms, mom, lr, rho, momentum,
                       epsilon, grad, True)
    return None


def ApplyCenteredRMSProp(var, mg, ms, mom, lr, rho, momentum, epsilon, grad,
                         use_locking=False, name=None):
    """ApplyCenteredRMSProp (ref variables); output 0 forwards var
    (musa_ext/kernels/training/musa_applyrmsprop_op.cc:387-444, :508-511)."""
    return _centered_rms_prop("ApplyCenteredRMSProp", var, mg, ms, mom, lr, rho, momentum,
                              epsilon, grad, bool(use_locking))


# ---------------------------------------------------------------- Adagrad --

def _adagrad(opname, var, accum, lr, epsilon, grad, update_slots, lock):
    def launch(lib, t, g, n, st):
        T = t[0].dtype
        fn = getattr(lib, "LaunchFusedApplyAdagradV2_" + _LONG[T])
        fn(_r._ptr(t[0]), _r._ptr(t[1]), _r._ptr(g), _scalar(lr, "lr", T),
           _scalar(epsilon, "epsilon", T), bool(update_slots), n, st)

    return _stateful(opname, ("var", "accum"), (var, accum), grad,
                     "Fused AdagradV2 variables (var/accum) not initialized.", lock, launch)


def ResourceApplyAdagradV2(var, accum, lr, epsilon, grad, use_locking=False,
                           update_slots=True, name=None):
    """ResourceApplyAdagradV2 for T in {float, double, half, bfloat16}:
    accum += grad^2 (with update_slots), var -= lr * grad / (sqrt(accum) +
    epsilon) (musa_ext/kernels/training/musa_applyadagrad_op.cc:179-235,
    registrations :292-320).  Returns None."""
    _adagrad("ResourceApplyAdagradV2", var, accum, lr, epsilon, grad, update_slots, True)
    return None


def ApplyAdagradV2(var, accum, lr, epsilon, grad, use_locking=False, update_slots=True,
                   name=None):
    """ApplyAdagradV2 (ref variables): same update, locks only with
    `use_locking`, output 0 forwards var
    (musa_ext/kernels/training/musa_applyadagrad_op.cc:237-290)."""
    return _adagrad("ApplyAdagradV2", var, accum, lr, epsilon, grad, update_slots,
                    bool(use_locking))


# ------------------------------------------------------- gradient descent --

def _sgd_checks(opname, var_t, delta):
    if tuple(var_t.shape) != tuple(delta.shape):
        raise InvalidArgumentError(
            "Variable and gradient must have the same shape. var: %s grad: %s"
            % (tuple(var_t.shape), tuple(delta.shape)))


def _alpha(alpha, dtype):
    arr = alpha.detach().cpu().numpy() if isinstance(alpha, torch.Tensor) else np.asarray(alpha)
    if arr.size != 1:
        raise InvalidArgumentError("lr must be a scalar, got %d elements" % arr.size)
    return _r._scalar_in(float(arr.reshape(())), dtype)


def _sgd(opname, var, alpha, delta, delta_dtypes):
    _r._require_cuda()
    v = _r._as_variable(var)
    locked = _lock([v])
    try:
        if v is not None:
            if not v.is_initialized:
                raise FailedPreconditionError("Variable not initialized.")
            v.prepare_for_update()
            var_t = v.tensor()
        else:
            var_t = var
        if not (isinstance(var_t, torch.Tensor) and var_t.is_cuda and var_t.is_contiguous()):
            raise InvalidArgumentError(
                "%s: var must be a contiguous device tensor (it is updated in place)" % opname)
        hf = _r._HostForm()
        d = hf.to_device(delta)
        _sgd_checks(opname, var_t, d)
        if d.dtype not in delta_dtypes(var_t.dtype):
            raise InvalidArgumentError(
                "%s: delta dtype %s is not accepted for a %s variable"
                % (opname, d.dtype, var_t.dtype))
        a = _alpha(alpha, var_t.dtype)
        n = var_t.numel()
        if n > 0:
            d = d.contiguous()
            lib = _r._lib()
            with torch.cuda.device(var_t.device):
                if var_t.dtype == torch.float32:
                    fn = (lib.LaunchResourceApplyGradientDescentFloat
                          if d.dtype == torch.float32
                          else lib.LaunchResourceApplyGradientDescentFloatBFloat16)
                else:
                    fn = getattr(lib, "LaunchResourceApplyGradientDescent_"
                                 + _LONG[var_t.dtype])
                fn(_r._ptr(var_t), _r._ptr(d), a, n, _r._stream())
        return var_t
    finally:
        _unlock(locked)


def ResourceApplyGradientDescent(var, alpha, delta, use_locking=False, name=None):
    """ResourceApplyGradientDescent for T in {float, half, bfloat16}:
    var -= alpha * delta
    (musa_ext/kernels/training/musa_applygradientdescent_op.cc:124-226; double
    is not registered there either).  Returns None."""
    def dts(T):
        if T not in (torch.float32, torch.float16, torch.bfloat16):
            raise InvalidArgumentError(
                "ResourceApplyGradientDescent: unsupported dtype %s" % (T,))
        return (T,)
    _sgd("ResourceApplyGradientDescent", var, alpha, delta, dts)
    return None


def MusaResourceApplyGradientDescentMixed(var, alpha, delta, use_locking=False, name=None):
    """MusaResourceApplyGradientDescentMixed: float variable, bfloat16 delta
    (musa_ext/kernels/training/musa_applygradientdescent_op.cc:230-303)."""
    def dts(T):
        if T != torch.float32:
            raise InvalidArgumentError(
                "MusaResourceApplyGradientDescentMixed expects float variables")
        return (torch.bfloat16,)
    _sgd("MusaResourceApplyGradientDescentMixed", var, alpha, delta, dts)
    return None


def MusaGroupedResourceApplyGradientDescentMixed(vars, alphas, deltas, use_locking=False,
                                                 name=None):
    """MusaGroupedResourceApplyGradientDescentMixed: N float variables, N
    scalar alphas, N deltas that are all float or all bfloat16, one launch
    (musa_ext/kernels/training/musa_applygradientdescent_op.cc:305-460).  The
    descriptors go to the kernel as launch parameters, so nothing is staged
    through device tables.  Returns None."""
    opname = "MusaGroupedResourceApplyGradientDescentMixed"
    _r._require_cuda()
    n_t = len(vars)
    if n_t < 1 or len(alphas) != n_t or len(deltas) != n_t:
        raise InvalidArgumentError(
            "%s: vars, alphas and deltas must be N >= 1 entries each" % opname)
    vs = [_r._as_variable(v) for v in vars]
    locked = _lock(vs)
    try:
        tensors = []
        for v, raw in zip(vs, vars):
            if v is not None:
                if not v.is_initialized:
                    raise FailedPreconditionError("Variable not initialized.")
                v.prepare_for_update()
                tensors.append(v.tensor())
            else:
                tensors.append(raw)
        hf = _r._HostForm()
        ds = [hf.to_device(d) for d in deltas]
        a_list = []
        for i, (t, d, a) in enumerate(zip(tensors, ds, alphas)):
            arr = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
            if arr.size != 1:
                raise InvalidArgumentError(
                    "alpha must be a scalar, got %d elements" % arr.size)
            a_list.append(_r._scalar_in(float(arr.reshape(())), torch.float32))
            if not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous()):
                raise InvalidArgumentError(
                    "%s: vars[%d] must be a contiguous device tensor" % (opname, i))
            if t.dtype != torch.float32:
                raise InvalidArgumentError(opname + " expects float variables")
            if d.dtype not in (torch.float32, torch.bfloat16):
                raise InvalidArgumentError(opname + " expects float or bfloat16 gradients")
            if d.dtype != ds[0].dtype:
                raise InvalidArgumentError(
                    "%s: every delta must have the dtype of the first (Tgrad)" % opname)
            _sgd_checks(opname, t, d)
        ds = [d.contiguous() for d in ds]
        devices = {t.device for t in tensors}
        if len(devices) != 1:
            raise InvalidArgumentError("%s: variables live on several devices" % opname)
        VP = ctypes.c_void_p * n_t
        var_ptrs = VP(*[t.data_ptr() for t in tensors])
        delta_ptrs = VP(*[d.data_ptr() for d in ds])
        al = (ctypes.c_float * n_t)(*a_list)
        sizes = (ctypes.c_int64 * n_t)(*[t.numel() for t in tensors])
        with torch.cuda.device(tensors[0].device):
            rc = _r._lib().LaunchGroupedGradientDescentHostTable(
                var_ptrs, delta_ptrs, al, sizes, n_t,
                1 if ds[0].dtype == torch.bfloat16 else 0, _r._stream())
        _r._check(rc, opname)
        return None
    finally:
        _unlock(locked)
