"""ctypes front end of oracle/cpu_ref.c (TEST INFRASTRUCTURE ONLY).

Loads oracle/build/libmusa_oracle.so, building it with `make` when it is
missing or was built for another CPU.  Used by the tests (as a second checker
beside np_ref.py) and by the benchmark's CPU-baseline leg; never by the
product.
"""
import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_DIR, "build", "libmusa_oracle.so")
_lib = None

DT = {"float32": 0, "float16": 1, "bfloat16": 2}


def build(force=False):
    if force and os.path.exists(_LIB):
        os.remove(_LIB)
    subprocess.run(["make", "-s", "-C", _DIR], check=True)
    return _LIB


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB):
        build()
    try:
        _lib = ctypes.CDLL(_LIB)
    except OSError:
        build(force=True)
        _lib = ctypes.CDLL(_LIB)
    i64, f32, vp, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
    _lib.cpu_ref_num_threads.restype = ci
    _lib.cpu_ref_set_num_threads.argtypes = [ci]
    _lib.cpu_ref_set_num_threads.restype = None
    _lib.cpu_bn_fwd_train.argtypes = [ci] + [vp] * 8 + [i64, i64, f32]
    _lib.cpu_bn_fwd_train.restype = None
    _lib.cpu_bn_grad.argtypes = [ci] + [vp] * 8 + [i64, i64, f32, ci]
    _lib.cpu_bn_grad.restype = None
    _lib.cpu_adam_f32.argtypes = [vp] * 4 + [f32] * 4 + [i64]
    _lib.cpu_adam_f32.restype = None
    _lib.cpu_bias_act.argtypes = [ci, vp, vp, vp, i64, i64, ci]
    _lib.cpu_bias_act.restype = None
    return _lib


def num_threads():
    return int(lib().cpu_ref_num_threads())


def set_num_threads(n):
    """Thread count of the following calls."""
    lib().cpu_ref_set_num_threads(int(n))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _code(a):
    return DT[str(a.dtype)]


def bn_fwd_train(x2d, scale, offset, epsilon):
    """x2d: [rows, C] C-contiguous.  Returns y, batch_mean, batch_var,
    saved_mean, saved_var."""
    x2d = np.ascontiguousarray(x2d)
    rows, c = x2d.shape
    y = np.empty_like(x2d)
    outs = [np.empty(c, np.float32) for _ in range(4)]
    scale = np.ascontiguousarray(scale, np.float32)
    offset = np.ascontiguousarray(offset, np.float32)
    lib().cpu_bn_fwd_train(_code(x2d), _p(x2d), _p(scale), _p(offset), _p(y),
                           *[_p(o) for o in outs], rows, c, float(epsilon))
    return (y, *outs)


def bn_grad(dy2d, x2d, scale, mean, variance, epsilon, is_training=True):
    dy2d = np.ascontiguousarray(dy2d)
    x2d = np.ascontiguousarray(x2d)
    rows, c = x2d.shape
    dx = np.empty_like(x2d)
    dscale = np.empty(c, np.float32)
    doffset = np.empty(c, np.float32)
    scale = np.ascontiguousarray(scale, np.float32)
    mean = np.ascontiguousarray(mean, np.float32)
    variance = np.ascontiguousarray(variance, np.float32)
    lib().cpu_bn_grad(_code(x2d), _p(dy2d), _p(x2d), _p(scale), _p(mean),
                      _p(variance), _p(dx), _p(dscale), _p(doffset), rows, c,
                      float(epsilon), int(bool(is_training)))
    return dx, dscale, doffset


def adam_f32(var, m, v, grad, beta1, beta2, epsilon, alpha):
    """In place on var, m, v (float32, contiguous)."""
    lib().cpu_adam_f32(_p(var), _p(m), _p(v), _p(grad), float(beta1),
                       float(beta2), float(epsilon), float(alpha), var.size)


def bias_act(x2d, bias, act):
    x2d = np.ascontiguousarray(x2d)
    rows, c = x2d.shape
    y = np.empty_like(x2d)
    bp = None if bias is None else _p(np.ascontiguousarray(bias))
    lib().cpu_bias_act(_code(x2d), _p(x2d), bp, _p(y), rows, c, int(act))
    return y
