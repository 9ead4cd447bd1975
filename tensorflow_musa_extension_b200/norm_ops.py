"""Op front end of the row normalisations: MusaLayerNorm, MusaLayerNormGrad,
MusaRmsNorm, MusaRmsNormGradDx.  Same names, argument meaning, checks and error
text as the reference ops; one launch each through the C ABI."""
import collections

import torch

from .errors import InvalidArgumentError
from . import raw_ops as _r

_LN_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
_RMS_DTYPES = (torch.float32, torch.bfloat16)

MusaLayerNormGradOutput = collections.namedtuple(
    "MusaLayerNormGrad", ["dx", "dgamma", "dbeta"])
MusaRmsNormOutput = collections.namedtuple(
    "MusaRmsNorm", ["y", "normalized", "inv_rms"])


def _rows(x):
    if x.dim() < 1:
        raise InvalidArgumentError("Input rank must be >= 1")
    last = x.shape[-1]
    return (x.numel() // last if last else 0), last


def _check_vector(v, name, last):
    if v.numel() != last:
        raise InvalidArgumentError(
            "%s size mismatch: expected %d, got %d" % (name, last, v.numel()))


def MusaLayerNorm(x, gamma, beta, epsilon=0.00001, name=None):
    """MusaLayerNorm for T in {float, half, bfloat16}: normalises the last
    axis, y = (x - mean) * rsqrt(var + epsilon) * gamma + beta
    (musa_ext/kernels/fusion/musa_layernorm_op.cc:26-100, op definition
    :118-124)."""
    _r._require_cuda()
    hf = _r._HostForm()
    xd, g, b = hf.to_device(x), hf.to_device(gamma), hf.to_device(beta)
    if xd.dtype not in _LN_DTYPES:
        raise InvalidArgumentError("MusaLayerNorm: unsupported dtype %s" % (xd.dtype,))
    if g.dtype != xd.dtype or b.dtype != xd.dtype:
        raise InvalidArgumentError("MusaLayerNorm: x, gamma and beta must share a dtype")
    rows, last = _rows(xd)
    _check_vector(g, "Gamma", last)
    _check_vector(b, "Beta", last)
    xd = xd.contiguous()
    with torch.cuda.device(xd.device):
        y = torch.empty_like(xd)
        if xd.numel():
            fn = getattr(_r._lib(), "LaunchLayerNorm_" + _r._SUFFIX[xd.dtype])
            rc = fn(_r._ptr(xd), _r._ptr(g.contiguous()), _r._ptr(b.contiguous()), _r._ptr(y),
                    None, None, rows, last, float(epsilon), _r._stream())
            _r._check(rc, "MusaLayerNorm")
    return hf.back(y)


def MusaLayerNormGrad(dy, x, gamma, beta, epsilon=0.00001, name=None):
    """MusaLayerNormGrad: (dx, dgamma, dbeta) from dy, x, gamma; the row
    statistics are recomputed from x
    (musa_ext/kernels/fusion/musa_layernorm_grad_op.cc:23-141, op definition
    :143-158)."""
    _r._require_cuda()
    hf = _r._HostForm()
    d, xd, g, b = (hf.to_device(t) for t in (dy, x, gamma, beta))
    if xd.dtype not in _LN_DTYPES:
        raise InvalidArgumentError("MusaLayerNormGrad: unsupported dtype %s" % (xd.dtype,))
    if any(t.dtype != xd.dtype for t in (d, g, b)):
        raise InvalidArgumentError("MusaLayerNormGrad: all inputs must share a dtype")
    if xd.dim() < 1:
        raise InvalidArgumentError("Input rank must be >= 1")
    if tuple(d.shape) != tuple(xd.shape):
        raise InvalidArgumentError(
            "dy and x must have the same shape: dy=%s, x=%s"
            % (tuple(d.shape), tuple(xd.shape)))
    rows, last = _rows(xd)
    _check_vector(g, "Gamma", last)
    _check_vector(b, "Beta", last)
    xd, d = xd.contiguous(), d.contiguous()
    with torch.cuda.device(xd.device):
        dx = torch.empty_like(xd)
        dgamma = torch.empty_like(g)
        dbeta = torch.empty_like(b)
        if last:
            lib = _r._lib()
            nbytes = lib.LayerNormGradWorkspaceBytes(rows, last)
            ws = _r._workspace(nbytes, xd.device)
            fn = getattr(lib, "LaunchLayerNormGrad_" + _r._SUFFIX[xd.dtype])
            rc = fn(_r._ptr(d), _r._ptr(xd), _r._ptr(g.contiguous()), _r._ptr(dx),
                    _r._ptr(dgamma), _r._ptr(dbeta), rows, last, float(epsilon), _r._ptr(ws),
                    ws.numel(), _r._stream())
            _r._check(rc, "MusaLayerNormGrad")
    return MusaLayerNormGradOutput(*hf.back_many([dx, dgamma, dbeta]))


def MusaRmsNorm(x, gamma, epsilon=0.00001, name=None):
    """MusaRmsNorm for T in {float, bfloat16}: returns (y, normalized,
    inv_rms), inv_rms shaped like x with a last axis of 1
    (musa_ext/kernels/nn/musa_rmsnorm_op.cc:24-87, op definition :175-201)."""
    _r._require_cuda()
    hf = _r._HostForm()
    xd, g = hf.to_device(x), hf.to_device(gamma)
    if xd.dtype not in _RMS_DTYPES or g.dtype != xd.dtype:
        raise InvalidArgumentError("MusaRmsNorm expects float/bfloat16 inputs")
    if xd.dim() < 1:
        raise InvalidArgumentError("Input rank must be >= 1")
    last = xd.shape[-1]
    if last <= 0:
        raise InvalidArgumentError("Last dimension must be positive")
    _check_vector(g, "Gamma", last)
    rows = xd.numel() // last
    xd = xd.contiguous()
    with torch.cuda.device(xd.device):
        y = torch.empty_like(xd)
        normalized = torch.empty_like(xd)
        inv = torch.empty(tuple(xd.shape[:-1]) + (1,), dtype=xd.dtype, device=xd.device)
        if xd.numel():
            lib = _r._lib()
            fn = lib.LaunchRmsNormFloat if xd.dtype == torch.float32 else lib.LaunchRmsNormBFloat16
            fn(_r._ptr(xd), _r._ptr(g.contiguous()), _r._ptr(y), _r._ptr(normalized),
               _r._ptr(inv), rows, last, float(epsilon), _r._stream())
    return MusaRmsNormOutput(*hf.back_many([y, normalized, inv]))


def MusaRmsNormGradDx(x, inv_rms, gamma, dy, name=None):
    """MusaRmsNormGradDx: the gradient of MusaRmsNorm with respect to x
    (musa_ext/kernels/nn/musa_rmsnorm_op.cc:96-146, op definition :163-173)."""
    _r._require_cuda()
    hf = _r._HostForm()
    xd, inv, g, d = (hf.to_device(t) for t in (x, inv_rms, gamma, dy))
    if xd.dtype not in _RMS_DTYPES or any(t.dtype != xd.dtype for t in (inv, g, d)):
        raise InvalidArgumentError("MusaRmsNormGradDx expects float/bfloat16 inputs")
    if tuple(xd.shape) != tuple(d.shape):
        raise InvalidArgumentError("MusaRmsNormGradDx x/dy shape mismatch")
    if g.dim() != 1:
        raise InvalidArgumentError("MusaRmsNormGradDx gamma must be rank 1")
    last = g.numel()
    if last <= 0 or xd.numel() % last != 0:
        raise InvalidArgumentError("MusaRmsNormGradDx invalid row size")
    rows = xd.numel() // last
    if inv.numel() != rows:
        raise InvalidArgumentError("MusaRmsNormGradDx inv size mismatch")
    xd, d = xd.contiguous(), d.contiguous()
    with torch.cuda.device(xd.device):
        dx = torch.empty_like(xd)
        if xd.numel():
            lib = _r._lib()
            fn = (lib.LaunchRmsNormGradDxFloat if xd.dtype == torch.float32
                  else lib.LaunchRmsNormGradDxBFloat16)
            fn(_r._ptr(xd), _r._ptr(inv.contiguous()), _r._ptr(g.contiguous()), _r._ptr(d),
               _r._ptr(dx), rows, last, _r._stream())
    return hf.back(dx)
