"""Adam wrappers over the fused kernels.

`apply_adam_mixed` and `MusaAdam` keep the names and the routing rules of the
reference's Python layer (python/_optimizers.py:57-113 and :221-396 of the
reference project).  The reference's MusaAdam subclasses Keras' Adam; Keras is
not part of this build, so MusaAdam here is a small stand-alone optimizer with
the same hyper-parameters, slot names ("m", "v") and dispatch:

  fp32 variable + grad in {fp32, fp16, bf16}  -> MusaResourceApplyAdamMixed
  fp16/bf16 variable with a same-dtype grad    -> ResourceApplyAdam (16-bit
                                                  state, fp32 arithmetic)
  amsgrad=True                                 -> rejected (the reference falls
                                                  back to stock Keras there)
"""
import torch

from . import raw_ops
from .errors import InvalidArgumentError, UnimplementedError


def apply_adam_mixed(var, m, v, beta1_power, beta2_power, lr, beta1, beta2,
                     epsilon, grad, use_locking=False, use_nesterov=False):
    """One Adam step with fp32 state and a grad of fp32, fp16 or bf16.

    var, m, v: fp32 `raw_ops.Variable`s or device tensors, updated in place.
    The six scalars may be any real scalars; they are read as fp32, as the
    reference casts them (python/_optimizers.py:91-94)."""
    return raw_ops.MusaResourceApplyAdamMixed(
        var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon, grad,
        use_locking=use_locking, use_nesterov=use_nesterov)


class MusaAdam:
    """Adam over device tensors, one fused kernel per variable and step."""

    _LOWP_GRAD_DTYPES = (torch.float32, torch.bfloat16, torch.float16)

    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999,
                 epsilon=1e-7, amsgrad=False, use_nesterov=False, name="MusaAdam"):
        if amsgrad:
            raise UnimplementedError(
                "MusaAdam: AMSGrad has no fused kernel; use amsgrad=False")
        self.learning_rate = float(learning_rate)
        self.beta_1 = float(beta_1)
        self.beta_2 = float(beta_2)
        self.epsilon = float(epsilon)
        self.use_nesterov = bool(use_nesterov)
        self.name = name
        self.iterations = 0
        self._slots = {}

    def get_slot(self, var, slot_name):
        if slot_name not in ("m", "v"):
            raise InvalidArgumentError("unknown slot %r" % (slot_name,))
        key = id(var)
        if key not in self._slots:
            t = var.tensor() if isinstance(var, raw_ops.Variable) else var
            self._slots[key] = {"m": torch.zeros_like(t), "v": torch.zeros_like(t)}
        return self._slots[key][slot_name]

    def apply_gradients(self, grads_and_vars):
        """One step over (grad, var) pairs; returns the new iteration count."""
        step = self.iterations + 1
        b1p = self.beta_1 ** step
        b2p = self.beta_2 ** step
        for grad, var in grads_and_vars:
            if grad is None:
                continue
            t = var.tensor() if isinstance(var, raw_ops.Variable) else var
            m = self.get_slot(var, "m")
            v = self.get_slot(var, "v")
            if t.dtype == torch.float32:
                if grad.dtype not in self._LOWP_GRAD_DTYPES:
                    raise InvalidArgumentError(
                        "MusaAdam: unsupported grad dtype %s" % (grad.dtype,))
                raw_ops.MusaResourceApplyAdamMixed(
                    t, m, v, b1p, b2p, self.learning_rate, self.beta_1, self.beta_2,
                    self.epsilon, grad, use_nesterov=self.use_nesterov)
            else:
                raw_ops.ResourceApplyAdam(
                    t, m, v, b1p, b2p, self.learning_rate, self.beta_1, self.beta_2,
                    self.epsilon, grad, use_nesterov=self.use_nesterov)
        self.iterations = step
        return step
