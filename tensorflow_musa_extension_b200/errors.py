"""Error classes with the names of the TensorFlow status codes that the
reference kernels raise through OP_REQUIRES (e.g.
musa_ext/kernels/nn/musa_biasadd_op.cc:34-35,
musa_ext/kernels/training/musa_applyadam_op.cc:158-186)."""


class OpError(RuntimeError):
    """Base class, like tf.errors.OpError."""


class InvalidArgumentError(OpError, ValueError):
    pass


class FailedPreconditionError(OpError):
    pass


class InternalError(OpError):
    pass


class UnimplementedError(OpError, NotImplementedError):
    pass


class NotFoundError(OpError):
    pass
