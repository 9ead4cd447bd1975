"""B200-native kernels for the memory-bound training path of the
`tensorflow_musa` plugin: FusedBatchNorm forward/gradient, ApplyAdam and
BiasAdd + activation chains, behind the plugin's op names.

Public surface (the reference package's, python/__init__.py:81-117 of the
reference project, restricted to this path):
    load_plugin, get_musa_ops, is_plugin_loaded, get_musa_devices
    raw_ops                 op front end (FusedBatchNormV3, ResourceApplyAdam, ...)
    apply_adam_mixed        functional wrapper of MusaResourceApplyAdamMixed

Importing the package does not load the kernel library; the first op call (or
`load_plugin()`) does, and raises if it is missing.  The reference auto-loads on
import and only warns on failure (python/__init__.py:70-78); here a missing
library is an error at first use so that a silent fallback cannot happen.
"""
from ._loader import (PLUGIN_LIBRARY, get_library, get_musa_devices,
                      get_musa_ops, is_plugin_loaded, load_plugin)
from . import errors

__version__ = "0.1.0"


def __getattr__(name):
    # raw_ops needs torch; import it lazily so that the loader and the build
    # helpers work in a bare interpreter.
    if name == "raw_ops":
        import importlib
        return importlib.import_module(".raw_ops", __name__)
    if name == "apply_adam_mixed":
        from .optimizers import apply_adam_mixed
        return apply_adam_mixed
    if name == "MusaAdam":
        from .optimizers import MusaAdam
        return MusaAdam
    raise AttributeError(name)
