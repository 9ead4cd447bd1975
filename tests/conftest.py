import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without a GPU is a collection-time skip, so that
    # `-m gpu` never passes by running nothing silently on the wrong box.
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return {name: np.load(os.path.join(GOLDEN, name + ".npz"))
            for name in ("adam_reference_numpy", "bn_torch_cpu",
                         "elementwise_literals", "bias_grad_torch_cpu",
                         "optimizer_cases", "row_norm_torch_cpu",
                         "adagrad_reference_numpy")}


@pytest.fixture(scope="session")
def kernel_lib():
    """The kernel library, built if needed; the tests call through this C ABI."""
    from tensorflow_musa_extension_b200 import build as b
    b.build()
    import tensorflow_musa_extension_b200 as pkg
    pkg.load_plugin()
    from tensorflow_musa_extension_b200 import raw_ops
    return raw_ops._lib()
