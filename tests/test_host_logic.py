"""Host-side logic of the op front end that needs no device: geometry, host
scalars, alpha, variable locking and copy-on-write, and the refusal to run
without a GPU."""
import threading

import numpy as np
import pytest
import torch

from tensorflow_musa_extension_b200 import errors, raw_ops
from oracle import np_ref


def test_geometry():
    assert raw_ops._geometry((32, 56, 56, 64), "NHWC") == (32 * 56 * 56, 64, 1)
    assert raw_ops._geometry((8, 6, 16, 16), "NCHW") == (8, 6, 256)
    assert raw_ops._geometry((512, 64), "NHWC") == (512, 64, 1)
    assert raw_ops._geometry((4, 7), "NCHW") == (4, 7, 1)
    with pytest.raises(errors.InvalidArgumentError):
        raw_ops._geometry((2, 3), "NDHWC")


@pytest.mark.parametrize("b1p,b2p", [(0.9 ** 10, 0.999 ** 10), (1.0, 1.0), (0.9, 0.999)])
def test_alpha_matches_oracle(b1p, b2p):
    a = raw_ops._adam_alpha(float(np.float32(1e-3)), float(np.float32(b1p)),
                            float(np.float32(b2p)))
    assert np.float32(a) == np_ref.adam_alpha(np.float32(1e-3), np.float32(b1p),
                                              np.float32(b2p))


def test_scalars_are_read_as_the_op_dtype():
    assert raw_ops._scalar_in(0.999, torch.float32) == float(np.float32(0.999))
    # bfloat16 keeps 8 mantissa bits: 0.999 reads back as 1.0
    assert raw_ops._scalar_in(0.999, torch.bfloat16) == 1.0
    assert raw_ops._scalar_in(np.array([0.5]), torch.float16) == 0.5
    assert raw_ops._scalar_in(torch.tensor(0.25), torch.float32) == 0.25
    with pytest.raises(errors.InvalidArgumentError):
        raw_ops._scalar_in(np.zeros(2), torch.float32)


def test_variable_copy_on_write():
    v = raw_ops.Variable(torch.zeros(4))
    t0 = v.tensor()
    v.prepare_for_update()
    assert v.tensor() is t0          # sole owner: update in place
    alias = v.value()
    v.prepare_for_update()
    assert v.tensor() is not t0 and alias is t0   # reader keeps the old buffer
    t1 = v.tensor()
    v.prepare_for_update()
    assert v.tensor() is t1
    v.copy_on_read_mode = True
    v.prepare_for_update()
    assert v.tensor() is not t1
    assert not raw_ops.Variable().is_initialized


def test_lock_order_is_deduplicated_and_released():
    a, b = raw_ops.Variable(torch.zeros(1)), raw_ops.Variable(torch.zeros(1))
    locked = raw_ops._adam_lock([a, b, a], tensors_only=False)
    assert len(locked) == 2 and a.mu.locked() and b.mu.locked()
    assert [id(x) for x in locked] == sorted(id(x) for x in (a, b))
    for x in locked:
        x.mu.release()
    assert raw_ops._adam_lock([a, b, a], tensors_only=True) == []


def test_concurrent_lockers_do_not_deadlock():
    a, b = raw_ops.Variable(torch.zeros(1)), raw_ops.Variable(torch.zeros(1))
    done = []

    def work(order):
        for _ in range(200):
            locked = raw_ops._adam_lock(order, tensors_only=False)
            for x in reversed(locked):
                x.mu.release()
        done.append(1)

    ts = [threading.Thread(target=work, args=(o,)) for o in ([a, b], [b, a])]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=20)
    assert len(done) == 2


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU refusal")
def test_ops_refuse_to_run_without_a_device():
    x = np.zeros((2, 2, 2, 4), np.float32)
    s = np.ones(4, np.float32)
    with pytest.raises(errors.InternalError, match="no CPU implementation"):
        raw_ops.FusedBatchNormV3(x, s, s, s, s)
    with pytest.raises(errors.InternalError):
        raw_ops.BiasAdd(x, s)
    with pytest.raises(errors.InternalError):
        raw_ops.ResourceApplyAdam(torch.zeros(4), torch.zeros(4), torch.zeros(4), 0.9,
                                  0.999, 1e-3, 0.9, 0.999, 1e-7, torch.zeros(4))


def test_musa_adam_rejects_amsgrad():
    from tensorflow_musa_extension_b200.optimizers import MusaAdam
    with pytest.raises(errors.UnimplementedError):
        MusaAdam(amsgrad=True)
