"""The allocation-free BatchNorm forward entry point against the regular one.

LaunchBnFwdTrainNoAlloc serves callers that are not allowed to allocate device
memory (allocation-free serving loops, host callbacks without a framework
allocator, processes whose memory was handed out in full at start): it brings
its own scratch inside the library image instead of taking a workspace.  It
must return what LaunchBnFwdTrain_* returns, call after call, although every
call reuses the same scratch and finds the previous call's contents in it.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.  It also passes alone in a fresh process
(the first call on a device resolves the scratch address).
"""
import numpy as np
import pytest
import torch

from helpers import RTOL, assert_close, bn_inputs, to_numpy, to_torch
from oracle import np_ref

pytestmark = pytest.mark.gpu

EPS = 1e-3
DT = {"float32": (0, "F32"), "float16": (1, "F16"), "bfloat16": (2, "BF16")}


def _run(lib, entry, x, scale, offset, workspace):
    rows, c = x.shape
    y = torch.empty_like(x)
    stats = [torch.empty(c, device="cuda") for _ in range(4)]
    st = torch.cuda.current_stream().cuda_stream
    head = [x.data_ptr(), scale.data_ptr(), offset.data_ptr(), None, None, y.data_ptr()] + \
        [t.data_ptr() for t in stats] + [rows, c, 1, EPS, 1.0]
    if workspace is None:
        rc = entry(*head, st)
    else:
        rc = entry(*head, workspace.data_ptr(), workspace.numel(), st)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return [y] + stats


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_calls_in_a_row_match_the_workspace_entry_point(kernel_lib, dtype):
    code, sfx = DT[dtype]
    regular = getattr(kernel_lib, "LaunchBnFwdTrain_" + sfx)

    def no_alloc(*args):
        return kernel_lib.LaunchBnFwdTrainNoAlloc(code, *args)

    # Two different problems back to back: the second call finds the first
    # call's partial sums in the shared scratch and must not be affected.
    for seed, shape, mean, std in ((31, (6000, 64), 0.5, 2.0), (32, (1234, 200), -3.0, 0.7)):
        x, s, o, _ = bn_inputs(seed, shape, dtype, mean, std)
        tx, ts, to = to_torch(x), to_torch(s), to_torch(o)
        need = kernel_lib.BnWorkspaceBytes(shape[0], shape[1], 1)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        want = _run(kernel_lib, regular, tx, ts, to, ws)
        got = _run(kernel_lib, no_alloc, tx, ts, to, None)
        rt = RTOL["f32_bn"] if dtype == "float32" else RTOL["lowp"]
        names = ["y", "batch_mean", "batch_var", "saved_mean", "saved_var"]
        for name, g, w in zip(names, got, want):
            w_np = to_numpy(w)
            scale_ = float(np.sqrt(np.mean(w_np.astype(np.float64) ** 2))) or 1.0
            assert_close(to_numpy(g), w_np, rt if name == "y" else RTOL["f32_bn"],
                         1e-6 * scale_, "%s seed %d" % (name, seed))
        # ... and what the CPU oracle returns for the same inputs.
        oracle = np_ref.fused_batch_norm(x, s, o, epsilon=EPS)
        for name, g, w in zip(names, got, oracle):
            rms = float(np.sqrt(np.mean(np.asarray(w, np.float64) ** 2))) or 1.0
            r = rt if name == "y" else RTOL["f32_bn"]
            assert_close(to_numpy(g), w, r, r * rms, "oracle %s seed %d" % (name, seed))


def test_sizes_beyond_the_scratch_are_refused(kernel_lib):
    cap = kernel_lib.BnNoAllocMaxChannels()
    assert cap == 8192
    c = cap + 8
    x = torch.zeros(4, c, device="cuda")
    v = torch.ones(c, device="cuda")
    outs = [torch.full((c,), 7.0, device="cuda") for _ in range(4)]
    y = torch.full_like(x, 7.0)
    st = torch.cuda.current_stream().cuda_stream
    rc = kernel_lib.LaunchBnFwdTrainNoAlloc(
        0, x.data_ptr(), v.data_ptr(), v.data_ptr(), None, None, y.data_ptr(),
        *[t.data_ptr() for t in outs], 4, c, 1, EPS, 1.0, st)
    assert rc == -4                      # MUSA_KERNELS_ETOOLARGE
    torch.cuda.synchronize()
    assert float(y.min()) == 7.0 and float(outs[0].min()) == 7.0   # nothing ran
    # The largest accepted width still works.
    x = torch.randn(64, cap, device="cuda")
    v = torch.ones(cap, device="cuda")
    outs = [torch.empty(cap, device="cuda") for _ in range(4)]
    y = torch.empty_like(x)
    rc = kernel_lib.LaunchBnFwdTrainNoAlloc(
        0, x.data_ptr(), v.data_ptr(), v.data_ptr(), None, None, y.data_ptr(),
        *[t.data_ptr() for t in outs], 64, cap, 1, EPS, 1.0, st)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.allclose(outs[2], x.mean(0), atol=1e-5)
