"""ApplyAdam on the GPU (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import np_ref
from helpers import (ADAM_HYPER, NP_BF16, RTOL, adam_inputs, assert_close, np_dtype,
                     to_numpy, to_torch)
from tensorflow_musa_extension_b200 import errors, raw_ops

pytestmark = pytest.mark.gpu

H = ADAM_HYPER


def _step_args():
    return (H["beta1_power"], H["beta2_power"], H["lr"], H["beta1"], H["beta2"],
            H["epsilon"])


@pytest.mark.parametrize("case", ["step10", "first_step_guard", "step1"])
def test_reference_numpy_golden(golden, kernel_lib, case):
    g = golden["adam_reference_numpy"]
    s = [float(x) for x in g[case + "/scalars"]]
    var, m, v = (to_torch(g[case + "/" + k].copy()) for k in ("var", "m", "v"))
    raw_ops.ResourceApplyAdam(var, m, v, s[0], s[1], s[2], s[3], s[4], s[5],
                              to_torch(g[case + "/grad"]))
    assert_close(to_numpy(m), g[case + "/expected_m"], RTOL["f32_adam"], 1e-10, "m")
    assert_close(to_numpy(v), g[case + "/expected_v"], RTOL["f32_adam"], 1e-14, "v")
    assert_close(to_numpy(var), g[case + "/expected_var"], RTOL["f32_adam"], 1e-8, "var")


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 255, 256, 1025, 262147])
def test_f32_sizes_and_ragged_tails(kernel_lib, n):
    rng, var, m, v = adam_inputs(3, n)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    ev, em, evv = np_ref.apply_adam(var, m, v, *_step_args(), g)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    raw_ops.ResourceApplyAdam(tv, tm, tvv, *_step_args(), to_torch(g))
    assert_close(to_numpy(tm), em, RTOL["f32_adam"], 1e-10, "m")
    assert_close(to_numpy(tvv), evv, RTOL["f32_adam"], 1e-14, "v")
    assert_close(to_numpy(tv), ev, RTOL["f32_adam"], 1e-8, "var")


@pytest.mark.parametrize("n", [0, 1, 2, 3, 255, 1025, 262147])
@pytest.mark.parametrize("nesterov", [False, True])
def test_double_follows_the_op_chain_bit_for_bit(kernel_lib, n, nesterov):
    """T = double: the reference runs thirteen element-wise ops that each
    round to double (musa_applyadam_op.cc:297-415); the one-pass kernel performs
    the same operations in the same order, so three steps agree with the NumPy
    restatement of the chain exactly, except where libm's sqrt and the
    device's IEEE sqrt could differ (they do not: both round correctly)."""
    rng = np.random.default_rng(50 + n)
    var = rng.normal(0, 0.05, n)
    m = rng.normal(0, 1e-4, n)
    v = rng.uniform(0, 1e-6, n)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    for step in range(1, 4):
        g = rng.normal(0, 1e-3, n)
        args = (0.9 ** step, 0.999 ** step, 1e-3, 0.9, 0.999, 1e-7)
        var, m, v = np_ref.apply_adam_op_chain(var, m, v, *args, g, use_nesterov=nesterov)
        raw_ops.ResourceApplyAdam(tv, tm, tvv, *args, to_torch(g), use_nesterov=nesterov)
    assert tv.dtype == torch.float64
    assert np.array_equal(to_numpy(tm), m)
    assert np.array_equal(to_numpy(tvv), v)
    assert np.array_equal(to_numpy(tv), var)


def test_double_through_apply_adam_and_misaligned_slices(kernel_lib):
    n = 4099
    rng = np.random.default_rng(61)
    var, m, v, g = (rng.normal(0, 0.05, n + 1) for _ in range(4))
    v = np.abs(v) * 1e-4
    ev, em, evv = np_ref.apply_adam_op_chain(var[1:], m[1:], v[1:], *_step_args(), g[1:])
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    out = raw_ops.ApplyAdam(tv[1:], tm[1:], tvv[1:], *_step_args(), to_torch(g)[1:])
    assert out.data_ptr() == tv[1:].data_ptr()
    assert np.array_equal(to_numpy(tv)[1:], ev) and to_numpy(tv)[0] == var[0]
    assert np.array_equal(to_numpy(tm)[1:], em)
    assert np.array_equal(to_numpy(tvv)[1:], evv)


def test_hundred_steps_fresh_grad_each_step(kernel_lib):
    """The benchmark protocol (100 steps, a fresh seeded grad per step) at a
    size the NumPy oracle finishes in seconds; includes a ragged tail."""
    n = (1 << 20) + 3
    rng, var, m, v = adam_inputs(3, n)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    for _ in range(100):
        g = rng.normal(0, 1e-3, n).astype(np.float32)
        var, m, v = np_ref.apply_adam(var, m, v, *_step_args(), g)
        raw_ops.ResourceApplyAdam(tv, tm, tvv, *_step_args(), to_torch(g))
    assert_close(to_numpy(tm), m, RTOL["f32_adam"], 1e-9, "m")
    assert_close(to_numpy(tvv), v, RTOL["f32_adam"], 1e-13, "v")
    assert_close(to_numpy(tv), var, RTOL["f32_adam"], 1e-7, "var")


def test_full_size_parameter_vector(kernel_lib):
    """ResNet-50's 25,557,032 parameters, three steps against the oracle."""
    n = 25_557_032
    rng, var, m, v = adam_inputs(3, n)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    for _ in range(3):
        g = rng.normal(0, 1e-3, n).astype(np.float32)
        var, m, v = np_ref.apply_adam(var, m, v, *_step_args(), g)
        raw_ops.ResourceApplyAdam(tv, tm, tvv, *_step_args(), to_torch(g))
    assert_close(to_numpy(tm), m, RTOL["f32_adam"], 1e-9, "m")
    assert_close(to_numpy(tvv), v, RTOL["f32_adam"], 1e-13, "v")
    assert_close(to_numpy(tv), var, RTOL["f32_adam"], 1e-7, "var")


def test_update_is_elementwise_independent_of_sharding(kernel_lib):
    """Range sharding must not change any element: one launch over the whole
    vector equals 8 launches over contiguous shards, bit for bit."""
    n = 1_000_003
    rng, var, m, v = adam_inputs(3, n)
    g = to_torch(rng.normal(0, 1e-3, n).astype(np.float32))
    a = [to_torch(t) for t in (var, m, v)]
    b = [to_torch(t) for t in (var, m, v)]
    raw_ops.ResourceApplyAdam(*a, *_step_args(), g)
    per = (n + 7) // 8
    for r in range(8):
        lo, hi = r * per, min(n, (r + 1) * per)
        raw_ops.ResourceApplyAdam(*[t[lo:hi] for t in b], *_step_args(), g[lo:hi])
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_misaligned_pointers_take_the_elementwise_path(kernel_lib):
    n = 4099
    rng, var, m, v = adam_inputs(4, n + 1)
    g = rng.normal(0, 1e-3, n + 1).astype(np.float32)
    ev, em, evv = np_ref.apply_adam(var[1:], m[1:], v[1:], *_step_args(), g[1:])
    tv, tm, tvv, tg = (to_torch(t) for t in (var, m, v, g))
    raw_ops.ResourceApplyAdam(tv[1:], tm[1:], tvv[1:], *_step_args(), tg[1:])
    assert_close(to_numpy(tv)[1:], ev, RTOL["f32_adam"], 1e-8, "var")
    assert_close(to_numpy(tm)[1:], em, RTOL["f32_adam"], 1e-10, "m")
    assert to_numpy(tv)[0] == var[0] and to_numpy(tm)[0] == m[0]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("nesterov", [False, True])
def test_same_type_16bit_state(kernel_lib, dtype, nesterov):
    dt = np.float16 if dtype == "float16" else NP_BF16
    n = 70001
    rng = np.random.default_rng(6)
    var = rng.normal(0, 0.5, n).astype(dt)
    m = rng.normal(0, 1e-2, n).astype(dt)
    v = rng.uniform(0, 1e-3, n).astype(dt)
    g = rng.normal(0, 1e-1, n).astype(dt)
    args = (0.9 ** 10, 0.999 ** 10, 1e-2, 0.9, 0.999, 1e-4)
    ev, em, evv = np_ref.apply_adam(var, m, v, *[np.asarray(a).astype(dt) for a in args],
                                    g, use_nesterov=nesterov)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    raw_ops.ResourceApplyAdam(tv, tm, tvv, *args, to_torch(g), use_nesterov=nesterov)
    # Same fp32 arithmetic, one rounding: at most one 16-bit ulp apart.
    assert_close(to_numpy(tm), em, RTOL["lowp"], 1e-8, "m")
    assert_close(to_numpy(tvv), evv, RTOL["lowp"], 1e-8, "v")
    assert_close(to_numpy(tv), ev, RTOL["lowp"], 1e-6, "var")


@pytest.mark.parametrize("gdtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("nesterov", [False, True])
def test_mixed_precision_op(kernel_lib, gdtype, nesterov):
    gdt = {"float32": np.float32, "float16": np.float16, "bfloat16": NP_BF16}[gdtype]
    n = 50003
    rng, var, m, v = adam_inputs(8, n)
    g = rng.normal(0, 1e-3, n).astype(gdt)
    ev, em, evv = np_ref.apply_adam(var, m, v, *_step_args(), g, use_nesterov=nesterov)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    raw_ops.MusaResourceApplyAdamMixed(tv, tm, tvv, *_step_args(), to_torch(g),
                                       use_nesterov=nesterov)
    assert_close(to_numpy(tm), em, RTOL["f32_adam"], 1e-10, "m")
    assert_close(to_numpy(tvv), evv, RTOL["f32_adam"], 1e-14, "v")
    assert_close(to_numpy(tv), ev, RTOL["f32_adam"], 1e-8, "var")


def test_f32_nesterov_is_honoured(kernel_lib):
    n = 1000
    rng, var, m, v = adam_inputs(9, n)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    ev, _, _ = np_ref.apply_adam(var, m, v, *_step_args(), g, use_nesterov=True)
    tv, tm, tvv = to_torch(var), to_torch(m), to_torch(v)
    raw_ops.ResourceApplyAdam(tv, tm, tvv, *_step_args(), to_torch(g), use_nesterov=True)
    assert_close(to_numpy(tv), ev, RTOL["f32_adam"], 1e-8, "var")


def test_apply_adam_forwards_var(kernel_lib):
    n = 64
    rng, var, m, v = adam_inputs(10, n)
    tv = to_torch(var)
    out = raw_ops.ApplyAdam(tv, to_torch(m), to_torch(v), *_step_args(),
                            to_torch(rng.normal(0, 1e-3, n).astype(np.float32)))
    assert out.data_ptr() == tv.data_ptr()


def test_variables_errors_and_copy_on_write(kernel_lib):
    n = 128
    rng, var, m, v = adam_inputs(11, n)
    g = to_torch(rng.normal(0, 1e-3, n).astype(np.float32))
    V = raw_ops.Variable
    with pytest.raises(errors.FailedPreconditionError, match="uninitialized"):
        raw_ops.ResourceApplyAdam(V(to_torch(var)), V(None, "m0"), V(to_torch(v)),
                                  *_step_args(), g)
    with pytest.raises(errors.InvalidArgumentError, match="var and m do not have the same shape"):
        raw_ops.ResourceApplyAdam(V(to_torch(var)), V(to_torch(m[:-1])), V(to_torch(v)),
                                  *_step_args(), g)
    with pytest.raises(errors.InvalidArgumentError, match="var and grad"):
        raw_ops.ResourceApplyAdam(V(to_torch(var)), V(to_torch(m)), V(to_torch(v)),
                                  *_step_args(), g[:-1])
    for idt in (np.int32, np.int64):
        # Registered by the reference, defined by neither TensorFlow's CPU
        # kernel nor an open statement of the integer chain: refused, and the
        # message says why.
        iv = to_torch(np.arange(n).astype(idt))
        with pytest.raises(errors.UnimplementedError, match="no integer ApplyAdam"):
            raw_ops.ResourceApplyAdam(iv, iv.clone(), iv.clone(), *_step_args(), iv.clone())
        assert np.array_equal(to_numpy(iv), np.arange(n))       # untouched
    vv = V(to_torch(var))
    snapshot = vv.value()
    raw_ops.ResourceApplyAdam(vv, V(to_torch(m)), V(to_torch(v)), *_step_args(), g)
    assert np.array_equal(to_numpy(snapshot), var)          # reader's view intact
    assert not np.array_equal(to_numpy(vv.tensor()), var)   # variable moved on
    assert not vv.mu.locked()


def test_musa_adam_matches_oracle_over_steps(kernel_lib):
    from tensorflow_musa_extension_b200.optimizers import MusaAdam
    n = 10000
    rng, var, _, _ = adam_inputs(12, n)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    tv = to_torch(var)
    opt = MusaAdam(learning_rate=1e-3)
    for step in range(1, 6):
        g = rng.normal(0, 1e-3, n).astype(NP_BF16)
        var, m, v = np_ref.apply_adam(var, m, v, 0.9 ** step, 0.999 ** step, 1e-3, 0.9,
                                      0.999, 1e-7, g)
        opt.apply_gradients([(to_torch(g), tv)])
    assert opt.iterations == 5
    assert_close(to_numpy(tv), var, RTOL["f32_adam"], 1e-8, "var")
    assert_close(to_numpy(opt.get_slot(tv, "m")), m, RTOL["f32_adam"], 1e-10, "m")


def test_sharded_broadcast_kernel_on_one_gpu(kernel_lib):
    """LaunchAdamShardBroadcastFloat with 4 "replicas" that all live on this
    GPU: each shard's launch must update its range in every copy, so after the
    4 launches every copy equals the un-sharded update, bit for bit."""
    import ctypes
    from tensorflow_musa_extension_b200.cross_replica import aligned_shard_range
    n, world = 1_000_003, 4
    rng, var, m, v = adam_inputs(21, n)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    want = [to_torch(t) for t in (var, m, v)]
    raw_ops.ResourceApplyAdam(*want, *_step_args(), to_torch(g))
    copies = [to_torch(var) for _ in range(world)]
    tm, tvv, tg = to_torch(m), to_torch(v), to_torch(g)
    ptrs = (ctypes.c_void_p * world)(*[c_.data_ptr() for c_ in copies])
    alpha = raw_ops._adam_alpha(*[float(np.float32(H[k])) for k in
                                  ("lr", "beta1_power", "beta2_power")])
    st = torch.cuda.current_stream().cuda_stream
    spans = [aligned_shard_range(n, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n and all(lo % 4 == 0 for lo, _ in spans)
    for r, (lo, hi) in enumerate(spans):
        rc = kernel_lib.LaunchAdamShardBroadcastFloat(
            ptrs, world, r, lo, tm[lo:hi].data_ptr(), tvv[lo:hi].data_ptr(),
            tg[lo:hi].data_ptr(), float(np.float32(H["beta1"])), float(np.float32(H["beta2"])),
            float(np.float32(H["epsilon"])), alpha, hi - lo, st)
        assert rc == 0
    torch.cuda.synchronize()
    for c_ in copies:
        assert torch.equal(c_, want[0])
    assert torch.equal(tm, want[1]) and torch.equal(tvv, want[2])
    # an unaligned range start takes the element-wise path and still matches
    copies2 = [to_torch(var) for _ in range(2)]
    ptrs2 = (ctypes.c_void_p * 2)(*[c_.data_ptr() for c_ in copies2])
    tm2, tv2 = to_torch(m), to_torch(v)
    rc = kernel_lib.LaunchAdamShardBroadcastFloat(
        ptrs2, 2, 1, 3, tm2[3:1000].data_ptr(), tv2[3:1000].data_ptr(), tg[3:1000].data_ptr(),
        float(np.float32(H["beta1"])), float(np.float32(H["beta2"])),
        float(np.float32(H["epsilon"])), alpha, 997, st)
    assert rc == 0
    torch.cuda.synchronize()
    for c_ in copies2:
        assert torch.equal(c_[3:1000], want[0][3:1000]) and torch.equal(c_[1000:], copies2[0][1000:])
        assert np.array_equal(to_numpy(c_[:3]), var[:3])


@pytest.mark.parametrize("gdtype", ["float16", "bfloat16"])
def test_sharded_adam_takes_16bit_gradients(kernel_lib, gdtype):
    """The range-sharded optimizer with fp32 state and a 16-bit gradient runs
    the mixed-precision op on its range: same bits as the op on the whole
    vector (world size 1 here; the ranges of a larger world are disjoint
    slices of the same update)."""
    from tensorflow_musa_extension_b200.cross_replica import ShardedAdam
    n = 100003
    rng = np.random.default_rng(12)
    var = rng.normal(0, 0.05, n).astype(np.float32)
    grad = rng.normal(0, 1e-3, n).astype(np_dtype(gdtype))
    h = ADAM_HYPER
    tv = to_torch(var)
    opt = ShardedAdam(tv, None, h["beta1"], h["beta2"], h["epsilon"])
    opt.step(to_torch(grad), h["lr"], h["beta1_power"], h["beta2_power"])
    wv, wm, wvv = (to_torch(a) for a in (var, np.zeros(n, np.float32), np.zeros(n, np.float32)))
    raw_ops.MusaResourceApplyAdamMixed(wv, wm, wvv, h["beta1_power"], h["beta2_power"], h["lr"],
                                       h["beta1"], h["beta2"], h["epsilon"], to_torch(grad))
    assert torch.equal(tv, wv) and torch.equal(opt.m, wm) and torch.equal(opt.v, wvv)
    # two disjoint ranges updated separately give the same bits
    a, b = to_torch(var), to_torch(var)
    cut = 50001
    for lo, hi in ((0, cut), (cut, n)):
        m0 = torch.zeros(hi - lo, device="cuda")
        v0 = torch.zeros(hi - lo, device="cuda")
        raw_ops.MusaResourceApplyAdamMixed(a[lo:hi], m0, v0, h["beta1_power"], h["beta2_power"],
                                           h["lr"], h["beta1"], h["beta2"], h["epsilon"],
                                           to_torch(grad)[lo:hi])
    assert torch.equal(a, wv)


@pytest.mark.parametrize("nesterov", [False, True])
@pytest.mark.parametrize("gdtype", ["float32", "float16", "bfloat16"])
def test_sharded_broadcast_kernel_with_mixed_gradients(kernel_lib, gdtype, nesterov):
    """LaunchAdamShardBroadcastMixed, 4 "replicas" on this GPU: fp32 state, a
    gradient of float / half / bfloat16, use_nesterov honoured - after the 4
    launches every copy equals MusaResourceApplyAdamMixed on the whole vector,
    bit for bit; an unaligned range start takes the element-wise form."""
    import ctypes
    from tensorflow_musa_extension_b200.cross_replica import aligned_shard_range
    n, world = 400_003, 4
    rng, var, m, v = adam_inputs(33, n)
    g = rng.normal(0, 1e-3, n).astype(np_dtype(gdtype))
    h = ADAM_HYPER
    want = [to_torch(t) for t in (var, m, v)]
    raw_ops.MusaResourceApplyAdamMixed(*want, h["beta1_power"], h["beta2_power"], h["lr"],
                                       h["beta1"], h["beta2"], h["epsilon"], to_torch(g),
                                       use_nesterov=nesterov)
    code = {"float32": 0, "float16": 1, "bfloat16": 2}[gdtype]
    alpha = raw_ops._adam_alpha(*[float(np.float32(h[k])) for k in
                                  ("lr", "beta1_power", "beta2_power")])
    st = torch.cuda.current_stream().cuda_stream
    f32 = lambda k: float(np.float32(h[k]))
    copies = [to_torch(var) for _ in range(world)]
    tm, tvv, tg = to_torch(m), to_torch(v), to_torch(g)
    ptrs = (ctypes.c_void_p * world)(*[c_.data_ptr() for c_ in copies])
    for r in range(world):
        lo, hi = aligned_shard_range(n, world, r)
        assert kernel_lib.LaunchAdamShardBroadcastMixed(
            code, ptrs, world, r, lo, tm[lo:hi].data_ptr(), tvv[lo:hi].data_ptr(),
            tg[lo:hi].data_ptr(), f32("beta1"), f32("beta2"), f32("epsilon"), alpha, hi - lo,
            nesterov, st) == 0
    torch.cuda.synchronize()
    for c_ in copies:
        assert torch.equal(c_, want[0])
    assert torch.equal(tm, want[1]) and torch.equal(tvv, want[2])
    one = to_torch(var)
    ptr1 = (ctypes.c_void_p * 1)(one.data_ptr())
    tm2, tv2 = to_torch(m), to_torch(v)
    assert kernel_lib.LaunchAdamShardBroadcastMixed(
        code, ptr1, 1, 0, 3, tm2[3:1000].data_ptr(), tv2[3:1000].data_ptr(),
        tg[3:1000].data_ptr(), f32("beta1"), f32("beta2"), f32("epsilon"), alpha, 997,
        nesterov, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(one[3:1000], want[0][3:1000]) and np.array_equal(to_numpy(one[:3]), var[:3])
    assert kernel_lib.LaunchAdamShardBroadcastMixed(
        7, ptr1, 1, 0, 0, tm2.data_ptr(), tv2.data_ptr(), tg.data_ptr(), 0.9, 0.999, 1e-7,
        alpha, 16, False, st) == -3


def test_fused_sharded_adam_runs_the_mixed_op(kernel_lib):
    """FusedShardedAdam with a bfloat16 gradient and use_nesterov, one replica:
    the same bits as MusaResourceApplyAdamMixed; transports that have no mixed
    form refuse."""
    from tensorflow_musa_extension_b200 import errors
    from tensorflow_musa_extension_b200.cross_replica import FusedShardedAdam, PeerVector
    n = 70_001
    rng = np.random.default_rng(8)
    var = rng.normal(0, 0.05, n).astype(np.float32)
    grad = rng.normal(0, 1e-3, n).astype(NP_BF16)
    h = ADAM_HYPER
    pv = PeerVector(None, n, torch.device("cuda", 0))
    pv.tensor.copy_(to_torch(var))
    opt = FusedShardedAdam(pv, None, h["beta1"], h["beta2"], h["epsilon"], use_nesterov=True)
    opt.step(to_torch(grad), h["lr"], h["beta1_power"], h["beta2_power"])
    wv, wm, wvv = (to_torch(a) for a in (var, np.zeros(n, np.float32), np.zeros(n, np.float32)))
    raw_ops.MusaResourceApplyAdamMixed(wv, wm, wvv, h["beta1_power"], h["beta2_power"], h["lr"],
                                       h["beta1"], h["beta2"], h["epsilon"], to_torch(grad),
                                       use_nesterov=True)
    torch.cuda.synchronize()
    assert torch.equal(pv.tensor, wv) and torch.equal(opt.m, wm) and torch.equal(opt.v, wvv)
    copies = FusedShardedAdam(pv, None, transport="copies")
    with pytest.raises(errors.InvalidArgumentError):
        copies.step(to_torch(grad), h["lr"], h["beta1_power"], h["beta2_power"])
    copies.close()


@pytest.mark.parametrize("chunks", [1, 2, 8])
def test_sharded_copy_engine_transport_on_one_gpu(kernel_lib, chunks):
    """LaunchAdamShardCopyFloat with 4 "replicas" that all live on this GPU:
    the local range is updated chunk by chunk and copy engines carry every
    finished chunk into the other copies; after the 4 shards' calls every copy
    equals the un-sharded update, bit for bit, and the caller's stream has
    joined the side streams (a plain synchronize of that stream is enough)."""
    import ctypes
    from tensorflow_musa_extension_b200.cross_replica import aligned_shard_range
    n, world = 300_003, 4
    rng, var, m, v = adam_inputs(22, n)
    g = rng.normal(0, 1e-3, n).astype(np.float32)
    want = [to_torch(t) for t in (var, m, v)]
    raw_ops.ResourceApplyAdam(*want, *_step_args(), to_torch(g))
    copies = [to_torch(var) for _ in range(world)]
    tm, tvv, tg = to_torch(m), to_torch(v), to_torch(g)
    ptrs = (ctypes.c_void_p * world)(*[c_.data_ptr() for c_ in copies])
    alpha = raw_ops._adam_alpha(*[float(np.float32(H[k])) for k in
                                  ("lr", "beta1_power", "beta2_power")])
    stream = torch.cuda.Stream()
    pipes = [kernel_lib.MusaShardPipeCreate(world, r) for r in range(world)]
    assert all(pipes)
    with torch.cuda.stream(stream):
        stream.wait_stream(torch.cuda.default_stream())
        for r in range(world):
            lo, hi = aligned_shard_range(n, world, r)
            rc = kernel_lib.LaunchAdamShardCopyFloat(
                pipes[r], ptrs, lo, tm[lo:hi].data_ptr(), tvv[lo:hi].data_ptr(),
                tg[lo:hi].data_ptr(), float(np.float32(H["beta1"])),
                float(np.float32(H["beta2"])), float(np.float32(H["epsilon"])), alpha, hi - lo,
                chunks, stream.cuda_stream)
            assert rc == 0
    stream.synchronize()
    for c_ in copies:
        assert torch.equal(c_, want[0])
    assert torch.equal(tm, want[1]) and torch.equal(tvv, want[2])
    for p in pipes:
        kernel_lib.MusaShardPipeDestroy(p)
    assert kernel_lib.MusaShardPipeCreate(0, 0) is None
    assert kernel_lib.MusaShardPipeCreate(4, 4) is None


def test_multicast_transport_refuses_what_it_cannot_run(kernel_lib):
    """LaunchAdamShardMulticastFloat needs whole 128-bit packs (range start on
    a pack, aligned pointers) and both addresses; anything else is refused
    before a kernel is launched.  (The transport itself needs two GPUs behind
    one NVSwitch: `bench.py --gpus N --adam-multicast` checks it against the
    oracle.)"""
    t = torch.zeros(64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = (0.9, 0.999, 1e-7, 1e-3)
    f = kernel_lib.LaunchAdamShardMulticastFloat
    assert f(t.data_ptr(), None, 0, t.data_ptr(), t.data_ptr(), t.data_ptr(), *args, 16, st) == -1
    assert f(t.data_ptr(), t.data_ptr(), 2, t.data_ptr(), t.data_ptr(), t.data_ptr(), *args, 16,
             st) == -1
    assert f(t.data_ptr(), t.data_ptr(), 0, t.data_ptr() + 4, t.data_ptr(), t.data_ptr(), *args,
             16, st) == -1
    assert f(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), t.data_ptr(), *args, 0,
             st) == 0
    torch.cuda.synchronize()
    assert not t.any()
