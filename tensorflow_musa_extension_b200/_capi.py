"""ctypes prototypes of every entry point declared in
include/musa_plugin_kernels.h.  `bind()` attaches argtypes/restype to a loaded
library and fails loudly if a symbol is missing."""
import ctypes

c_i64 = ctypes.c_int64
c_f32 = ctypes.c_float
c_f64 = ctypes.c_double
c_vp = ctypes.c_void_p
c_int = ctypes.c_int
c_bool = ctypes.c_bool
c_size = ctypes.c_size_t

_ADAM_SAME = [c_vp, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32, c_i64, c_bool, c_vp]
_BIAS_ACT = [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_int, c_vp]
_NADAM = [c_vp, c_vp, c_vp, c_vp] + [c_f32] * 6 + [c_i64, c_vp]
_RMSPROP = [c_vp, c_vp, c_vp, c_vp] + [c_f64] * 4 + [c_i64, c_vp]
_CRMSPROP = [c_vp] * 5 + [c_f64] * 4 + [c_i64, c_vp]
_SGD = [c_vp, c_vp, c_f32, c_i64, c_vp]
_ADAGRAD = [c_vp, c_vp, c_vp, c_f64, c_f64, c_bool, c_i64, c_vp]
_SGD_TABLE = [c_vp] * 5 + [c_int, c_int, c_vp]
_LAYER_NORM = [c_vp] * 6 + [c_i64, c_i64, c_f32, c_vp]
_LAYER_NORM_GRAD = [c_vp] * 6 + [c_i64, c_i64, c_f32, c_vp, c_size, c_vp]
_RMS_NORM = [c_vp] * 5 + [c_i64, c_i64, c_f32, c_vp]
_RMS_NORM_GRAD = [c_vp] * 5 + [c_i64, c_i64, c_vp]
_BIAS_GRAD = [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]
_RELU_GRAD = [c_vp, c_vp, c_vp, c_i64, c_vp]
_BIAS_RELU_GRAD = [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]
_BN_TRAIN = [c_vp] * 10 + [c_i64, c_i64, c_i64, c_f32, c_f32, c_vp, c_size, c_vp]
_BN_INFER = [c_vp] * 6 + [c_i64, c_i64, c_i64, c_f32, c_vp]
_BN_GRAD = [c_vp] * 8 + [c_i64, c_i64, c_i64, c_f32, c_bool, c_vp, c_size, c_vp]

# name -> (restype, argtypes)
PROTOTYPES = {
    "MusaKernelsVersion": (ctypes.c_char_p, []),
    "MusaKernelsTargetArch": (c_int, []),
    "LaunchResourceApplyAdamFloat":
        (None, [c_vp, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32, c_i64, c_vp]),
    "LaunchApplyAdamSameType_BFloat16": (None, _ADAM_SAME),
    "LaunchApplyAdamSameType_Half": (None, _ADAM_SAME),
    "LaunchApplyAdamMixed_Float": (None, _ADAM_SAME),
    "LaunchApplyAdamMixed_Half": (None, _ADAM_SAME),
    "LaunchApplyAdamMixed_BFloat16": (None, _ADAM_SAME),
    "LaunchApplyAdam_F64": (None, [c_vp, c_vp, c_vp, c_vp, c_f64, c_f64, c_f64, c_f64,
                                   c_i64, ctypes.c_bool, c_vp]),
    "LaunchBiasAct_F32": (c_int, _BIAS_ACT),
    "LaunchBiasAct_F16": (c_int, _BIAS_ACT),
    "LaunchBiasAct_BF16": (c_int, _BIAS_ACT),
    "LaunchBiasAct_F64": (c_int, _BIAS_ACT),
    "LaunchBiasAct_I32": (c_int, _BIAS_ACT),
    "LaunchBiasAct_I64": (c_int, _BIAS_ACT),
    "LaunchResourceApplyNadam_Float": (None, _NADAM),
    "LaunchFusedResourceApplyRMSProp_Float": (None, _RMSPROP),
    "LaunchFusedResourceApplyCenteredRMSProp_Float": (None, _CRMSPROP),
    "LaunchResourceApplyNadam_Half": (None, _NADAM),
    "LaunchFusedResourceApplyRMSProp_Half": (None, _RMSPROP),
    "LaunchFusedResourceApplyCenteredRMSProp_Half": (None, _CRMSPROP),
    "LaunchResourceApplyNadam_BFloat16": (None, _NADAM),
    "LaunchFusedResourceApplyRMSProp_BFloat16": (None, _RMSPROP),
    "LaunchFusedResourceApplyCenteredRMSProp_BFloat16": (None, _CRMSPROP),
    "LaunchResourceApplyNadam_Double": (None, _NADAM),
    "LaunchFusedResourceApplyRMSProp_Double": (None, _RMSPROP),
    "LaunchFusedResourceApplyCenteredRMSProp_Double": (None, _CRMSPROP),
    "LaunchFusedApplyAdagradV2_Float": (None, _ADAGRAD),
    "LaunchFusedApplyAdagradV2_Half": (None, _ADAGRAD),
    "LaunchFusedApplyAdagradV2_BFloat16": (None, _ADAGRAD),
    "LaunchFusedApplyAdagradV2_Double": (None, _ADAGRAD),
    "LaunchResourceApplyGradientDescentFloat": (None, _SGD),
    "LaunchResourceApplyGradientDescentFloatBFloat16": (None, _SGD),
    "LaunchResourceApplyGradientDescent_Half": (None, _SGD),
    "LaunchResourceApplyGradientDescent_BFloat16": (None, _SGD),
    "LaunchGroupedResourceApplyGradientDescentFloat": (None, _SGD_TABLE),
    "LaunchGroupedResourceApplyGradientDescentFloatBFloat16": (None, _SGD_TABLE),
    "LaunchGroupedGradientDescentHostTable":
        (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "LaunchLayerNorm_F32": (c_int, _LAYER_NORM),
    "LaunchLayerNorm_F16": (c_int, _LAYER_NORM),
    "LaunchLayerNorm_BF16": (c_int, _LAYER_NORM),
    "LayerNormGradWorkspaceBytes": (c_size, [c_i64, c_i64]),
    "LaunchLayerNormGrad_F32": (c_int, _LAYER_NORM_GRAD),
    "LaunchLayerNormGrad_F16": (c_int, _LAYER_NORM_GRAD),
    "LaunchLayerNormGrad_BF16": (c_int, _LAYER_NORM_GRAD),
    "LaunchRmsNormFloat": (None, _RMS_NORM),
    "LaunchRmsNormBFloat16": (None, _RMS_NORM),
    "LaunchRmsNormGradDxFloat": (None, _RMS_NORM_GRAD),
    "LaunchRmsNormGradDxBFloat16": (None, _RMS_NORM_GRAD),
    "BiasGradWorkspaceBytes": (c_size, [c_i64, c_i64, c_i64, c_int]),
    "LaunchBiasAddGrad_F32": (c_int, _BIAS_GRAD),
    "LaunchBiasAddGrad_F16": (c_int, _BIAS_GRAD),
    "LaunchBiasAddGrad_BF16": (c_int, _BIAS_GRAD),
    "LaunchBiasAddGrad_F64": (c_int, _BIAS_GRAD),
    "LaunchBiasAddGrad_I32": (c_int, _BIAS_GRAD),
    "LaunchBiasAddGrad_I64": (c_int, _BIAS_GRAD),
    "LaunchReluGrad_F32": (c_int, _RELU_GRAD),
    "LaunchReluGrad_F16": (c_int, _RELU_GRAD),
    "LaunchReluGrad_BF16": (c_int, _RELU_GRAD),
    "LaunchBiasAddReluGrad_F32": (c_int, _BIAS_RELU_GRAD),
    "LaunchBiasAddReluGrad_F16": (c_int, _BIAS_RELU_GRAD),
    "LaunchBiasAddReluGrad_BF16": (c_int, _BIAS_RELU_GRAD),
    "BnWorkspaceBytes": (c_size, [c_i64, c_i64, c_i64]),
    "LaunchBnFwdTrain_F32": (c_int, _BN_TRAIN),
    "LaunchBnFwdTrain_F16": (c_int, _BN_TRAIN),
    "LaunchBnFwdTrain_BF16": (c_int, _BN_TRAIN),
    "LaunchBnFwdInfer_F32": (c_int, _BN_INFER),
    "LaunchBnFwdInfer_F16": (c_int, _BN_INFER),
    "LaunchBnFwdInfer_BF16": (c_int, _BN_INFER),
    "LaunchBnGrad_F32": (c_int, _BN_GRAD),
    "LaunchBnGrad_F16": (c_int, _BN_GRAD),
    "LaunchBnGrad_BF16": (c_int, _BN_GRAD),
    "BnNoAllocMaxChannels": (c_size, []),
    "LaunchBnFwdTrainNoAlloc":
        (c_int, [c_int] + [c_vp] * 10 + [c_i64, c_i64, c_i64, c_f32, c_f32, c_vp]),
    "LaunchBesselCorrection": (None, [c_vp, c_f32, c_int, c_vp]),
    "LaunchVarianceToInvStd": (None, [c_vp, c_vp, c_f32, c_int, c_vp]),
    "LaunchBnStatsSums":
        (c_int, [c_int, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]),
    "LaunchBnStatsSumsCount":
        (c_int, [c_int, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]),
    "LaunchBnApplyFromSums":
        (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_f64, c_vp, c_vp, c_f32, c_vp,
                 c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_f32, c_vp]),
    "LaunchBnStatsMoments":
        (c_int, [c_int, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]),
    "LaunchBnMergeMoments": (c_int, [c_vp, c_int, c_i64, c_vp, c_vp]),
    "LaunchBnApplyFromMoments":
        (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_f64, c_vp, c_vp, c_f32, c_vp,
                 c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_f32, c_vp]),
    "LaunchBnFinalizeFromSums":
        (c_int, [c_vp, c_f64] + [c_vp] * 6 + [c_i64, c_f32, c_vp]),
    "LaunchBnApply":
        (c_int, [c_int] + [c_vp] * 6 + [c_i64, c_i64, c_i64, c_f32, c_vp]),
    "LaunchBnGradStatsSums":
        (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp]),
    "LaunchBnGradApplyFromSums":
        (c_int, [c_int] + [c_vp] * 6 + [c_f64] + [c_vp] * 3
         + [c_i64, c_i64, c_i64, c_f32, c_vp]),
}

PROTOTYPES.update({
    "MusaExchangeCreate": (c_vp, [c_int, c_int, c_i64]),
    "MusaExchangeIpcHandle": (c_int, [c_vp, c_vp]),
    "MusaExchangeOpenPeers": (c_int, [c_vp, c_vp]),
    "LaunchExchangeSums": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "MusaExchangeStatus": (c_int, [c_vp]),
    "MusaExchangeDestroy": (None, [c_vp]),
    "LaunchExchangeMoments": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "LaunchBnStatsMomentsExchange":
        (c_int, [c_int, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp, c_vp]),
    "LaunchBnGradStatsSumsExchange":
        (c_int, [c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_size, c_vp,
                 c_vp]),
    "MusaExchangeSelfTest": (c_int, [c_int, c_i64, c_vp, c_int, c_int, c_int, c_vp]),
    "MusaPeerAlloc": (c_vp, [c_i64]),
    "MusaPeerFree": (c_int, [c_vp]),
    "MusaPeerIpcHandle": (c_int, [c_vp, c_vp]),
    "MusaPeerOpen": (c_vp, [c_vp]),
    "MusaPeerClose": (c_int, [c_vp]),
    "MusaPeerCopyAsync": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "LaunchAdamShardBroadcastFloat":
        (c_int, [c_vp, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32,
                 c_i64, c_vp]),
    "LaunchAdamShardBroadcastMixed":
        (c_int, [c_int, c_vp, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32,
                 c_i64, c_bool, c_vp]),
    "LaunchAdamShardMulticastFloat":
        (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32, c_i64, c_vp]),
    "MusaShardPipeCreate": (c_vp, [c_int, c_int]),
    "MusaShardPipeDestroy": (None, [c_vp]),
    "LaunchAdamShardCopyFloat":
        (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32, c_i64,
                 c_int, c_vp]),
})

# Hooks outside the reference boundary: launch-shape sweeps and tracing.
class MusaLaunchCounter(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("calls", ctypes.c_longlong),
                ("bytes", ctypes.c_longlong), ("host_ns", ctypes.c_longlong),
                ("kernels", ctypes.c_longlong)]


PROTOTYPES.update({
    "MusaKernelsSetTuning": (c_int, [c_int, c_int]),
    "MusaKernelsGetTuning": (c_int, [c_int]),
    "MusaKernelsTraceEnable": (c_int, [c_int]),
    "MusaKernelsTraceSnapshot": (c_int, [ctypes.POINTER(MusaLaunchCounter), c_int]),
    "MusaKernelsTraceReset": (None, []),
    "MusaKernelsLaunchCount": (ctypes.c_longlong, []),
})
EXTRA_PROTOTYPES = {}


def trace_snapshot(lib):
    """{launcher: {"calls", "bytes", "host_ns", "kernels"}} of the tracing counters."""
    n = lib.MusaKernelsTraceSnapshot(None, 0)
    buf = (MusaLaunchCounter * max(n, 1))()
    n = lib.MusaKernelsTraceSnapshot(buf, n)
    return {buf[i].name.decode(): {"calls": buf[i].calls, "bytes": buf[i].bytes,
                                   "host_ns": buf[i].host_ns, "kernels": buf[i].kernels}
            for i in range(n)}

# Entry points of include/musa_plugin_runtime.h that the staging pipeline
# drives (streams, events, asynchronous copies, the pinned pool).
c_u64 = ctypes.c_uint64
_P_VP = ctypes.POINTER(c_vp)
RUNTIME_PROTOTYPES = {
    "MusaRtLastError": (ctypes.c_char_p, []),
    "MusaRtCreateDevice": (c_int, [c_int]),
    "MusaRtCreateStream": (c_int, [c_int, _P_VP]),
    "MusaRtDestroyStream": (c_int, [c_int, c_vp]),
    "MusaRtRawStream": (c_vp, [c_vp]),
    "MusaRtCreateEvent": (c_int, [c_int, _P_VP]),
    "MusaRtDestroyEvent": (c_int, [c_int, c_vp]),
    "MusaRtRecordEvent": (c_int, [c_int, c_vp, c_vp]),
    "MusaRtGetEventStatus": (c_int, [c_int, c_vp]),
    "MusaRtWaitForEvent": (c_int, [c_int, c_vp, c_vp]),
    "MusaRtBlockHostForEvent": (c_int, [c_int, c_vp]),
    "MusaRtBlockHostUntilDone": (c_int, [c_int, c_vp]),
    "MusaRtMemcpyDtoH": (c_int, [c_int, c_vp, c_vp, c_vp, c_u64]),
    "MusaRtMemcpyHtoD": (c_int, [c_int, c_vp, c_vp, c_vp, c_u64]),
    "MusaRtPinnedAllocate": (c_vp, [c_int, c_u64]),
    "MusaRtPinnedFreeAsync": (c_int, [c_int, c_vp, c_u64, c_vp]),
}

ERROR_NAMES = {
    -1: "invalid argument (null pointer or negative size)",
    -2: "workspace missing, misaligned or too small",
    -3: "unsupported dtype or activation code",
    -4: "size beyond what the entry point holds",
}


def bind(lib):
    """Attach prototypes; AttributeError names the first missing symbol."""
    for table in (PROTOTYPES, EXTRA_PROTOTYPES, RUNTIME_PROTOTYPES):
        for name, (restype, argtypes) in table.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
    return lib
