"""The C-ABI library loads without a GPU and exports every symbol that
include/musa_plugin_kernels.h declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "musa_plugin_kernels.h")
ALL_HEADERS = [os.path.join(ROOT, "include", n)
               for n in ("musa_plugin_kernels.h", "musa_plugin_graph.h",
                         "musa_plugin_runtime.h")]


def declared_functions(header=HEADER):
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_expected_families():
    names = declared_functions()
    for must in ("LaunchResourceApplyAdamFloat", "LaunchApplyAdamSameType_BFloat16",
                 "LaunchApplyAdamMixed_Half", "LaunchBiasAct_F16",
                 "LaunchBnFwdTrain_BF16", "LaunchBnGrad_F16", "BnWorkspaceBytes",
                 "LaunchBnStatsSums", "LaunchBnGradApplyFromSums",
                 "LaunchBesselCorrection", "LaunchVarianceToInvStd"):
        assert must in names
    assert len(names) >= 30


def test_library_exports_every_declared_symbol(kernel_lib):
    total = 0
    for header in ALL_HEADERS:
        names = declared_functions(header)
        assert names, header
        for name in names:
            assert hasattr(kernel_lib, name), "missing export: %s (%s)" % (name, header)
        total += len(names)
    assert total >= 90


def test_prototype_table_covers_the_header(kernel_lib):
    from tensorflow_musa_extension_b200 import _capi
    assert set(declared_functions()) <= set(_capi.PROTOTYPES) | set(_capi.EXTRA_PROTOTYPES)
    assert set(_capi.PROTOTYPES) <= set(declared_functions())


def test_identity_and_pure_host_queries(kernel_lib):
    assert kernel_lib.MusaKernelsTargetArch() == 100
    assert b"sm_100a" in kernel_lib.MusaKernelsVersion()
    # Workspace sizing is host arithmetic: positive, bounded, zero when empty.
    n = kernel_lib.BnWorkspaceBytes(256 * 28 * 28, 256, 1)
    assert 0 < n <= 8 << 20
    assert kernel_lib.BnWorkspaceBytes(0, 64, 1) == 0
    assert kernel_lib.BnWorkspaceBytes(-1, 64, 1) == 0
    big = kernel_lib.BnWorkspaceBytes(256 * 7 * 7, 2048, 1)
    assert 0 < big <= 8 << 20


def test_argument_errors_need_no_device(kernel_lib):
    # Refused before any CUDA call: negative sizes and unknown codes.
    assert kernel_lib.LaunchBiasAct_F32(None, None, None, -1, 4, 1, 0, None) == -1
    assert kernel_lib.LaunchBiasAct_F32(None, None, None, 0, 4, 1, 0, None) == 0
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert kernel_lib.LaunchBiasAct_F32(p, p, p, 1, 4, 1, 99, None) == -3
    assert kernel_lib.LaunchBnStatsSums(7, p, p, 2, 4, 1, p, 64, None) == -3
    assert kernel_lib.LaunchBnFwdTrain_F32(p, p, p, None, None, p, p, p, p, p, 2, 4, 1,
                                           1e-3, 1.0, None, 0, None) == -2
    assert kernel_lib.LaunchBnFwdTrain_F32(p, p, p, None, None, p, p, p, p, p, 2, 4, 1,
                                           1e-3, 0.5, p, 1 << 20, None) == -1


def test_tuning_hook_round_trip(kernel_lib):
    old = kernel_lib.MusaKernelsGetTuning(1)
    assert kernel_lib.MusaKernelsSetTuning(1, 4) == old
    assert kernel_lib.MusaKernelsGetTuning(1) == 4
    kernel_lib.MusaKernelsSetTuning(1, old)
    assert kernel_lib.MusaKernelsSetTuning(999, 1) == -1


def test_loader_reports_search_locations(monkeypatch, tmp_path):
    from tensorflow_musa_extension_b200 import _loader
    monkeypatch.setattr(_loader, "PLUGIN_LIBRARY", "libdoes_not_exist.so")
    monkeypatch.setenv("LD_LIBRARY_PATH", str(tmp_path))
    with pytest.raises(FileNotFoundError) as e:
        _loader._find_plugin_library()
    msg = str(e.value)
    assert "Searched locations" in msg and str(tmp_path) in msg
    assert "/usr/local/musa/lib" in msg


def test_loader_finds_library_on_ld_library_path(monkeypatch, tmp_path):
    from tensorflow_musa_extension_b200 import _loader
    fake = tmp_path / "libfake_plugin.so"
    fake.write_bytes(b"")
    monkeypatch.setattr(_loader, "PLUGIN_LIBRARY", "libfake_plugin.so")
    monkeypatch.setenv("LD_LIBRARY_PATH", str(tmp_path))
    assert _loader._find_plugin_library() == str(fake)


def test_launcher_tracing_counts_calls_and_bytes(kernel_lib):
    """Tracing is off unless asked for; switched on, every launcher call adds
    to its counters (calls, algorithmic bytes).  Calls that return before any
    CUDA work (empty inputs) are enough to see that without a device."""
    from tensorflow_musa_extension_b200 import _capi
    was = kernel_lib.MusaKernelsTraceEnable(0)
    kernel_lib.MusaKernelsTraceReset()
    assert kernel_lib.LaunchBiasAct_F32(None, None, None, 0, 4, 1, 0, None) == 0
    before = _capi.trace_snapshot(kernel_lib)
    assert all(v["calls"] == 0 for v in before.values())        # off: nothing counted
    kernel_lib.MusaKernelsTraceEnable(1)
    try:
        for _ in range(3):
            assert kernel_lib.LaunchBiasAct_F32(None, None, None, 0, 4, 1, 0, None) == 0
        kernel_lib.LaunchRmsNormFloat(None, None, None, None, None, 0, 128, 1e-5, None)
        snap = _capi.trace_snapshot(kernel_lib)
        assert snap["LaunchBiasAct"]["calls"] == 3 and snap["LaunchBiasAct"]["bytes"] == 0
        assert snap["LaunchRmsNorm"]["calls"] == 1
        assert snap["LaunchBiasAct"]["host_ns"] >= 0
        assert snap["LaunchBiasAct"]["kernels"] == 0             # empty inputs launch nothing
        kernel_lib.MusaKernelsTraceReset()
        assert _capi.trace_snapshot(kernel_lib)["LaunchBiasAct"]["calls"] == 0
    finally:
        kernel_lib.MusaKernelsTraceEnable(was)
