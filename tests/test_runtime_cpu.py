"""The device runtime (stream-executor callbacks, registry, event manager,
pinned bounce pool) on the host-only driver: no GPU needed.  One subprocess per
case, as the reference isolates its runtime tests
(test/ops/pluggable_se_api_test.py:50-343)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

CASES = ["identity_and_init", "device_enumeration", "registry_lifecycle",
         "streams_and_copies", "pageable_bounce",
         "pinned_pool_reuse_waits_for_the_stream", "event_manager", "stream_dependency",
         "events_and_timers", "concurrent_pool_and_copies"]


@pytest.mark.parametrize("case", CASES)
def test_runtime_case(kernel_lib, case):
    env = {k: v for k, v in os.environ.items()
           if not k.startswith("MUSA_SE_") and k not in (
               "MUSA_STRICT_DEVICE_ENUM", "TENSORFLOW_MUSA_USE_LEGACY_DEVICE")}
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "runtime_fake_worker.py"),
                        case], env=env, capture_output=True, text=True, timeout=180)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "case ok: " + case in p.stdout


def test_every_case_is_listed():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    src = open(os.path.join(ROOT, "tests", "runtime_fake_worker.py")).read()
    import re
    assert sorted(re.findall(r"^def case_(\w+)", src, re.M)) == sorted(CASES)
