"""The native core under the host sanitizers: a stand-alone program (csrc/core/selftest.cpp) that drives the
codec, IR, partitioner, stage search, deployment, batch arithmetic and the thread-owning utilities is built with
AddressSanitizer + UndefinedBehaviorSanitizer and with ThreadSanitizer, and must finish without a report."""
import subprocess

import pytest


@pytest.mark.parametrize("sanitize", ["address,undefined", "thread"])
def test_native_core_selftest_is_clean_under(sanitize):
    from rannc_b200 import build

    exe = build.build_selftest(sanitize)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "selftest ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    assert "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-4000:]
