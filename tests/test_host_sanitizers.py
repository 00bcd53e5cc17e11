"""The host runtime under ThreadSanitizer and AddressSanitizer + UBSan.

A native program (``parameter_server_b200/csrc/host/selftest``) runs a 1 + 2 + 2 node cluster over the
in-process van with several application threads per worker: membership, concurrent pushes, pulls that
wait for a push, heartbeats, the failure detector, shutdown.  A sanitizer finding makes it exit non-zero.
"""
import os
import subprocess

import pytest

from parameter_server_b200.utils import build


@pytest.mark.parametrize("van", ["inproc", "tcp"])
@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_host_runtime_under_sanitizer(sanitizer, van, tmp_path):
    exe = build.build_host_selftest(sanitizer)
    if exe is None:
        pytest.skip(f"compiler has no -fsanitize={sanitizer}")
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67",
               UBSAN_OPTIONS="halt_on_error=1 exitcode=68")
    r = subprocess.run([str(exe)] + ["tcp" if van == "tcp" else "inproc", str(tmp_path)], capture_output=True, text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert "): ok" in out
    assert "ThreadSanitizer" not in out and "AddressSanitizer" not in out and "runtime error" not in out, out[-4000:]
