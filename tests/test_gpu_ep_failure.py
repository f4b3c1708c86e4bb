"""Failure detection of the library's own NCCL path, with the failure made on the host: a test double of NCCL
(tests/cpp/fake_nccl.c) reports an asynchronous error, or a host function keeps the stream busy past the timeout.
No kernel waits, faults or hangs: the device is idle while the host-side wait runs out."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _fake_nccl() -> Path:
    out = ROOT / "tests" / "cpp" / "_build" / "libfake_nccl.so"
    src = ROOT / "tests" / "cpp" / "fake_nccl.c"
    if not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        out.parent.mkdir(exist_ok=True)
        subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-o", str(out), str(src)], check=True)
    return out


def _run(scenario: str, extra_env: dict) -> dict:
    env = dict(os.environ)
    env["NVMAI_CUDA_NCCL_LIB"] = str(_fake_nccl())
    env["NVMAI_CUDA_NVTX"] = "1"           # the host-side ranges run too (without a profiler they record nothing)
    env.update(extra_env)
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "ep_failure_child.py"), scenario], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])


def test_async_nccl_error_aborts_the_communicator_and_the_handle_recovers():
    from nvmai_b200 import _lib
    out = _run("async_error", {})
    assert out["code"] == _lib.ENCCL and out["aborts"] == 1
    assert out["waited_s"] < 2.0            # found by polling, long before the 5 s limit
    assert out["after"] == _lib.EINVAL and out["recovered"]


def test_host_timeout_aborts_a_step_that_does_not_finish():
    from nvmai_b200 import _lib
    out = _run("timeout", {})
    assert out["code"] == _lib.ETIMEOUT and out["aborts"] == 1
    assert 0.1 < out["waited_s"] < 2.0
    assert out["after"] == _lib.EINVAL and out["recovered"]
