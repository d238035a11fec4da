"""The library inside a driver context created by the caller, in a process of its own (a device
serves one context per process, and the other tests of this run use the primary context)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_adopts_the_callers_driver_context(gpu):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ctx_adopt_worker.py")
    r = subprocess.run([sys.executable, worker], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), (r.stdout[-2000:], r.stderr[-2000:])
