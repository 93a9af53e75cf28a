"""The device-side status path for a wait that gave up (WE_B200_ST_WAIT_EXPIRED), without hurting the GPU: the
debug build of the library can make the first CTA of an unsplit launch wait, with a limit of one millisecond, on
a barrier nobody arrives on -- before that CTA has issued any copy or product, so nothing is in flight when the
wait runs out -- after which the CTA takes the exit every aborting CTA takes (status word, tear-down, tensor
memory freed).  Checked: the status word reads WAIT_EXPIRED, `ops.check_status` raises and clears it, and the
next ordinary call on the same context is correct.  Runs in a child process because the debug build is a
separate shared object (the library is loaded once per process)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_expired_wait_sets_the_status_word_and_leaves_the_context_usable():
    from world_engine_b200.csrc import build
    lib = build.build(debug=True)                      # (built in-tree if it is not there yet)
    env = dict(os.environ, WE_B200_LIB=lib)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "expired_wait_child.py")], env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert "CLEAN_BEFORE ok" in lines
    assert "STATUS 1" in lines, r.stdout            # WE_B200_ST_WAIT_EXPIRED
    assert "RAISED yes: True" in lines
    assert "CLEARED 0" in lines
    assert "AFTER ok" in lines and "STATE ok" in lines
