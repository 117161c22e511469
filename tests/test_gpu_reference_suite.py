"""The reference project's own test files, run UNCHANGED against this package.

`__graft_entry__.build()` copies them (when a reference checkout is available at build time)
into the git-ignored `baseline/_ref/tests`; here they run in a child pytest whose import path
holds this package's `custom`, `models` and `backend`, exactly where the reference's tests
expect their own.  The only addition is a conftest of ours that seeds torch per test (the
reference's tests draw unseeded inputs against tolerances a few draws in a thousand exceed).
Skipped when the files were not staged."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITE = os.path.join(ROOT, "baseline", "_ref", "tests")


@pytest.mark.skipif(not os.path.isfile(os.path.join(SUITE, "test_custom_linear.py")),
                    reason="reference test files were not staged at build time")
def test_reference_tests_pass_unchanged():
    env = dict(os.environ)
    env["PYTHONPATH"] = os.path.join(ROOT, "fp4-training_b200") + os.pathsep + env.get("PYTHONPATH", "")
    out = subprocess.run([sys.executable, "-m", "pytest", SUITE, "-q", "-p", "no:cacheprovider",
                          "--rootdir", SUITE, "-c", os.devnull],
                         capture_output=True, text=True, timeout=1500, cwd=SUITE, env=env)
    tail = (out.stdout + out.stderr)[-3000:]
    assert out.returncode == 0, "the reference's tests failed against this package:\n" + tail
    assert " passed" in out.stdout, tail
