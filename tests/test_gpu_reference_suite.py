"""The reference's own asc2 test-suite, unmodified, on the CUDA platform.

``ASC2_REFERENCE_TESTS`` names a directory holding the reference project's ``python/test/asc2`` tree (its
``conftest.py``, ``kernels/`` and ``operations/``, exactly as the reference ships them).  The suite is run in a
child pytest with this package's ``asc`` / ``asc2`` first on ``PYTHONPATH`` and one option of the reference's
conftest (python/test/asc2/conftest.py:27-33) changed from its default: ``--backend CUDA``.  ``--platform`` keeps
the reference's default (an Ascend 950 part); ``set_platform`` on the CUDA back end takes the device it finds, and
the tests the reference guards with ``require_c310`` (conftest.py:62-69: features of that Ascend generation, such
as 1-D softmax and most operation tests) therefore run instead of being skipped.  The reference's files are not
part of this repository, so without the variable the test is skipped.

What has to hold: every test of the reference passes, none fails, none is skipped.
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

PKG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "pyasc_b200")


def run_reference_suite(ref_dir: str, extra=()):
    env = dict(os.environ)
    env["PYTHONPATH"] = PKG_DIR + os.pathsep + env.get("PYTHONPATH", "")
    env.pop("DRY_RUN", None)
    cmd = [sys.executable, "-m", "pytest", ref_dir, "--backend", "CUDA", "--import-mode=importlib",
           "-p", "no:cacheprovider", "-q", "-rfEs", "--no-header", *extra]
    # cwd outside this repository: its tests/conftest.py must not be picked up next to the reference's own
    proc = subprocess.run(cmd, env=env, cwd=ref_dir, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=3000)
    counts = {k: 0 for k in ("passed", "failed", "skipped", "error", "errors")}
    tail = proc.stdout.strip().splitlines()[-1] if proc.stdout.strip() else ""
    for n, key in re.findall(r"(\d+) (passed|failed|skipped|errors?)", tail):
        counts[key] = int(n)
    counts["error"] += counts.pop("errors")
    return proc, counts


def test_reference_asc2_suite_passes_unmodified():
    ref_dir = os.environ.get("ASC2_REFERENCE_TESTS")
    if not ref_dir or not os.path.isdir(os.path.join(ref_dir, "kernels")):
        pytest.skip("ASC2_REFERENCE_TESTS does not name the reference's python/test/asc2 directory")
    proc, counts = run_reference_suite(os.path.abspath(ref_dir))
    report = os.environ.get("ASC2_REFERENCE_REPORT")
    if report:
        with open(report, "w") as f:
            f.write(proc.stdout)
    summary = "\n".join(proc.stdout.splitlines()[-60:])
    assert counts["failed"] == 0 and counts["error"] == 0 and counts["skipped"] == 0, summary
    assert counts["passed"] >= 240, summary            # 10 kernel files + 8 operation files, parametrised
    assert proc.returncode == 0, summary
