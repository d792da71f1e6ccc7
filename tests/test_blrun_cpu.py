# SPDX-License-Identifier: MIT
"""The blrun launcher without a GPU: it starts N ranks with the torchrun-style
environment, the payload runs with no ambient capabilities and no_new_privs,
the ranks form a "barlink" group (CPU tensors over gloo), and a failing rank's
exit code comes back while the other ranks are taken down."""
import os
import shutil
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PAYLOAD = os.path.join(ROOT, "tests", "_blrun_payload.py")


@pytest.fixture(scope="module")
def blrun(tmp_path_factory):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    # the launcher finds the repository as the parent of its own directory
    d = tmp_path_factory.mktemp("repo") / "tools"
    d.mkdir()
    exe = d / "blrun"
    subprocess.check_call([cc, "-O2", "-Wall", "-o", str(exe), os.path.join(ROOT, "tools", "blrun.c")])
    os.symlink(os.path.join(ROOT, "barlink_sm86_b200"), d.parent / "barlink_sm86_b200")
    return str(exe)


def _env():
    env = dict(os.environ, BL_PYTHON=sys.executable, BL_CPU_ONLY="1")
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    return env


def test_two_ranks_form_a_group_without_capabilities(blrun):
    p = subprocess.run([blrun, "-n", "2", PAYLOAD], env=_env(), capture_output=True, text=True, timeout=180)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "payload rank 0 of 2 ok" in p.stdout and "payload rank 1 of 2 ok" in p.stdout


def test_a_failing_rank_ends_the_job_with_its_exit_code(blrun):
    t0 = time.time()
    p = subprocess.run([blrun, "-n", "2", PAYLOAD, "fail"], env=_env(), capture_output=True, text=True, timeout=120)
    assert p.returncode == 5, (p.returncode, p.stdout + p.stderr)
    assert time.time() - t0 < 45  # rank 0 did not sleep out its 60 s


def test_bad_arguments(blrun):
    assert subprocess.run([blrun], capture_output=True).returncode == 2
    assert subprocess.run([blrun, "-n", "9", PAYLOAD], capture_output=True, env=_env()).returncode == 2
    env = dict(_env(), BL_DEVICES="0")
    assert subprocess.run([blrun, "-n", "2", PAYLOAD], capture_output=True, env=env).returncode == 2
