# SPDX-License-Identifier: MIT
"""Multi-GPU tests: one process per GPU over the link (needs >= 2 GPUs)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_ranks(script, world, timeout=600, extra_env=None):
    port = _free_port()
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    env.update(extra_env or {})
    env.setdefault("BL_PG_ID", "t%d" % port)
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, script), str(r), str(world), str(port)],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outs = []
    ok = True
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            ok = False
        outs.append(out)
        ok = ok and p.returncode == 0
    text = "\n".join("--- rank %d ---\n%s" % (i, o) for i, o in enumerate(outs))
    assert ok, text
    return text


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_process_group_over_the_link(world):
    if world not in _worlds():
        pytest.skip("needs %d GPUs" % world)
    print(_run_ranks("_pg_worker.py", world))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_process_group_with_in_switch_reduction(world):
    """The same worker with the arenas bound to an NVSwitch multicast object (BL_NVLS=1): the
    multimem all-reduce is exercised bit-exactly; the worker leaves out its timed-out-wait case
    and every rank exits through barrier -> shutdown."""
    if world not in _worlds():
        pytest.skip("needs %d GPUs" % world)
    out = _run_ranks("_pg_worker.py", world, extra_env={"BL_NVLS": "1"})
    print(out)
    if "multicast=True" in out:
        assert "nvls large messages ok" in out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_model(world):
    if world not in _worlds():
        pytest.skip("needs %d GPUs" % world)
    print(_run_ranks("_tp_worker.py", world))


@pytest.mark.parametrize("world", [2, 4])
def test_single_process_mode_on_real_gpus(world):
    """One process drives N GPUs (the reference's original mode: bl.init(devices, pool_mb))."""
    if world not in _worlds():
        pytest.skip("needs %d GPUs" % world)
    import subprocess
    import sys
    p = subprocess.run([sys.executable, os.path.join(HERE, "_sp_worker.py"), str(world)], capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0 and "single-process mode" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]
