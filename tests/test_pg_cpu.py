# SPDX-License-Identifier: MIT
"""The "barlink" c10d backend and the tensor-parallel model on CPU tensors
over gloo ranks (no GPU): plumbing, the tiny-Qwen2 TP=2 config of the
benchmark plan, and host-side failure cases."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(mode, world, timeout=300):
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "_cpu_worker.py"), mode, str(r),
                               str(world), str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(world)]
    res = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<killed after %d s>" % timeout
        res.append((p.returncode, out))
    return res


def test_collectives_over_gloo_ranks():
    res = _run("collectives", 2)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)


def test_collectives_four_ranks():
    res = _run("collectives", 4)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)


def test_tiny_qwen2_tp2_matches_single_rank():
    res = _run("tiny", 2)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)
    assert "max abs logit error" in res[0][1]


def test_tiny_qwen2_tp8_replicated_kv_heads():
    """8 ranks, 2 KV heads: every KV head lives on 4 ranks and its query heads are dealt out."""
    res = _run("tiny", 8, timeout=600)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)


def test_checkpoint_export_and_sharded_load():
    res = _run("checkpoint", 2)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)
    assert "checkpoint round trip" in res[0][1]


def test_tiny_mmdit_tp2_matches_single_rank():
    res = _run("mmdit", 2)
    assert all(rc == 0 for rc, _ in res), "\n".join(o for _, o in res)
    assert "rel-L2 vs one rank" in res[0][1]


def test_rank_that_never_joins_gives_a_timeout_not_a_hang():
    res = _run("late", 2, timeout=120)
    assert res[1][0] == 0          # the absent rank
    assert res[0][0] == 3, res[0][1]  # the waiting rank got an exception from the rendezvous


def test_rank_that_fails_between_steps_is_seen_on_the_host():
    res = _run("raise", 2)
    assert res[1][0] == 7
    assert res[0][0] == 0 and "saw the failure" in res[0][1], res[0][1]
