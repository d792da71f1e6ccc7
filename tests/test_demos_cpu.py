# SPDX-License-Identifier: MIT
"""The demo pipelines end to end on CPU with tiny models: worker at TP=1 and
at TP=2 over gloo ranks, then the compare scripts on the files they wrote."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(cmd, timeout=300, env=None):
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert p.returncode == 0, "%s\n%s\n%s" % (" ".join(cmd), p.stdout[-2000:], p.stderr[-2000:])
    return p.stdout


def _torchrun(n, script, *args):
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
            "--master-addr", "127.0.0.1", "--master-port", str(_port()), script, *args]


def test_flux_demo_tp2_matches_tp1_on_cpu(tmp_path):
    out = str(tmp_path)
    w = os.path.join(ROOT, "demos", "flux_tp", "worker.py")
    common = ["--config", "tiny", "--backend", "gloo", "--img-tokens", "64", "--txt-tokens", "16", "--steps", "1",
              "--warmup", "0", "--out", out]
    _run([sys.executable, w, "--tag", "tp1"] + common)
    _run(_torchrun(2, w, "--tag", "tp2", *common))
    text = _run([sys.executable, os.path.join(ROOT, "demos", "flux_tp", "compare.py"), "--dir", out])
    assert "CORRECTNESS PASSED" in text
    res = json.load(open(os.path.join(out, "correctness_tp2_vs_tp1.json")))
    assert res["cosine"] > 0.999 and res["passed"]


def test_qwen_demo_tp2_matches_tp1_on_cpu(tmp_path):
    out = str(tmp_path)
    w = os.path.join(ROOT, "demos", "qwen_tp", "worker.py")
    common = ["--model", "tiny", "--backend", "gloo", "--batch", "2", "--prompt-len", "16", "--gen", "4",
              "--warmup", "1", "--quant", "w8a16", "--out", out]
    _run([sys.executable, w, "--tag", "tp1"] + common)
    _run(_torchrun(2, w, "--tag", "tp2", *common))
    _run(_torchrun(2, w, "--tag", "tp2nocomm", "--no-comm", *common))
    text = _run([sys.executable, os.path.join(ROOT, "demos", "qwen_tp", "compare.py"), "--dir", out,
                 "--nocomm-tag", "tp2nocomm"])
    assert "CORRECTNESS PASSED" in text
    res = json.load(open(os.path.join(out, "correctness_tp2_vs_tp1.json")))
    assert res["argmax_agree"] == 1.0 and res["common_prefix_min"] == res["steps"]
    assert "comm_ms_per_token" in res


def test_qwen_smoke_script_on_cpu():
    text = _run([sys.executable, os.path.join(ROOT, "demos", "qwen_tp", "smoke.py")], timeout=600)
    assert "SMOKE OK" in text
