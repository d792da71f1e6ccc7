# SPDX-License-Identifier: MIT
"""Compare two outputs saved by worker.py (same seed and inputs).

Tensor parallelism changes GEMM shapes and the order of the row-parallel
sums, so two bf16 runs differ by rounding noise; an fp32-arithmetic anchor
(`worker.py --compute-fp32 --tag anchor`) measures that floor.  Pass bar, as
in the reference (demos/flux2_tp/compare.py:49-68): cosine > 0.999 and
rel-L2 < 3 % between the two runs.
"""
import argparse
import json
import os
import sys

import torch


def rel_stats(a, b):
    d = a - b
    return {"rel_l2": (d.norm() / b.norm()).item(), "max_abs_err": d.abs().max().item(),
            "cosine": torch.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    ap.add_argument("--left-tag", default="tp1")
    ap.add_argument("--right-tag", default="tp2")
    ap.add_argument("--anchor-tag", default="anchor")
    a = ap.parse_args()
    load = lambda tag: torch.load(os.path.join(a.dir, "output_%s.pt" % tag))
    left, right = load(a.left_tag), load(a.right_tag)
    if left.shape != right.shape:
        print("FAIL: shapes differ: %s vs %s" % (tuple(left.shape), tuple(right.shape)))
        sys.exit(1)
    s = rel_stats(right, left)
    s["close_frac_atol_2e-2"] = torch.isclose(right, left, atol=2e-2, rtol=1e-2).float().mean().item()
    if os.path.exists(os.path.join(a.dir, "output_%s.pt" % a.anchor_tag)):
        anchor = load(a.anchor_tag)
        s["anchor_left_rel_l2"] = rel_stats(left, anchor)["rel_l2"]
        s["anchor_right_rel_l2"] = rel_stats(right, anchor)["rel_l2"]
    stats = lambda tag: json.load(open(os.path.join(a.dir, "stats_%s.json" % tag)))
    sl, sr = stats(a.left_tag), stats(a.right_tag)
    s.update(left_tag=a.left_tag, right_tag=a.right_tag, left_ms=sl["mean_ms_per_step"],
             right_ms=sr["mean_ms_per_step"], speedup=sl["mean_ms_per_step"] / sr["mean_ms_per_step"])
    s["passed"] = bool(s["cosine"] > 0.999 and s["rel_l2"] < 0.03)
    print("cosine=%.6f rel_L2=%.5f max_abs_err=%.5f close(2e-2)=%.4f"
          % (s["cosine"], s["rel_l2"], s["max_abs_err"], s["close_frac_atol_2e-2"]))
    if "anchor_left_rel_l2" in s:
        print("fp32 anchor: %s %.4f / %s %.4f rel_L2" % (a.left_tag, s["anchor_left_rel_l2"], a.right_tag,
                                                          s["anchor_right_rel_l2"]))
    print("%s: %.1f ms/step  %s: %.1f ms/step  speedup %.2fx" % (a.left_tag, s["left_ms"], a.right_tag,
                                                                 s["right_ms"], s["speedup"]))
    with open(os.path.join(a.dir, "correctness_%s_vs_%s.json" % (a.right_tag, a.left_tag)), "w") as f:
        json.dump(s, f, indent=2)
    print("CORRECTNESS PASSED" if s["passed"] else "CORRECTNESS FAILED")
    sys.exit(0 if s["passed"] else 1)


if __name__ == "__main__":
    main()
