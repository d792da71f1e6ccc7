# SPDX-License-Identifier: MIT
"""Compare two decode runs saved by worker.py: first-position logits
(cosine, rel-L2, arg-max agreement) and the generated token streams.

Greedy streams of two numerically different runs (TP=1 vs TP=N, or link vs
NCCL: other summation orders) may part ways at a near-tie and then stay apart,
so the stream check reports the length of the common prefix; the pass bar is
on the logits, as in the reference (demos/qwen_tp/qwen38_int8/compare.py:30-70):
cosine > 0.999 and the same arg max for every sequence.  With `--derive-comm`
and a no-comm control run the communication cost per token is
1/tps_full - 1/tps_nocomm (demos/qwen_tp/qwen38_int8/results/README.md:17)."""
import argparse
import json
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    ap.add_argument("--left-tag", default="tp1")
    ap.add_argument("--right-tag", default="tp2")
    ap.add_argument("--nocomm-tag", default=None)
    a = ap.parse_args()
    ld = lambda kind, tag: torch.load(os.path.join(a.dir, "%s_%s.pt" % (kind, tag)))
    st = lambda tag: json.load(open(os.path.join(a.dir, "stats_%s.json" % tag)))
    l, r = ld("logits", a.left_tag), ld("logits", a.right_tag)
    d = r - l
    res = {"rel_l2": (d.norm() / l.norm()).item(), "max_abs_err": d.abs().max().item(),
           "cosine": torch.cosine_similarity(l.flatten(), r.flatten(), dim=0).item(),
           "argmax_agree": (l.argmax(-1) == r.argmax(-1)).float().mean().item()}
    tl, tr = ld("tokens", a.left_tag), ld("tokens", a.right_tag)
    n = min(tl.shape[1], tr.shape[1])
    same = (tl[:, :n] == tr[:, :n])
    prefix = [int((~row).nonzero()[0]) if (~row).any() else n for row in same]
    res["common_prefix_min"], res["common_prefix_mean"], res["steps"] = min(prefix), sum(prefix) / len(prefix), n
    sl, sr = st(a.left_tag), st(a.right_tag)
    res.update(left_tag=a.left_tag, right_tag=a.right_tag, left_tok_s=sl["tokens_per_s"],
               right_tok_s=sr["tokens_per_s"], speedup=sr["tokens_per_s"] / sl["tokens_per_s"])
    if a.nocomm_tag:
        sn = st(a.nocomm_tag)
        res["comm_ms_per_token"] = sr["decode_ms_per_token"] - sn["decode_ms_per_token"]
    res["passed"] = bool(res["cosine"] > 0.999 and res["argmax_agree"] == 1.0)
    print("logits: cosine=%.6f rel_L2=%.5f argmax agreement=%.3f | tokens: common prefix min %d / mean %.1f of %d"
          % (res["cosine"], res["rel_l2"], res["argmax_agree"], res["common_prefix_min"],
             res["common_prefix_mean"], n))
    print("%s: %.1f tok/s  %s: %.1f tok/s  ratio %.2fx%s"
          % (a.left_tag, res["left_tok_s"], a.right_tag, res["right_tok_s"], res["speedup"],
             "" if "comm_ms_per_token" not in res else "  comm %.3f ms/token" % res["comm_ms_per_token"]))
    with open(os.path.join(a.dir, "correctness_%s_vs_%s.json" % (a.right_tag, a.left_tag)), "w") as f:
        json.dump(res, f, indent=2)
    print("CORRECTNESS PASSED" if res["passed"] else "CORRECTNESS FAILED")
    sys.exit(0 if res["passed"] else 1)


if __name__ == "__main__":
    main()
