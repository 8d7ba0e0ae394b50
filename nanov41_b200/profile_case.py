"""Small fixed workload for profiler captures: a few launches of every kernel of the FP8 forward.

    python -m nanov41_b200.profile_case [--tokens 4096] [--experts 16] [--iters 2]

Shapes follow BASELINE config 2 (k=6, D=I=1024) at a size whose buffers stay far below a GB, so
an `ncu --set full` capture of one kernel ends by itself in about a minute.
"""
from __future__ import annotations

import argparse

import torch

from . import ops
from .workloads import make_case


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--iters", type=int, default=2)
    args = ap.parse_args()
    c = make_case(T=args.tokens, E=args.experts, k=6, D=1024, I=1024, seed=1)
    g = {n: t.cuda() for n, t in c.items()}
    wq = ops.quantize_expert_weights(g["w1"], g["w3"], g["w2"])
    for _ in range(args.iters):
        out = ops.moe_forward_fp8(g["x"], wq, g["weights"], g["indices"], 10.0)
    ops.check_status()
    print("profile_case ok", float(out.float().abs().mean()))


if __name__ == "__main__":
    main()
