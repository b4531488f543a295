"""Runs one small, configurable MoE-layer case a few times: the command to put
under a profiler (``ncu ... python bench_case.py ...``).  Harness, not product:
it only drives the library through ``deepstrix_b200.moe``.

The layer has the full-size shapes (hidden 4096, ffn 2048, top-8) but, by
default, only 64 routed experts, so that the whole case holds under 1 GB on the
device while every launch still streams far more than the L2 holds.
"""
from __future__ import annotations

import argparse

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from deepstrix_b200 import moe, synth  # noqa: E402
from deepstrix_b200.config import CONFIGS, FMT_MXFP4, FMT_Q8_0, RouterConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--fmt", default="mxfp4", choices=["mxfp4", "q8_0"])
    ap.add_argument("--uniform-routing", action="store_true", help="drive the router with random logits (prefill workload)")
    ap.add_argument("--zipf", action="store_true", help="router bias skewed to a Zipf(1.1) popularity profile (configuration 3's routing)")
    args = ap.parse_args()
    base = CONFIGS[1]
    cfg = base.with_(fmt=FMT_MXFP4 if args.fmt == "mxfp4" else FMT_Q8_0,
                     router=RouterConfig(n_expert=args.experts, n_used=8, n_group=8, topk_group=4, route_scale=2.5))
    torch.cuda.set_device(0)
    w = synth.make_layer(cfg, 1)
    if args.zipf:
        w["router_bias"] = synth.zipf_bias(cfg)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=args.tokens)
    x = torch.from_numpy(synth.make_tokens(cfg, 1, args.tokens).view(np.int16)).cuda().view(torch.bfloat16)
    logits = None
    if args.uniform_routing:
        logits = torch.from_numpy(synth.uniform_logits(cfg, 2, args.tokens)).cuda()
    layer.profile(True)
    for i in range(args.iters):
        out = layer.forward(x, logits=logits)
        torch.cuda.synchronize()
        ms = layer.stage_ms()
        print(f"iter {i}: " + "  ".join(f"{k}={v * 1e3:.1f}us" for k, v in ms.items() if v >= 0))
    assert layer.check() == 0
    hist = layer.routing(args.tokens)["hist"]
    d = int((hist > 0).sum())
    print(f"tokens={args.tokens} experts={args.experts} distinct_experts_touched={d} busiest={int(hist.max())} "
          f"experts_with_at_most_8_rows={int(((hist > 0) & (hist <= 8)).sum())} at_most_24={int(((hist > 0) & (hist <= 24)).sum())} "
          f"out_norm={out.float().norm().item():.4f}")


if __name__ == "__main__":
    main()
