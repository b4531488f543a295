"""Times the reference's own CPU model of the expert FFN (scripts/v41_oracle/kernel.py: act_quant, fp4_gemm --
dequantise to f32, torch matmul) on the full-size decode layer, beside the OpenMP port that bench.py times.

Test infrastructure, like everything under oracle/.  It imports the reference tree unmodified, so it runs only
where that tree is present (the build container); bench.py cannot call it on a GPU box and reports the port.

    python oracle/time_reference_kernelpy.py --reference /path/to/deepstrix [--tokens 4]

One step = the routed experts a batch of tokens picked plus the shared expert, each as
mid = silu(min(gate(x), c)) * clamp(up(x)) * w; out += down(mid), with every product through fp4_gemm on
FP8-quantised activations, the way the reference's inference/model.py drives an MoE layer.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from deepstrix_b200 import synth  # noqa: E402
from deepstrix_b200.config import CONFIGS  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DEEPSTRIX_REFERENCE", ""), help="root of the reference (deepstrix) source tree")
    ap.add_argument("--tokens", type=int, default=4)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args()
    if not args.reference:
        ap.error("give the reference tree with --reference (or DEEPSTRIX_REFERENCE)")
    path = os.path.join(args.reference, "scripts", "v41_oracle", "kernel.py")
    spec = importlib.util.spec_from_file_location("ref_kernel", path)
    K = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(K)
    torch.set_default_dtype(torch.bfloat16)   # the reference's GEMMs return the default dtype

    cfg = CONFIGS[1]
    w = synth.make_layer(cfg, 1)
    T, k = args.tokens, cfg.router.n_used
    x = torch.from_numpy(synth.bf16_bits_to_f32(synth.make_tokens(cfg, 1, T, stream=7)))
    logits = x.numpy() @ w["router_w"].T
    sel = synth._route_numpy(logits.astype(np.float32), w["router_bias"], cfg)
    wt = np.full(sel.shape, 1.0 / k, dtype=np.float32)   # routing weights do not change the timing

    def mat(name, e):
        q, s = w[name]
        return torch.from_numpy(q[e]), torch.from_numpy(s[e].astype(np.int32) - 127).float().exp2()   # E8M0 byte -> 2^(e-127)

    def ffn(e, names, rows, weights):
        xq, xs = K.act_quant(x[rows].to(torch.bfloat16), 32, "ue8m0")
        g = K.fp4_gemm(xq, xs, *mat(names[0], e)).float()
        u = K.fp4_gemm(xq, xs, *mat(names[1], e)).float()
        g = g.clamp(max=cfg.clamp)
        u = u.clamp(-cfg.clamp, cfg.clamp)
        mid = torch.nn.functional.silu(g) * u * weights[:, None]
        mq, ms = K.act_quant(mid.to(torch.bfloat16), 32, "ue8m0")
        return K.fp4_gemm(mq, ms, *mat(names[2], e)).float()

    def step():
        out = torch.zeros((T, cfg.hidden))
        for e in np.unique(sel):
            t_idx, s_idx = np.nonzero(sel == e)
            out[t_idx] += ffn(int(e), ("gate", "up", "down"), t_idx, torch.from_numpy(wt[t_idx, s_idx]))
        out += ffn(0, ("shared_gate", "shared_up", "shared_down"), np.arange(T), torch.ones(T))
        return out

    step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    print(f"reference kernel.py (dequantise + torch matmul), {torch.get_num_threads()} threads: {T} tokens, "
          f"{len(np.unique(sel))} experts + shared: {dt:.2f} s per layer step = {T / dt:.2f} tokens/s")


if __name__ == "__main__":
    main()
