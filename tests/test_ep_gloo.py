"""Expert-parallel dispatch/combine on 2 CPU ranks (gloo): host logic only, with the
oracle as the per-rank expert compute.  The sum over ranks must reproduce the
single-process layer (the reference's loopback test idea,
tests/remote_experts_loopback.rs: remote partial + local partial = plain MoE)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    from deepstrix_b200.ep import ExpertParallelMoe
    from oracle import oracle
    cfg = MoeConfig(hidden=256, ffn=256, shared_ffn=256, router=RouterConfig(n_expert=8, n_used=3, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    E, k, H = 8, 3, 256
    w = synth.make_layer(cfg, 4)
    T = 11 + 3 * rank                                   # ragged: different token counts per rank
    x = synth.bf16_bits_to_f32(synth.make_tokens(cfg, 4, T, stream=rank))
    logits = oracle.router_logits(x, w["router_w"])
    sel, wt = oracle.router_topk(logits, w["router_bias"], k, 1, 1, 1, 2.5)
    if rank == 1:
        sel[0, :] = [0, 1, 2]                           # a token whose picks all live on rank 0
    per = E // world
    lo = rank * per
    shard = {n: (w[n][0][lo:lo + per], w[n][1][lo:lo + per]) for n in ("gate", "up", "down")}
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))

    def local_compute(xr, s, ww):
        s = s.numpy().copy() - lo
        s[(s < 0) | (s >= per)] = -1                    # picks owned elsewhere are skipped
        out = oracle.moe_layer_f32(cfg.fmt, xr.numpy(), s, ww.numpy(), shard["gate"], shard["up"], shard["down"], n_expert=per)
        return torch.from_numpy(out)

    def shared_compute(xr):
        none = np.full((xr.shape[0], k), -1, np.int32)
        out = oracle.moe_layer_f32(cfg.fmt, xr.numpy(), none, np.zeros_like(none, np.float32), shard["gate"], shard["up"], shard["down"],
                                   shared=shared, n_expert=per)
        return torch.from_numpy(out)

    ep = ExpertParallelMoe(E, None, local_compute, shared_compute)
    out = ep.forward(torch.from_numpy(x), torch.from_numpy(sel), torch.from_numpy(wt)).numpy()
    ref = oracle.moe_layer_f32(cfg.fmt, x, sel, wt, w["gate"], w["up"], w["down"], shared=shared, n_expert=E)
    err = float(np.linalg.norm(out - ref) / np.linalg.norm(ref))
    results[rank] = (err, ep.last_stats["sent_rows"], ep.last_stats["received_rows"])
    dist.barrier()
    dist.destroy_process_group()


def test_ep_two_ranks_match_single_process():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for r in range(world):
            err, sent, recv = results[r]
            assert err < 1e-5, (r, err)          # f32 everywhere: only the association of the final sums differs
            assert sent > 0 and recv > 0


def test_build_dispatch_lists():
    from deepstrix_b200.ep import build_dispatch
    sel = torch.tensor([[0, 5], [6, 7], [-1, 2], [3, 4]], dtype=torch.int32)
    tok, counts = build_dispatch(sel, 2, 4)          # experts 0-3 on rank 0, 4-7 on rank 1
    assert counts.tolist() == [3, 3]
    assert tok.tolist() == [0, 2, 3, 0, 1, 3]        # each token once per destination, ascending
