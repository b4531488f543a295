"""Expert-parallel benchmark leg (configuration 4): a stack of 8 full-size MoE
layers, 256 experts sharded evenly over the GPUs of one node, the shared expert
replicated, 4096 bf16 tokens per GPU.  Dispatch and combine go over peer memory
(rows stored straight into the owner's HBM through NVLink, no host round trip);
``DSX_EP_TRANSPORT=nccl`` selects per-peer NCCL send/recv instead.

Launched by ``bench.py`` under ``torch.distributed.run`` (one rank per GPU; with one rank the same stack
runs with all 256 experts on that GPU, the point the expert-parallel lines are compared with).
Harness, not product: it drives the library through ``deepstrix_b200.moe`` / ``deepstrix_b200.ep``.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

N_LAYERS = 8
TOKENS_PER_GPU = 4096




def open_peer_memory(world: int, rank: int, cap: int, hidden: int, k: int):
    """A connected PeerMemoryComm, or None on EVERY rank when any rank could not allocate its slab or map
    its peers' memory (no peer access between some pair of GPUs, IPC not permitted in this container)."""
    from deepstrix_b200.ep import PeerMemoryComm

    def all_ok(ok: bool) -> bool:
        flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return float(flag.item()) >= 1.0

    comm, why = None, ""
    try:
        comm = PeerMemoryComm(world, rank, cap, hidden, k)
    except Exception as e:
        why = str(e)
    if world == 1 and comm is not None:   # a process cannot open its own IPC handle, and has no peer to map
        comm.connect_local([comm])
        return comm
    if all_ok(comm is not None):
        handles = [None] * world
        dist.all_gather_object(handles, comm.export_handle())   # every rank takes part: all slabs exist
        try:
            comm.connect(handles)
            mapped = True
        except Exception as e:
            why, mapped = str(e), False
        if all_ok(mapped):
            return comm
    if why:
        print(f"[rank {rank}] peer-memory transport unavailable ({why}); every rank falls back to NCCL send/recv", flush=True)
    if comm is not None:
        comm.close()
    return None


def selfcheck(rank: int, world: int, use_peer: bool = True):
    """Small layer, experts sharded over the ranks: the expert-parallel result must equal the
    unsharded layer computed on the same GPU (configuration 4's check, at a size that takes a
    second).  Covers both kernel families: 16 tokens (GEMV kernels) and 160 (tensor-core path)."""
    from deepstrix_b200 import CONFIGS, moe, synth
    from deepstrix_b200.ep import ExpertParallelMoe, ExpertParallelPeerMemory, PeerMemoryComm
    cfg = CONFIGS[0]
    E, k, H = cfg.router.n_expert, cfg.router.n_used, cfg.hidden
    per, lo = E // world, rank * (E // world)
    w = synth.make_layer(cfg, 0)
    full = moe.build_layer_from_host(cfg, w, max_tokens=160 * world)
    shard = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.ffn, *[tuple(a[lo:lo + per] for a in w[n]) for n in ("gate", "up", "down")])
    shared = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    rw, rb = torch.from_numpy(w["router_w"]).cuda(), torch.from_numpy(w["router_bias"]).cuda()
    part = moe.MoeLayer(cfg, shard, shared, rw, rb, max_tokens=160 * world)
    # the shared expert runs on a side stream while the owned experts run on the main one: a layer's
    # workspace (groups, mid, partial rows) serves one call at a time, so the shared pass gets its own
    part_sh = moe.MoeLayer(cfg, shard, shared, rw, rb, max_tokens=160)
    router = moe.RouterTopk(cfg.router)
    comm = open_peer_memory(world, rank, 160, H, k) if use_peer else None
    worst = 0.0
    for T in (16, 160):
        x = torch.from_numpy(synth.make_tokens(cfg, 0, T, stream=50 + rank).view(np.int16)).cuda().view(torch.bfloat16)
        sel, wt = router.launch_batched(router.logits(x, rw), rb)
        none_sel = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
        ep = ExpertParallelMoe(E, None, lambda xr, s, ww: part.forward_picks(xr, s, ww, expert_lo=lo, with_shared=False),
                               lambda xr: part_sh.forward_picks(xr, none_sel, torch.zeros_like(wt), expert_lo=lo, with_shared=True))
        got = ep.forward(x, sel, wt)
        # the peer-memory transport moves the same rows and adds in the same order; the owner sees all
        # world*cap slots at once, so it may take the other kernel family: compare both with the unsharded layer
        got = got.float()
        ref = full.forward(x).float()
        worst = max(worst, float((got - ref).norm() / ref.norm()))
        if comm is not None:
            ep2 = ExpertParallelPeerMemory(E, comm, lambda xr, s, ww: part.forward_picks(xr, s, ww, expert_lo=lo, with_shared=False),
                                           lambda xr: part_sh.forward_picks(xr, none_sel, torch.zeros_like(wt), expert_lo=lo, with_shared=True))
            raw2 = ep2.forward(x, sel.contiguous(), wt.contiguous())
            worst = max(worst, float((raw2.float() - ref).norm() / ref.norm()))
            # the same step with the owner's rows stored straight into the sources' slabs: the same bits
            ep3 = ExpertParallelPeerMemory(E, comm, None, lambda xr: part_sh.forward_picks(xr, none_sel, torch.zeros_like(wt), expert_lo=lo, with_shared=True),
                                           local_compute_to=lambda xr, s, ww, to: part.forward_picks_to(xr, s, ww, to, expert_lo=lo, with_shared=False))
            raw3 = ep3.forward(x, sel.contiguous(), wt.contiguous())
            assert torch.equal(raw3.view(torch.int16), raw2.view(torch.int16)), "rows stored through the table differ from the give-back pass"
    assert part.check() == 0 and part_sh.check() == 0 and full.check() == 0 and (comm is None or comm.check() == 0)
    dist.barrier()
    if comm is not None:
        comm.close()
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst = float(t.item())
    assert worst < 1e-2, f"expert-parallel result differs from the unsharded layer: rel-L2 {worst}"
    return worst


def run(args):
    from deepstrix_b200 import CONFIGS, moe, synth
    from deepstrix_b200.ep import ExpertParallelMoe, ExpertParallelPeerMemory, PeerMemoryComm
    import bench as B

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "the expert-parallel bench needs CUDA devices"
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    transport = os.environ.get("DSX_EP_TRANSPORT", "peer")
    check_err = selfcheck(rank, world, use_peer=transport != "nccl")
    cfg = CONFIGS[4]
    E, k, H, F = cfg.router.n_expert, cfg.router.n_used, cfg.hidden, cfg.ffn
    per = E // world
    lo = rank * per
    T = TOKENS_PER_GPU
    hbm_peak, bf16_peak, peak_kind = B.measured_peaks()

    # every rank draws the same layer and keeps its shard; the routed weights are reused by the 8
    # layers (a shard is 427 MB at 8 GPUs, well above L2), router weights differ per layer
    w = synth.make_layer(cfg, 4)
    shard = {n: (w[n][0][lo:lo + per], w[n][1][lo:lo + per]) for n in ("gate", "up", "down")}
    routed = moe.RoutedExpertWeights.from_host(cfg.fmt, H, F, shard["gate"], shard["up"], shard["down"])
    shared = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    del w, shard
    routers = []
    for layer_i in range(N_LAYERS):
        rng = synth.rng_for(4, 500 + layer_i)
        rw = torch.from_numpy(rng.normal(0.0, 0.02, size=(E, H)).astype(np.float32)).cuda()
        rb = torch.from_numpy(rng.normal(0.0, 0.01, size=(E,)).astype(np.float32)).cuda()
        routers.append((rw, rb))
    max_rows = T * world                       # every token of every rank at worst
    layer = moe.MoeLayer(cfg, routed, shared, routers[0][0], routers[0][1], max_tokens=max_rows)
    # the shared expert runs on a side stream beside the dispatch: it needs its own workspace
    layer_sh = moe.MoeLayer(cfg, routed, shared, routers[0][0], routers[0][1], max_tokens=T)
    router = moe.RouterTopk(cfg.router)
    none_sel = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
    none_w = torch.zeros((T, k), dtype=torch.float32, device="cuda")

    def local_compute(xr, s, ww):
        return layer.forward_picks(xr, s, ww, expert_lo=lo, with_shared=False)

    # the shared expert's rows are written on the side stream and read on the main one: two fixed buffers taken in turn
    # (the side stream waits for the main one before every call, so the reader of a buffer is always done with it)
    sh_out = [torch.empty((T, H), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    sh_turn = [0]

    def local_compute_to(xr, s, ww, out_rows):
        layer.forward_picks_to(xr, s, ww, out_rows, expert_lo=lo, with_shared=False)

    def shared_compute(xr):
        sh_turn[0] ^= 1
        return layer_sh.forward_picks(xr, none_sel, none_w, expert_lo=lo, with_shared=True, out=sh_out[sh_turn[0]])

    comm = open_peer_memory(world, rank, T, H, k) if transport != "nccl" else None
    if comm is None:
        ep = ExpertParallelMoe(E, None, local_compute, shared_compute)
    else:
        ep = ExpertParallelPeerMemory(E, comm, local_compute, shared_compute,
                                      local_compute_to=None if os.environ.get("DSX_EP_GIVE_BACK_PASS") == "1" else local_compute_to)
    stats = {"received_rows": [], "fanout": []}

    norm_w = torch.ones((H,), device="cuda", dtype=torch.float32)
    ones_t = torch.ones((T, 1), device="cuda", dtype=torch.float32)

    def step(x):
        # between layers, the steps the model has either side of the MoE path, on the library's own kernels: the layer's
        # bf16 output is mixed into the f32 residual stream (dsx_hc_post, one stream), whose RMSNorm is the next bf16 input
        res = x.float().view(T, 1, H)
        for rw, rb in routers:
            logits = router.logits(x, rw)
            sel, wt = router.launch_batched(logits, rb)
            out = ep.forward(x, sel.contiguous(), wt.contiguous())
            if comm is None:
                stats["received_rows"].append(ep.last_stats["received_rows"])
                stats["fanout"].append(ep.last_stats["fanout"])
            res = moe.HcPost.launch_batched(out, res, ones_t, ones_t)
            _, x = moe.RmsNorm.launch_weighted_batched(res.view(T, H), norm_w)
        return x

    xs = [torch.from_numpy(synth.make_tokens(cfg, 4, T, stream=1000 * rank + i).view(np.int16)).cuda().view(torch.bfloat16) for i in range(4)]
    sampler = B.ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    warm = max(args.warmup, 3)
    for i in range(warm):
        step(xs[i % 4])
    stats = {"received_rows": [], "fanout": []}
    torch.cuda.synchronize()
    dist.barrier()
    moe.launch_count(reset=True)
    t_w0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e0.record()
    for i in range(args.steps):
        step(xs[i % 4])
        marks[i].record()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t_w1 = time.time()
    step_ms = [a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks)]
    launches = moe.launch_count()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    assert layer.check() == 0 and layer_sh.check() == 0 and (comm is None or comm.check() == 0)

    # end to end: tokens start in pinned host memory, the stack's output returns to the host
    xh = [t.cpu().pin_memory() for t in xs]
    oh = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    for i in range(2):
        oh.copy_(step(xh[i % 4].cuda(non_blocking=True)), non_blocking=True)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for i in range(args.steps):
        oh.copy_(step(xh[i % 4].cuda(non_blocking=True)), non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    e2e = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e = float(e2e.item())
    # one more pass with per-phase events (rank 0's view)
    ep.profile = True
    t_r0 = torch.cuda.Event(enable_timing=True); t_r1 = torch.cuda.Event(enable_timing=True)
    t_r0.record()
    step(xs[0])
    t_r1.record()
    phases = ep.phase_ms()
    phases["step_total"] = t_r0.elapsed_time(t_r1)
    ep.profile = False
    if comm is not None:   # rows received in the last layer of the last step; every sent row is received once
        got_rows = float(comm.counts().sum().item())
        rows = torch.tensor([got_rows, got_rows / T], device="cuda")
    else:
        rows = torch.tensor([float(np.mean(stats["received_rows"])), float(np.mean(stats["fanout"]))], device="cuda")
    dist.all_reduce(rows, op=dist.ReduceOp.SUM)
    if sampler:
        sampler.stop()
    if rank == 0:
        layer_tokens = world * T * N_LAYERS * args.steps
        picks_per_rank = T * k                                 # on average every rank computes T*k picks + T shared rows
        flops_rank_step = N_LAYERS * 2.0 * 3 * F * H * (picks_per_rank + T)
        tf = flops_rank_step * args.steps / (ms * 1e-3) / 1e12
        line = {
            "metric": B.METRIC, "value": layer_tokens / (ms * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "block-scaled FP4 MMAs: stored MXFP4 weights x activations as 3 MXFP4 terms, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"config4: stack of {N_LAYERS} full-size MoE layers, 256 experts sharded over {world} GPUs "
                                   f"({per} per GPU), shared expert replicated, {T} bf16 tokens per GPU; value counts tokens x layers",
                       "tokens_per_gpu": T, "layers": N_LAYERS, "parallelism": f"ep{world}",
                       "exchange": ("peer memory: rows, picks and weights stored straight into the owner's HBM over NVLink (CUDA IPC mapping), "
                                    "slots by a device-side scan, the owner's combine kernel stores its partial rows straight into the sources' HBM, "
                                    "two device-side barriers per layer, no host round trip"
                                    if comm is not None else
                                    "per-peer NCCL send/recv batches (token rows + picks + weights once per owner rank; one partial row back)"),
                       "l2": "each layer streams the rank's expert shard (%.0f MB) and %d token rows: far above L2" % (routed.device_bytes / 1e6, T)},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": bf16_peak, "unit": "TFLOP/s", "frac": tf / bf16_peak, "traffic": None,
                         "kernel": "mx_gemm_kernel (tcgen05 kind::mxf4 block-scaled; 3 MMAs per algorithmic product)", "peak_kind": peak_kind,
                         "note": "per-GPU expert FLOPs of the whole step over the step time (exchange and routing included)"},
            "e2e": {"value": layer_tokens / (e2e * 1e-3), "unit": B.UNIT, "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2,
                    "ms_per_step": e2e / args.steps},
            "gpu_launches": launches,
            "clocks": sampler.summary(t_w0, t_w1) if sampler else None,
            "ep": {"step_ms_rank0": [round(v, 3) for v in step_ms], "phase_ms_per_step_rank0": {n: round(v, 3) for n, v in phases.items()}, "selfcheck_rel_l2_vs_unsharded_layer": check_err, "mean_received_rows_per_rank_per_layer": float(rows[0].item()) / world, "mean_fanout": float(rows[1].item()) / world},
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
