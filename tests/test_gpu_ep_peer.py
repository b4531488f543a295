"""Expert-parallel exchange over peer memory, several ranks emulated on one GPU.

The ranks live in one process (`dsx_ep_connect_local`): every phase is run for all ranks before
the next one, which gives the ordering the cross-rank barriers give between processes.  The
result of every rank must match the unsharded layer on the same tokens; slots and counts are
checked against a host restatement of the dispatch rule."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,T", [(2, 16), (4, 12), (2, 160)])
def test_peer_memory_exchange_matches_unsharded_layer(world, T):
    import torch
    from deepstrix_b200 import CONFIGS, moe, synth
    from deepstrix_b200.ep import PeerMemoryComm
    torch.cuda.set_device(0)
    cfg = CONFIGS[0]
    E, k, H = cfg.router.n_expert, cfg.router.n_used, cfg.hidden
    per = E // world
    w = synth.make_layer(cfg, 0)
    full = moe.build_layer_from_host(cfg, w, max_tokens=T)
    rw, rb = torch.from_numpy(w["router_w"]).cuda(), torch.from_numpy(w["router_bias"]).cuda()
    router = moe.RouterTopk(cfg.router)
    shared = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    parts, xs, sels, wts = [], [], [], []
    for r in range(world):
        lo = r * per
        shard = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.ffn, *[tuple(a[lo:lo + per] for a in w[n]) for n in ("gate", "up", "down")])
        parts.append(moe.MoeLayer(cfg, shard, shared, rw, rb, max_tokens=world * T))
        x = torch.from_numpy(synth.make_tokens(cfg, 0, T, stream=70 + r).view(np.int16)).cuda().view(torch.bfloat16)
        sel, wt = router.launch_batched(router.logits(x, rw), rb)
        xs.append(x); sels.append(sel.contiguous()); wts.append(wt.contiguous())
    comms = [PeerMemoryComm(world, r, T, H, k) for r in range(world)]
    for c in comms:
        c.connect_local(comms)
    outs = []
    for rep in range(3):   # several steps: the slabs are reused from step to step
        for r in range(world):
            comms[r].dispatch(xs[r], sels[r], wts[r], E)
        for r in range(world):
            rows, sel, wt = comms[r].prepare()
            if rep == 2:   # the owner's layer stores its rows straight into the sources' slabs: no give-back pass
                table = comms[r].back_rows()
                counts = comms[r].counts().cpu().numpy()
                addr = table.cpu().numpy().reshape(world, T)
                for src in range(world):   # an address for every received row, none for the unused slots
                    assert (addr[src, :counts[src]] != 0).all() and (addr[src, counts[src]:] == 0).all()
                parts[r].forward_picks_to(rows, sel, wt, table, expert_lo=r * per, with_shared=False)
            else:
                part = parts[r].forward_picks(rows, sel, wt, expert_lo=r * per, with_shared=False)
                comms[r].give_back(part)
        none_sel = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
        res = []
        for r in range(world):
            sh = parts[r].forward_picks(xs[r], none_sel, torch.zeros_like(wts[r]), expert_lo=r * per, with_shared=True)
            res.append(comms[r].sum(sh, T).float().cpu().numpy())
        outs.append(res)
    torch.cuda.synchronize()
    for r in range(world):
        assert parts[r].check() == 0 and comms[r].check() == 0
        ref = full.forward(xs[r]).float().cpu().numpy()
        err = np.linalg.norm(outs[0][r] - ref) / np.linalg.norm(ref)
        assert err < 1e-2, (r, err)
        assert np.array_equal(outs[0][r], outs[1][r])
        assert np.array_equal(outs[0][r], outs[2][r])      # rows stored through the table: the same bits
    # counts: tokens of source s with at least one pick owned by rank d
    for d in range(world):
        got = comms[d].counts().cpu().numpy()
        for s in range(world):
            own = sels[s].cpu().numpy() // per
            assert got[s] == int((own == d).any(axis=1).sum()), (d, s)
    for c in comms:
        c.close()


def test_barrier_wait_runs_out_and_reports():
    """A rank whose peer never reaches the barrier: the waiting kernel gives up after its poll limit, sets
    error bit 1 and returns; nothing hangs, the context stays usable and the next, complete barrier is clean.
    (The failure is made on the host side: rank 1 simply does not call the barrier.)"""
    import time
    import torch
    from deepstrix_b200 import moe
    from deepstrix_b200.ep import PeerMemoryComm
    torch.cuda.set_device(0)
    comms = [PeerMemoryComm(2, r, 8, 256, 2) for r in range(2)]
    for c in comms:
        c.connect_local(comms)
        c.set_barrier_polls(2000)      # 2000 polls of >= 100 ns: well under 10 ms
    t0 = time.perf_counter()
    comms[0].barrier()                 # rank 1 never arrives
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    rc = moe.lib().dsx_ep_check(comms[0]._h, None, None)
    assert rc == -3                    # DSX_ERR_DEVICE, and the word was cleared by the call
    assert comms[0].check() == 0
    comms[1].barrier()                 # rank 1 catches up: rank 0's epoch is already published, no wait
    torch.cuda.synchronize()
    assert comms[1].check() == 0
    comms[0].barrier()                 # alone again (the ranks share one stream here): gives up again, cleanly
    torch.cuda.synchronize()
    assert comms[0].check() == 1
    x = torch.arange(1024, device="cuda").sum().item()   # the context still runs kernels
    assert x == 1023 * 512
    for c in comms:
        c.close()


def test_peer_memory_exchange_config4_shapes_against_oracle(oracle, full_mxfp4):
    """One layer of configuration 4 (hidden 4096, expert width 2048, 256 experts over 4 ranks, group-limited
    top-8) through the exchange, four ranks emulated on one GPU, 96 tokens per rank: every rank's owner pass
    sees 384 slots (tensor-core path for its busy experts, grouped GEMV for the rest).  Checked against the
    CPU oracle on a sample of every rank's tokens."""
    import torch
    from deepstrix_b200 import moe, synth
    from deepstrix_b200.ep import PeerMemoryComm
    torch.cuda.set_device(0)
    cfg, w = full_mxfp4["cfg"], full_mxfp4["w"]
    world, T = 4, 96
    E, k, H = cfg.router.n_expert, cfg.router.n_used, cfg.hidden
    per = E // world
    rw, rb = full_mxfp4["rw"], full_mxfp4["rb"]
    router = moe.RouterTopk(cfg.router)
    parts, xs, xbs, sels, wts = [], [], [], [], []
    for r in range(world):
        lo = r * per
        shard = moe.RoutedExpertWeights.from_host(cfg.fmt, H, cfg.ffn, *[tuple(a[lo:lo + per] for a in w[n]) for n in ("gate", "up", "down")])
        parts.append(moe.MoeLayer(cfg, shard, full_mxfp4["shared"], rw, rb, max_tokens=world * T))
        xb = synth.make_tokens(cfg, 4, T, stream=300 + r)
        x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
        sel, wt = router.launch_batched(router.logits(x, rw), rb)
        xs.append(x); xbs.append(xb); sels.append(sel.contiguous()); wts.append(wt.contiguous())
    comms = [PeerMemoryComm(world, r, T, H, k) for r in range(world)]
    for c in comms:
        c.connect_local(comms)
    for r in range(world):
        comms[r].dispatch(xs[r], sels[r], wts[r], E)
    for r in range(world):
        rows, sel, wt = comms[r].prepare()
        comms[r].give_back(parts[r].forward_picks(rows, sel, wt, expert_lo=r * per, with_shared=False))
    none_sel = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))
    sample = np.arange(0, T, 4)
    for r in range(world):
        sh = parts[r].forward_picks(xs[r], none_sel, torch.zeros_like(wts[r]), expert_lo=r * per, with_shared=True)
        got = comms[r].sum(sh, T).float().cpu().numpy()
        assert parts[r].check() == 0 and comms[r].check() == 0
        sel_h, wt_h = sels[r].cpu().numpy(), wts[r].cpu().numpy()
        ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xbs[r][sample]), sel_h[sample], wt_h[sample], w["gate"], w["up"], w["down"],
                                   shared=shared, clamp=cfg.clamp, n_expert=E)
        err = np.linalg.norm(got[sample] - ref) / np.linalg.norm(ref)
        assert err < 1e-2, (r, err)     # two more bf16 roundings than the unsharded layer (partial rows travel as bf16)
    for c in comms:
        c.close()
    for p in parts:
        p.close()
