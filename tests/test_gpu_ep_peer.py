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
    for rep in range(2):   # twice: the slabs are reused from step to step
        for r in range(world):
            comms[r].dispatch(xs[r], sels[r], wts[r], E)
        given = []
        for r in range(world):
            rows, sel, wt = comms[r].prepare()
            part = parts[r].forward_picks(rows, sel, wt, expert_lo=r * per, with_shared=False)
            comms[r].give_back(part)
            given.append(part)
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
    # counts: tokens of source s with at least one pick owned by rank d
    for d in range(world):
        got = comms[d].counts().cpu().numpy()
        for s in range(world):
            own = sels[s].cpu().numpy() // per
            assert got[s] == int((own == d).any(axis=1).sum()), (d, s)
    for c in comms:
        c.close()
