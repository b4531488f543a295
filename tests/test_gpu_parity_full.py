"""Full-size parity: the configurations the benchmark times, at the sizes it times them.

The CPU oracle runs about a hundred tokens per second at these shapes, so the
8192- and 2048-token cases check routing, histogram, offsets and permutation on
ALL tokens (integer work: bit for bit) and layer outputs on a few hundred tokens
chosen from the GPU's own permutation so that every kind of expert segment is
covered (first and last row of every expert, experts split over several
segments, experts small enough to be handed to the grouped GEMV).  Tokens are
independent, so the oracle can be run on a subset of rows.  The three-regime
structure follows crates/v4flash-kernels/tests/mxfp4_moe_sweep.rs:183-263 of the
reference (routing regimes x sizes)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2


def rel_l2(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _shared_of(w):
    return tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))


def _check_routing(oracle, cfg, w_bias, routing, logits):
    r = cfg.router
    osel, ow = oracle.router_topk(logits, w_bias, r.n_used, r.n_group, r.topk_group, r.score_fn, r.route_scale, r.weight_eps)
    assert np.array_equal(routing["selected"], osel)
    assert np.array_equal(routing["weights"].view(np.uint32), ow.view(np.uint32))
    oh, oo, op = oracle.group_build(osel, r.n_expert)
    assert np.array_equal(routing["hist"], oh) and np.array_equal(routing["offsets"], oo) and np.array_equal(routing["perm"], op)
    return osel, ow, oh, oo, op


def _oracle_rows(oracle, cfg, w, xb, osel, ow, tokens):
    from deepstrix_b200 import synth
    tokens = np.asarray(tokens)
    return oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb[tokens]), osel[tokens], ow[tokens], w["gate"], w["up"], w["down"],
                                shared=_shared_of(w), clamp=cfg.clamp, n_expert=cfg.router.n_expert)


def _tokens_at_rows(op, k, rows):
    return np.unique(op[np.asarray(rows)] // k)


def test_layer_config2_full_size_rows_of_every_expert(torch_cuda, moe, oracle, full_mxfp4):
    """Configuration 2: 8192 tokens, uniform-random routing, MXFP4.  Outputs of 256+ tokens against the
    oracle: the first sorted row of every even expert, the last of every odd one (so both ends of split
    segments and all 256 experts are touched), plus the whole batch cross-checked against the independent
    grouped-GEMV kernels on three 64-token slices."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    cfg, w = full_mxfp4["cfg"], full_mxfp4["w"]
    T, k, E = 8192, cfg.router.n_used, cfg.router.n_expert
    layer = moe.MoeLayer(cfg, full_mxfp4["routed"], full_mxfp4["shared"], full_mxfp4["rw"], full_mxfp4["rb"], max_tokens=T)
    xb = synth.make_tokens(cfg, 2, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    logits_h = synth.uniform_logits(cfg, 2, T)
    logits = torch.from_numpy(logits_h).cuda()
    out = layer.forward(x, logits=logits)
    assert layer.check() == 0
    osel, ow, oh, oo, op = _check_routing(oracle, cfg, w["router_bias"], layer.routing(T), logits_h)
    assert oh.min() > 128 and oh.max() > 256      # every expert busy, some above one segment
    out = out.float().cpu().numpy()
    assert np.isfinite(out).all()
    rows = [oo[e] if e % 2 == 0 else oo[e + 1] - 1 for e in range(E)]
    big = int(np.argmax(oh))
    rows += [oo[big] + oh[big] // 2 - 1, oo[big] + oh[big] // 2]      # either side of the busiest expert's split
    tokens = _tokens_at_rows(op, k, rows)          # a token sits in 8 experts' segments: fewer tokens than rows
    assert tokens.size >= 100
    extra = np.random.default_rng(9).choice(T, size=max(0, 256 - tokens.size), replace=False)
    tokens = np.unique(np.concatenate([tokens, extra]))
    ref = _oracle_rows(oracle, cfg, w, xb, osel, ow, tokens)
    err = rel_l2(out[tokens], ref)
    assert err <= REL_L2_TOL, err
    worst = max(rel_l2(out[t:t + 1], ref[i:i + 1]) for i, t in enumerate(tokens))
    assert worst <= 2 * REL_L2_TOL, worst          # no single row hides behind the average
    for lo in (0, 4096 + 17, T - 64):
        sl = slice(lo, lo + 64)
        dec = layer.forward(x[sl].contiguous(), logits=logits[sl].contiguous()).float().cpu().numpy()   # 64 tokens: GEMV kernels
        assert rel_l2(out[sl], dec) < 8e-3
    layer.close()


def test_layer_mid_batch_full_size_all_tokens(torch_cuda, moe, oracle, full_mxfp4):
    """512 tokens x 256 experts with the group-limited router (16 rows per expert on average): the regime
    where small experts go to the grouped GEMV and the others to the tensor cores in the same call.
    Every token against the oracle."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    cfg, w = full_mxfp4["cfg"], full_mxfp4["w"]
    T = 512
    layer = moe.MoeLayer(cfg, full_mxfp4["routed"], full_mxfp4["shared"], full_mxfp4["rw"], full_mxfp4["rb"], max_tokens=T)
    xb = synth.make_tokens(cfg, 1, T, stream=11)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out = layer.forward(x).float().cpu().numpy()
    assert layer.check() == 0
    routing = layer.routing(T)
    ref_logits = oracle.router_logits(synth.bf16_bits_to_f32(xb), w["router_w"])
    assert np.abs(routing["logits"] - ref_logits).max() < 5e-5
    osel, ow, oh, oo, op = _check_routing(oracle, cfg, w["router_bias"], routing, routing["logits"])
    assert (oh <= 8).any() and (oh > 8).any()     # both kernel families in one call (experts with at most 8 rows go to the GEMV)
    ref = _oracle_rows(oracle, cfg, w, xb, osel, ow, np.arange(T))
    err = rel_l2(out, ref)
    assert err <= REL_L2_TOL, err
    worst = max(rel_l2(out[t:t + 1], ref[t:t + 1]) for t in range(T))
    assert worst <= 2 * REL_L2_TOL, worst
    layer.close()


def test_layer_config3_full_size(torch_cuda, moe, oracle):
    """Configuration 3 as the benchmark builds it: Q8_0 experts, 256 experts, 2048 tokens, router bias
    skewed to a Zipf(1.1) popularity profile.  Routing, histogram, offsets and permutation bit-exact on all
    2048 tokens; outputs of 256+ tokens against the oracle, chosen to cover the busiest expert (several
    segments, first / middle / last rows), experts with 9..60 rows (one tensor tile) and experts with at
    most 8 rows (handed to the grouped GEMV)."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[3]
    T, k, E = 2048, cfg.router.n_used, cfg.router.n_expert
    w = synth.make_layer(cfg, 3)
    w["router_bias"] = synth.zipf_bias(cfg)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=T)
    xb = synth.make_tokens(cfg, 3, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out = layer.forward(x).float().cpu().numpy()
    assert layer.check() == 0
    routing = layer.routing(T)
    ref_logits = oracle.router_logits(synth.bf16_bits_to_f32(xb), w["router_w"])
    assert np.abs(routing["logits"] - ref_logits).max() < 5e-5
    osel, ow, oh, oo, op = _check_routing(oracle, cfg, w["router_bias"], routing, routing["logits"])
    big = int(np.argmax(oh))
    assert oh[big] > 512                                   # several segments
    mids = [e for e in range(E) if 9 <= oh[e] <= 60]
    smalls = [e for e in range(E) if 1 <= oh[e] <= 8]
    assert mids and smalls
    rows = list(range(oo[big], oo[big] + 24)) + list(range(oo[big] + oh[big] // 2 - 12, oo[big] + oh[big] // 2 + 12)) + \
        list(range(oo[big + 1] - 24, oo[big + 1]))
    for e in mids[:4]:
        rows += list(range(oo[e], oo[e + 1]))[:20]
    for e in smalls[:8]:
        rows += list(range(oo[e], oo[e + 1]))[:8]
    tokens = _tokens_at_rows(op, k, rows)
    rng = np.random.default_rng(5)
    extra = rng.choice(T, size=max(0, 256 - tokens.size), replace=False)
    tokens = np.unique(np.concatenate([tokens, extra]))
    assert 100 <= tokens.size <= 400
    ref = _oracle_rows(oracle, cfg, w, xb, osel, ow, tokens)
    err = rel_l2(out[tokens], ref)
    assert err <= REL_L2_TOL, err
    worst = max(rel_l2(out[t:t + 1], ref[i:i + 1]) for i, t in enumerate(tokens))
    assert worst <= 2 * REL_L2_TOL, worst
    layer.close()
