"""GPU parity: every kernel through the C ABI against the CPU oracle.

Integer / index results must match bit for bit; layer outputs within
rel-L2 <= 1e-2 of the dequantised-f32 oracle (the tolerance the workload
definition states for bf16 activations)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2


def rel_l2(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


# ------------------------------------------------------------------ repack
@pytest.mark.parametrize("layout", ["hf", "ggml", "sb2"])
def test_repack_mxfp4_roundtrip_bitexact(torch_cuda, moe, oracle, layout):
    torch = torch_cuda
    rng = np.random.default_rng(1)
    H, F, n = 512, 256, 3
    st = moe.RoutedExpertWeights(0, n, H, F)
    src = {}
    for which, (rows, k) in {moe.MAT_GATE: (F, H), moe.MAT_UP: (F, H), moe.MAT_DOWN: (H, F)}.items():
        q = rng.integers(0, 256, (n, rows, k // 2), dtype=np.uint8)
        s = rng.integers(0, 255, (n, rows, k // 32), dtype=np.uint8)
        src[which] = (q, s)
        if layout == "hf":
            st.load(which, moe.SRC_MXFP4_HF, q, s)
        else:
            sb2 = np.stack([oracle.mxfp4_repack_hf_to_sb2(q[i], s[i]) for i in range(n)])
            if layout == "sb2":
                st.load(which, moe.SRC_MXFP4_SB2, sb2)
            else:  # ggml 17-byte blocks from the super-block bytes
                sb = sb2.reshape(n, rows, k // 256, 136)
                blocks = np.concatenate([sb[..., 128:136, None], sb[..., :128].reshape(n, rows, k // 256, 8, 16)], axis=-1)
                # same thing from device memory, one slot at a time
                for i in range(n):
                    st.load(which, moe.SRC_MXFP4_GGML, torch.from_numpy(np.ascontiguousarray(blocks[i])).cuda(), None, slot=i)
    for which, (q, s) in src.items():
        for i in range(n):
            uq, us = st.unpack(i, which)
            assert np.array_equal(uq.cpu().numpy(), q[i]) and np.array_equal(us.cpu().numpy(), s[i])


def test_repack_q8_0_roundtrip_bitexact(torch_cuda, moe):
    rng = np.random.default_rng(2)
    H, F = 512, 256
    st = moe.RoutedExpertWeights(1, 2, H, F)
    for which, (rows, k) in {moe.MAT_GATE: (F, H), moe.MAT_UP: (F, H), moe.MAT_DOWN: (H, F)}.items():
        q = rng.integers(-128, 128, (2, rows, k), dtype=np.int8)
        s = rng.uniform(1e-3, 1e-2, (2, rows, k // 32)).astype(np.float16)
        blocks = np.concatenate([s.view(np.uint8).reshape(2, rows, k // 32, 2), q.view(np.uint8).reshape(2, rows, k // 32, 32)], -1)
        st.load(which, moe.SRC_Q8_0_SPLIT, q[0:1], s[0:1], slot=0)
        st.load(which, moe.SRC_Q8_0_BLOCKS, np.ascontiguousarray(blocks[1:2]), None, slot=1)
        for i in range(2):
            uq, us = st.unpack(i, which)
            assert np.array_equal(uq.cpu().numpy(), q[i]) and np.array_equal(us.cpu().numpy().view(np.uint16), s[i].view(np.uint16))


# ------------------------------------------------------------------ router
@pytest.mark.parametrize("E,k,n_group,topk_group,score_fn", [
    (256, 8, 8, 4, 1), (256, 6, 1, 1, 0), (64, 6, 8, 4, 1), (384, 6, 1, 1, 0), (256, 10, 1, 1, 1), (128, 3, 4, 2, 1), (512, 8, 16, 4, 0)])
def test_router_topk_bitexact(torch_cuda, moe, oracle, E, k, n_group, topk_group, score_fn):
    torch = torch_cuda
    from deepstrix_b200.config import RouterConfig
    rng = np.random.default_rng(E + k)
    T = 333
    logits = (rng.standard_normal((T, E)) * 1.5).astype(np.float32)
    logits[0] = 0.0                       # all equal -> lowest indices
    logits[1, : E // 2] = 0.25            # two plateaus
    logits[1, E // 2:] = -0.25
    logits[2] = np.round(logits[2], 1)    # many exact ties
    logits[3] = 30.0
    logits[4] = -30.0
    logits[5, ::2] = 25.0
    bias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    cfg = RouterConfig(n_expert=E, n_used=k, n_group=n_group, topk_group=topk_group, score_fn=score_fn, route_scale=2.5)
    r = moe.RouterTopk(cfg)
    for b in (bias, None):
        sel, w = r.launch_batched(torch.from_numpy(logits).cuda(), None if b is None else torch.from_numpy(b).cuda())
        osel, ow = oracle.router_topk(logits, b, k, n_group, topk_group, score_fn, 2.5)
        assert np.array_equal(sel.cpu().numpy(), osel)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), ow.view(np.uint32))


@pytest.mark.parametrize("E,k,n_alt,n_group,topk_group,score_fn", [(256, 8, 4, 8, 4, 1), (384, 6, 4, 1, 1, 0), (64, 6, 2, 8, 4, 1)])
def test_router_alternatives_and_range_bitexact(torch_cuda, moe, oracle, E, k, n_alt, n_group, topk_group, score_fn):
    """The reference's extras of the top-k (router_topk_par.hip:18-21,140-160,231-236): alternatives are the
    ranks k+1..k+n_alt, they leave picks and weights untouched, and the score range is max - min."""
    from deepstrix_b200.config import RouterConfig
    rng = np.random.Generator(np.random.PCG64(77 + E))
    T = 97
    logits = rng.normal(0.0, 1.3, size=(T, E)).astype(np.float32)
    logits[3, 10] = logits[3, 200 % E]   # a tie among the leaders
    bias = rng.normal(0.0, 0.01, size=(E,)).astype(np.float32)
    cfg = RouterConfig(n_expert=E, n_used=k, n_group=n_group, topk_group=topk_group, score_fn=score_fn, route_scale=2.5)
    router = moe.RouterTopk(cfg)
    lg, b = torch_cuda.from_numpy(logits).cuda(), torch_cuda.from_numpy(bias).cuda()
    sel, w, alts, alt_w, srange = router.launch_batched_ex(lg, b, n_alt=n_alt, want_range=True)
    sel0, w0 = router.launch_batched(lg, b)
    assert torch_cuda.equal(sel, sel0) and torch_cuda.equal(w, w0)
    osel, ow, oalts, oalt_w, orange = oracle.router_topk_ex(logits, bias, k, n_alt, n_group, topk_group, score_fn, 2.5, cfg.weight_eps)
    assert np.array_equal(sel.cpu().numpy(), osel)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), ow.view(np.uint32))
    assert np.array_equal(alts.cpu().numpy(), oalts)
    assert np.array_equal(alt_w.cpu().numpy().view(np.uint32), oalt_w.view(np.uint32))
    assert np.array_equal(srange.cpu().numpy().view(np.uint32), orange.view(np.uint32))
    # the alternatives are what a longer top-k would have picked next
    longer, _ = oracle.router_topk(logits, bias, k + n_alt, n_group, topk_group, score_fn, 2.5, cfg.weight_eps)
    assert np.array_equal(longer[:, k:], oalts)


@pytest.mark.parametrize("E,k,n_alt,n_protect,dry,score_fn", [(256, 8, 4, 2, False, 0), (384, 6, 4, 2, True, 0), (64, 6, 0, 0, False, 1), (128, 8, 2, 8, False, 0)])
def test_router_cache_prior_bitexact(torch_cuda, moe, oracle, E, k, n_alt, n_protect, dry, score_fn):
    """The cache prior of the reference's router (router_topk_par.hip:82-99,173-210): protected picks stay,
    the rest follows score + prior, weights come from the unbiased probabilities of what is emitted."""
    from deepstrix_b200.config import RouterConfig
    rng = np.random.Generator(np.random.PCG64(500 + E + n_protect))
    T = 61
    logits = rng.normal(0.0, 1.3, size=(T, E)).astype(np.float32)
    bias = rng.normal(0.0, 0.01, size=(E,)).astype(np.float32)
    prior = np.where(rng.random(E) < 0.3, 0.2, 0.0).astype(np.float32)   # a boost on the experts "held locally"
    cfg = RouterConfig(n_expert=E, n_used=k, n_group=1, topk_group=1, score_fn=score_fn, route_scale=1.5)
    router = moe.RouterTopk(cfg)
    lg, b, pr = (torch_cuda.from_numpy(a).cuda() for a in (logits, bias, prior))
    sel, w, alts, alt_w, orig = router.launch_batched_prior(lg, b, pr, n_protect, n_alt=n_alt, prior_dry=dry)
    osel, ow, oalts, oalt_w, oorig = oracle.router_topk_prior(logits, bias, k, n_alt, prior, n_protect, dry, score_fn, 1.5, cfg.weight_eps)
    assert np.array_equal(sel.cpu().numpy(), osel) and np.array_equal(orig.cpu().numpy(), oorig)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), ow.view(np.uint32))
    if n_alt:
        assert np.array_equal(alts.cpu().numpy(), oalts)
        assert np.array_equal(alt_w.cpu().numpy().view(np.uint32), oalt_w.view(np.uint32))
    # what must hold whatever the prior: the plain ranking is the plain router's, protected picks survive
    psel, _ = oracle.router_topk(logits, bias, k, 1, 1, score_fn, 1.5, cfg.weight_eps)
    plain, prior_pick = (osel, oorig) if dry else (oorig, osel)
    assert np.array_equal(plain, psel)
    assert np.array_equal(prior_pick[:, :n_protect], psel[:, :n_protect])
    if n_protect == k:
        assert np.array_equal(prior_pick, psel)


def test_expert_sel_count_bank(torch_cuda, moe):
    """The selection statistics bank accumulates over calls and layers; out-of-range ids are dropped
    (expert_sel_count.hip:17-28)."""
    rng = np.random.Generator(np.random.PCG64(41))
    E, n_layer = 256, 3
    bank = torch_cuda.zeros((n_layer * E,), dtype=torch_cuda.int32, device="cuda")
    want = np.zeros((n_layer, E), np.int64)
    for layer, T in ((1, 700), (1, 33), (2, 5000)):
        sel = rng.integers(-2, E + 3, size=(T, 8)).astype(np.int32)
        moe.ExpertSelCount.launch(bank, torch_cuda.from_numpy(sel).cuda(), layer, E)
        ok = (sel >= 0) & (sel < E)
        want[layer] += np.bincount(sel[ok], minlength=E)
    assert np.array_equal(bank.cpu().numpy().reshape(n_layer, E), want)


def test_layer_drafter_shape(torch_cuda, moe, oracle):
    """The drafter's grouped MoE shape (128 experts, top-3, a 5-token block, no group limit,
    sqrt-softplus scores; mxfp4_pair_matvec.hip:566-596): every distinct expert's weights are read
    once for all the tokens that picked it."""
    from deepstrix_b200.config import CONFIGS, RouterConfig
    cfg = CONFIGS[0].with_(router=RouterConfig(n_expert=128, n_used=3, n_group=1, topk_group=1, score_fn=0, route_scale=1.5))
    out, ref, layer, w, x, routing = _layer_case(torch_cuda, moe, oracle, cfg, 0, 5)
    assert rel_l2(out, ref) <= REL_L2_TOL
    assert int((routing["hist"] > 0).sum()) <= 15


def test_router_logits_close_and_batch_invariant(torch_cuda, moe, oracle):
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[1]
    rng = np.random.default_rng(4)
    W = rng.normal(0, 0.02, (256, 4096)).astype(np.float32)
    xb = synth.make_tokens(cfg, 1, 37)
    r = moe.RouterTopk(cfg.router)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    Wd = torch.from_numpy(W).cuda()
    lg = r.logits(x, Wd).cpu().numpy()
    ref = oracle.router_logits(synth.bf16_bits_to_f32(xb), W)
    assert np.abs(lg - ref).max() < 2e-5
    # the same token gives the same bits alone and inside a batch
    one = r.logits(x[17:18].contiguous(), Wd).cpu().numpy()
    assert np.array_equal(one[0].view(np.uint32), lg[17].view(np.uint32))


@pytest.mark.parametrize("T,E,H", [(128, 256, 4096), (129, 256, 4096), (191, 64, 2048), (257, 384, 5120), (1000, 256, 4096)])
def test_router_logits_tiled_same_bits_as_row_kernel(torch_cuda, moe, oracle, T, E, H):
    """Large batches take the tiled kernel (ragged last tile, odd token counts); slices of at most
    64 tokens take the warp-per-row kernel.  Same f32 operation order, so the bits must agree."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS, RouterConfig
    rng = np.random.default_rng(T + E)
    W = rng.normal(0, 0.02, (E, H)).astype(np.float32)
    xf = rng.normal(0, 1.0, (T, H)).astype(np.float32)
    x = torch.from_numpy(xf).cuda().to(torch.bfloat16)
    Wd = torch.from_numpy(W).cuda()
    r = moe.RouterTopk(RouterConfig(n_expert=E, n_used=6, n_group=1, topk_group=1, route_scale=2.5))
    big = r.logits(x, Wd).cpu().numpy()
    assert big.shape == (T, E)
    small = np.concatenate([r.logits(x[a:a + 50].contiguous(), Wd).cpu().numpy() for a in range(0, T, 50)])
    assert np.array_equal(big.view(np.uint32), small.view(np.uint32))
    rows = [0, T // 2, T - 2, T - 1]
    ref = oracle.router_logits(x[rows].float().cpu().numpy(), W)
    assert np.abs(big[rows] - ref).max() < 5e-5


# ------------------------------------------------------------------ groups
@pytest.mark.parametrize("T,k,E,chunk", [(1, 8, 256, 8), (16, 6, 64, 8), (64, 8, 256, 8), (300, 8, 256, 32), (2048, 8, 256, 128), (5000, 6, 384, 32)])
def test_group_build_bitexact(torch_cuda, moe, oracle, T, k, E, chunk):
    torch = torch_cuda
    rng = np.random.default_rng(T)
    sel = np.stack([rng.choice(E, k, replace=False) for _ in range(T)]).astype(np.int32)
    if T > 4:
        sel[1, 0] = -1
        sel[3, k - 1] = E + 5
        sel[2, :] = sel[2, 0]  # a repeated id (not produced by the router, but the builder must count it)
    hist, offs, perm, items, n_items = moe.MoeGroupBuilder.launch(torch.from_numpy(sel).cuda(), E, chunk)
    oh, oo, op = oracle.group_build(sel, E)
    assert np.array_equal(hist.cpu().numpy(), oh)
    assert np.array_equal(offs.cpu().numpy(), oo)
    assert np.array_equal(perm.cpu().numpy()[: op.size], op)
    oi, on = oracle.work_items(oh, chunk)
    assert int(n_items.item()) == on
    assert np.array_equal(items.cpu().numpy()[:on], oi)
    # written set: the wrapper pre-fills perm and the work items with -1; nothing beyond the valid counts may
    # have been touched (the reference checks written sets the same way, tests/mxfp4_moe_sweep.rs:100,154-179)
    assert (perm.cpu().numpy()[op.size:] == -1).all()
    assert (items.cpu().numpy()[on:] == -1).all()


# ------------------------------------------------------------------- layer
def _layer_case(torch, moe, oracle, cfg, config_id, T, pin_logits=False, max_tokens=None, prebuilt=None):
    from deepstrix_b200 import synth
    if prebuilt is not None:   # weights already resident (the session's full-size layer)
        w = prebuilt["w"]
        layer = moe.MoeLayer(cfg, prebuilt["routed"], prebuilt["shared"], prebuilt["rw"], prebuilt["rb"], max_tokens=max_tokens or max(T, 1))
    else:
        w = synth.make_layer(cfg, config_id)
        layer = moe.build_layer_from_host(cfg, w, max_tokens=max_tokens or max(T, 1))
    xb = synth.make_tokens(cfg, config_id, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out = layer.forward(x)
    assert layer.check() == 0
    routing = layer.routing(T)
    out = out.float().cpu().numpy()
    r = cfg.router
    # routing must be bit-exact given the same logits
    osel, ow = oracle.router_topk(routing["logits"], w["router_bias"], r.n_used, r.n_group, r.topk_group, r.score_fn, r.route_scale, r.weight_eps)
    assert np.array_equal(routing["selected"], osel)
    assert np.array_equal(routing["weights"].view(np.uint32), ow.view(np.uint32))
    oh, oo, op = oracle.group_build(osel, r.n_expert)
    assert np.array_equal(routing["hist"], oh) and np.array_equal(routing["offsets"], oo) and np.array_equal(routing["perm"], op)
    ref_logits = oracle.router_logits(synth.bf16_bits_to_f32(xb), w["router_w"])
    assert np.abs(routing["logits"] - ref_logits).max() < 5e-5
    shared = ((w["shared_gate"][0][0], w["shared_gate"][1][0]), (w["shared_up"][0][0], w["shared_up"][1][0]),
              (w["shared_down"][0][0], w["shared_down"][1][0])) if cfg.shared_ffn else None
    ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), osel, ow, w["gate"], w["up"], w["down"], shared=shared,
                               clamp=cfg.clamp, mid_round=0, n_expert=r.n_expert)
    return out, ref, layer, w, x, routing


def test_layer_config0_small(torch_cuda, moe, oracle):
    from deepstrix_b200.config import CONFIGS
    out, ref, *_ = _layer_case(torch_cuda, moe, oracle, CONFIGS[0], 0, 16)
    err = rel_l2(out, ref)
    assert err <= REL_L2_TOL, err
    assert err < 6e-3  # bf16 output rounding alone is ~2e-3


@pytest.mark.parametrize("T", [1, 8, 32, 64])
def test_layer_config1_decode(torch_cuda, moe, oracle, full_mxfp4, T):
    from deepstrix_b200.config import CONFIGS
    out, ref, layer, w, x, routing = _layer_case(torch_cuda, moe, oracle, CONFIGS[1], 1, T, max_tokens=64, prebuilt=full_mxfp4)
    assert rel_l2(out, ref) <= REL_L2_TOL
    # a token's result does not depend on its batch: token 0 alone gives the same bits
    if T > 1:
        alone = layer.forward(x[0:1].contiguous()).float().cpu().numpy()
        assert np.array_equal(alone[0], out[0])


@pytest.mark.parametrize("T", [1, 5, 9, 64, 70, 300])
def test_layer_writes_exactly_its_rows(torch_cuda, moe, oracle, T):
    """Written-set check in place of a memory sanitizer (tests/mxfp4_moe_sweep.rs:100,154-179 of the
    reference does the same with sentinels): the output buffer is pre-filled with a NaN pattern, and after
    the call rows 0..T-1 are all finite while the rows past the batch still hold the pattern, for every
    kernel family (one-launch routers, grouped GEMV, tensor-core path with its GEMV hand-off)."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[0]
    w = synth.make_layer(cfg, 0)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=T)
    xb = synth.make_tokens(cfg, 0, T, stream=3)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    guard = 8
    buf = torch.full(((T + guard) * cfg.hidden,), 0x7FC1, dtype=torch.int16, device="cuda")
    out = buf[: T * cfg.hidden].view(torch.bfloat16).view(T, cfg.hidden)
    layer.forward(x, out=out)
    assert layer.check() == 0
    got = buf.cpu().numpy().view(np.uint16)
    assert (got[T * cfg.hidden:] == 0x7FC1).all()
    assert np.isfinite(out.float().cpu().numpy()).all()
    layer.close()


def test_fused_decode_router_every_batch_size(torch_cuda, moe, oracle):
    """The one-launch decode router (logits + top-k + group build) at every tile shape it has:
    routing bit-exact with the oracle given its logits, logits the same bits as the stand-alone
    logits kernel (which the larger batches use)."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[0]
    r = cfg.router
    w = synth.make_layer(cfg, 0)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=64)
    router = moe.RouterTopk(r)
    rw = torch_cuda.from_numpy(w["router_w"]).cuda()
    for T in (1, 2, 3, 4, 5, 7, 8, 9, 16, 33, 64):
        xb = synth.make_tokens(cfg, 0, T, stream=T)
        x = torch_cuda.from_numpy(xb.view(np.int16)).cuda().view(torch_cuda.bfloat16)
        layer.forward(x)
        assert layer.check() == 0
        got = layer.routing(T)
        alone = router.logits(x, rw).cpu().numpy()
        assert np.array_equal(got["logits"].view(np.uint32), alone.view(np.uint32)), T
        osel, ow = oracle.router_topk(got["logits"], w["router_bias"], r.n_used, r.n_group, r.topk_group, r.score_fn, r.route_scale, r.weight_eps)
        assert np.array_equal(got["selected"], osel), T
        assert np.array_equal(got["weights"].view(np.uint32), ow.view(np.uint32)), T
        oh, oo, op = oracle.group_build(osel, r.n_expert)
        assert np.array_equal(got["hist"], oh) and np.array_equal(got["offsets"], oo) and np.array_equal(got["perm"], op), T
    layer.close()


def test_layer_q8_0_small(torch_cuda, moe, oracle):
    from deepstrix_b200.config import CONFIGS, FMT_Q8_0
    cfg = CONFIGS[0].with_(fmt=FMT_Q8_0)
    out, ref, *_ = _layer_case(torch_cuda, moe, oracle, cfg, 3, 24)
    assert rel_l2(out, ref) <= REL_L2_TOL


def test_layer_many_tokens_per_expert_and_no_shared(torch_cuda, moe, oracle):
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=0, router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=0, route_scale=1.5))
    out, ref, *_ = _layer_case(torch_cuda, moe, oracle, cfg, 0, 200)   # 25 tokens per expert on average: several items per expert
    assert rel_l2(out, ref) <= REL_L2_TOL


@pytest.mark.parametrize("T,E,k", [(65, 32, 4), (300, 32, 4), (2500, 32, 4)])
def test_layer_prefill_tensor_core_path_small(torch_cuda, moe, oracle, T, E, k):
    """Batches above 64 tokens run the tcgen05 grouped GEMM: ragged segments (some experts
    above 256 tokens, so they split), shared expert, several reduction chunks."""
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=256,
                    router=RouterConfig(n_expert=E, n_used=k, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    moe.launch_count(reset=True)
    out, ref, layer, *_ = _layer_case(torch_cuda, moe, oracle, cfg, 2, T)
    assert rel_l2(out, ref) <= REL_L2_TOL


def test_layer_prefill_matches_oracle_with_the_same_activation_terms(torch_cuda, moe, oracle):
    """The block-scaled path multiplies the stored FP4 weights by three MXFP4 terms per activation row.  Against
    an oracle that sees the activations through the same three terms (and mid rounded to f16, as the kernel stores
    it) what is left is f32 summation order and the bf16 rounding of the output: well under the distance to the
    exact-activation oracle, which the other tests hold to 1e-2."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=256,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    out, ref, layer, w, x, routing = _layer_case(torch_cuda, moe, oracle, cfg, 2, 700)
    xb = synth.make_tokens(cfg, 2, 700)
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))
    same = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), routing["selected"], routing["weights"], w["gate"], w["up"], w["down"],
                                shared=shared, clamp=cfg.clamp, mid_round=1, n_expert=32, act_mode=oracle.act_mxfp4(3))
    exact_err, same_err = rel_l2(out, ref), rel_l2(out, same)
    assert exact_err <= REL_L2_TOL
    assert same_err < 2.2e-3 and same_err < exact_err, (same_err, exact_err)


def test_layer_prefill_cta_pairs_same_bits(torch_cuda, moe, monkeypatch):
    """The block-scaled GEMMs run one tile per CTA or two neighbouring tiles per CTA pair (cta_group::2, picked per call by
    the rows per expert).  Both forms add the same products in the same order: pinned either way by DSX_MX_PAIR, the layer
    output is the same bits, on segments of every kind (short, 129..192 rows with their second scale chunk, split experts)."""
    import numpy as np
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    torch = torch_cuda
    cfg = MoeConfig(hidden=1024, ffn=512, shared_ffn=512,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    w = synth.make_layer(cfg, 2)
    monkeypatch.setenv("DSX_MX_PAIR", "0")
    single = moe.build_layer_from_host(cfg, w, max_tokens=2500)
    monkeypatch.setenv("DSX_MX_PAIR", "1")
    pair = moe.build_layer_from_host(cfg, w, max_tokens=2500)
    for T in (70, 700, 1200, 2500):
        x = torch.from_numpy(synth.make_tokens(cfg, 2, T).view(np.int16)).cuda().view(torch.bfloat16)
        a = single.forward(x)
        b = pair.forward(x)
        torch.cuda.synchronize()
        assert single.check() == 0 and pair.check() == 0
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), T


@pytest.mark.parametrize("T", [300, 2500])
def test_layer_prefill_forward_replays_from_a_cuda_graph(torch_cuda, moe, T):
    """A large-batch forward allocates nothing and synchronises nothing, so a serving loop can capture it once and replay
    it: both forms of the block-scaled GEMM (300 tokens: single CTAs with two accumulator buffers; 2500 tokens: CTA pairs
    launched as clusters), the quantisers, the GEMV hand-off and the combine.  The replays write the bits of the eager call."""
    import ctypes as C
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    torch = torch_cuda
    lib = moe.lib()
    cfg = MoeConfig(hidden=1024, ffn=512, shared_ffn=512,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    layer = moe.build_layer_from_host(cfg, synth.make_layer(cfg, 4), max_tokens=T)
    x = torch.from_numpy(synth.make_tokens(cfg, 4, T).view(np.int16)).cuda().view(torch.bfloat16)
    want = layer.forward(x)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    out = torch.zeros_like(x)
    with torch.cuda.stream(stream):
        layer.forward(x, out=out)   # first-use work on this stream outside the capture
        stream.synchronize()
        moe._check(lib.dsx_graph_begin_capture(C.c_void_p(stream.cuda_stream)))
        layer.forward(x, out=out)
        g = C.c_void_p()
        moe._check(lib.dsx_graph_end_capture(C.c_void_p(stream.cuda_stream), C.byref(g)))
        for _ in range(2):
            out.zero_()
            moe._check(lib.dsx_graph_launch(g, C.c_void_p(stream.cuda_stream)))
            stream.synchronize()
            assert layer.check() == 0
            assert torch.equal(out.view(torch.int16), want.view(torch.int16))
        lib.dsx_graph_destroy(g)


def test_layer_prefill_config0_shapes(torch_cuda, moe, oracle):
    from deepstrix_b200.config import CONFIGS
    out, ref, *_ = _layer_case(torch_cuda, moe, oracle, CONFIGS[0], 0, 192)
    assert rel_l2(out, ref) <= REL_L2_TOL


@pytest.mark.parametrize("T", [96, 1500])
def test_layer_prefill_q8_0_zipf(torch_cuda, moe, oracle, T):
    """Configuration 3 in miniature: Q8_0 experts on the tensor-core path with a Zipf(1.1)-skewed
    router bias, so a few experts get several segments and many get a handful of tokens."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import FMT_Q8_0, MoeConfig, RouterConfig
    torch = torch_cuda
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=256, fmt=FMT_Q8_0,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    w = synth.make_layer(cfg, 3)
    w["router_bias"] = synth.zipf_bias(cfg)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=T)
    xb = synth.make_tokens(cfg, 3, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out = layer.forward(x).float().cpu().numpy()
    assert layer.check() == 0
    r = layer.routing(T)
    rc = cfg.router
    osel, ow = oracle.router_topk(r["logits"], w["router_bias"], rc.n_used, 1, 1, 1, 2.5)
    assert np.array_equal(r["selected"], osel)
    if T > 1000:
        assert r["hist"].max() > 256 and r["hist"].max() > 6 * max(r["hist"].min(), 1)   # skewed: busiest expert needs several segments
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))
    ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), osel, ow, w["gate"], w["up"], w["down"], shared=shared,
                               clamp=cfg.clamp, n_expert=rc.n_expert)
    assert rel_l2(out, ref) <= REL_L2_TOL


def test_prefill_block_scales_beyond_f16(torch_cuda, moe, oracle):
    """Block scales above 2^13 (the most an f16 expansion of the weights could hold): the block-scaled
    tensor-core path takes the E8M0 scales as stored and must match the oracle; a decode-only store (no
    tensor-core planes) takes the grouped-GEMV kernels for the same batch and matches as well."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=0,
                    router=RouterConfig(n_expert=32, n_used=2, n_group=1, topk_group=1, score_fn=1, route_scale=1.0))
    w = synth.make_layer(cfg, 5)
    for name in ("gate", "up", "down"):
        w[name][1][...] = 127          # unit scales
    w["gate"][1][:, :, 0] = 143        # one block per row at 2^16 (the SwiGLU clamp bounds what follows)
    w["down"][1][:, :, 1] = 141        # and one at 2^14 in the second product, which is linear in it
    xb = synth.make_tokens(cfg, 5, 96).copy()
    # The 2^16 block decides the sign of every gate pre-activation and the clamp turns that sign into 0 or 10: a
    # step function, under which ANY rounding of the activations it multiplies flips a few outputs.  Values on the
    # E2M1 grid are exact in f16 and in one MXFP4 term alike, so both kernel families see that block exactly.
    grid = np.array([-3, -2, -1.5, -1, -0.5, 0.5, 1, 1.5, 2, 3], dtype=np.float32)
    xb[:, :32] = synth.f32_to_bf16_bits(np.random.default_rng(5).choice(grid, size=(96, 32)))
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    for decode_only in (False, True):
        layer = moe.build_layer_from_host(cfg, w, max_tokens=96, decode_only=decode_only)
        layer.forward(x)               # first call: one-time set-up
        moe.launch_count(reset=True)
        out = layer.forward(x).float().cpu().numpy()
        if decode_only:
            assert moe.launch_count() == 6     # logits, top-k, group build, gate/up GEMV, down GEMV, combine
        else:
            assert moe.launch_count() > 6      # segments, activation terms, two tensor-core kernels on top
        assert layer.check() == 0
        r = layer.routing(96)
        ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), r["selected"], r["weights"], w["gate"], w["up"], w["down"],
                                   clamp=cfg.clamp, n_expert=32)
        assert np.isfinite(out).all() and rel_l2(out, ref) <= REL_L2_TOL
        layer.close()


def test_activation_beyond_f16_sets_the_range_bit(torch_cuda, moe, oracle):
    """The decode kernels and the f16-operand tensor-core kernels multiply in f16: a token value beyond 65504
    must raise bit 16 of the layer's error word (the rows it feeds are inf / NaN), a clean batch must not,
    and the word is clear again after it was read.  The block-scaled path takes bf16 tokens as they are:
    the same value there is no error and the result stays finite and on the oracle."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import FMT_MXFP4, FMT_Q8_0, MoeConfig, RouterConfig
    base = MoeConfig(hidden=512, ffn=256, shared_ffn=0,
                     router=RouterConfig(n_expert=32, n_used=2, n_group=1, topk_group=1, score_fn=1, route_scale=1.0))
    for T, decode_only, fmt in ((6, False, FMT_MXFP4), (96, True, FMT_MXFP4), (96, False, FMT_Q8_0), (400, False, FMT_MXFP4)):
        cfg = base.with_(fmt=fmt)
        w = synth.make_layer(cfg, 9)
        xb = synth.make_tokens(cfg, 9, T).copy()
        clean = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
        big = clean.clone()
        big[T // 2, 7] = 98304.0             # 1.5 * 2^16: a bf16 value, above the largest f16
        layer = moe.build_layer_from_host(cfg, w, max_tokens=T, decode_only=decode_only)
        out = layer.forward(clean).float().cpu().numpy()
        assert layer.check() == 0 and np.isfinite(out).all()
        out = layer.forward(big).float().cpu().numpy()
        word = layer.check()
        if T == 400:                         # block-scaled FP4 terms hold the full bf16 range
            r = layer.routing(T)
            # (an expert with at most 8 rows is handed to the f16 kernels even in a large batch; not so here)
            assert (r["hist"][r["selected"][T // 2]] > 8).all()
            assert word == 0 and np.isfinite(out).all()
            xf = synth.bf16_bits_to_f32(big.view(torch.int16).cpu().numpy().view(np.uint16))
            ref = oracle.moe_layer_f32(cfg.fmt, xf, r["selected"], r["weights"], w["gate"], w["up"], w["down"], clamp=cfg.clamp, n_expert=32)
            assert rel_l2(out, ref) <= REL_L2_TOL
        else:
            assert word == 16
            keep = np.arange(T) != T // 2    # the other tokens' rows are untouched
            assert np.isfinite(out[keep]).all()
        assert layer.check() == 0
        layer.close()


def test_set_weights_switches_kernel_family(torch_cuda, moe, oracle):
    """A layer built on an MXFP4 store with tensor-core planes (block-scaled kernels, no f16 row copy allocated) is
    re-pointed at a decode-only MXFP4 store and then at the planes again: the same batch must meet the oracle each
    time (the f16-operand kernels' row buffer and the tensor maps follow the store), and a 96-token batch must take
    the kernel family the bound store calls for."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=256,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=1, route_scale=2.5))
    w = synth.make_layer(cfg, 4)
    T = 300
    planes = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, w["gate"], w["up"], w["down"])
    planes_sh = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    plain = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, w["gate"], w["up"], w["down"], decode_only=True)
    plain_sh = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"],
                                                 decode_only=True)
    rw, rb = torch.from_numpy(w["router_w"]).cuda(), torch.from_numpy(w["router_bias"]).cuda()
    layer = moe.MoeLayer(cfg, planes, planes_sh, rw, rb, max_tokens=T)
    xb = synth.make_tokens(cfg, 4, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))
    outs = []
    for routed, sh in ((planes, planes_sh), (plain, plain_sh), (planes, planes_sh)):
        layer.set_weights(routed, sh, rw, rb)
        out = layer.forward(x).float().cpu().numpy()
        assert layer.check() == 0
        r = layer.routing(T)
        ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), r["selected"], r["weights"], w["gate"], w["up"], w["down"],
                                   shared=shared, clamp=cfg.clamp, n_expert=32)
        assert rel_l2(out, ref) <= REL_L2_TOL
        outs.append(out)
    assert np.array_equal(outs[0], outs[2])                 # the same kernels, the same bits
    assert not np.array_equal(outs[0], outs[1])             # f16 operands against three MXFP4 terms: close, not identical
    layer.close()


def test_forward_picks_split_sums_to_full(torch_cuda, moe, oracle):
    """Owner-of-a-subset form: two half stores, each returning its weighted partial
    sum, add up to the full layer (the reference's het-split property,
    tests/mxfp4_pair_oracle.rs:198-241)."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[0]
    E = cfg.router.n_expert
    w = synth.make_layer(cfg, 0)
    full = moe.build_layer_from_host(cfg, w, max_tokens=16)
    xb = synth.make_tokens(cfg, 0, 16)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out_full = full.forward(x).float().cpu().numpy()
    r = full.routing(16)
    sel = torch.from_numpy(r["selected"]).cuda()
    wt = torch.from_numpy(r["weights"]).cuda()
    rw = torch.from_numpy(w["router_w"]).cuda()
    acc = np.zeros_like(out_full)
    for lo in (0, E // 2):
        sl = slice(lo, lo + E // 2)
        half = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, tuple(a[sl] for a in w["gate"]),
                                                 tuple(a[sl] for a in w["up"]), tuple(a[sl] for a in w["down"]))
        shared = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
        layer = moe.MoeLayer(cfg, half, shared, rw, None, max_tokens=16)
        acc += layer.forward_picks(x, sel, wt, expert_lo=lo, with_shared=(lo == 0)).float().cpu().numpy()
        assert layer.check() == 0
    assert rel_l2(acc, out_full) < 8e-3   # three bf16 roundings instead of one


@pytest.mark.parametrize("T", [3, 40, 300])
def test_layer_mxfp4_routed_q8_0_shared_other_width(torch_cuda, moe, oracle, T):
    """The reference's own weight layout: MXFP4 routed experts with a Q8_0 shared expert
    (crates/v4flash-kernels/src/weight_contract.rs:83-89, kernels/shared_expert_fused.hip:143-160), here also
    with a shared width that differs from the routed one.  The shared expert then runs as a pass of its own; every
    kernel family (one-launch router + grouped GEMV at 3 tokens, separate kernels at 40, tensor cores at 300)."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import FMT_MXFP4, FMT_Q8_0, MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=512, fmt=FMT_MXFP4,
                    router=RouterConfig(n_expert=32, n_used=4, n_group=1, topk_group=1, score_fn=0, route_scale=1.5))
    w = synth.make_layer(cfg.with_(shared_ffn=0), 7)
    rng = synth.rng_for(7, 4242)
    sg = synth.make_matrix(rng, FMT_Q8_0, 1, cfg.shared_ffn, cfg.hidden)
    su = synth.make_matrix(rng, FMT_Q8_0, 1, cfg.shared_ffn, cfg.hidden)
    sd = synth.make_matrix(rng, FMT_Q8_0, 1, cfg.hidden, cfg.shared_ffn)
    routed = moe.RoutedExpertWeights.from_host(FMT_MXFP4, cfg.hidden, cfg.ffn, w["gate"], w["up"], w["down"])
    shared = moe.RoutedExpertWeights.from_host(FMT_Q8_0, cfg.hidden, cfg.shared_ffn, sg, su, sd)
    rw, rb = torch.from_numpy(w["router_w"]).cuda(), torch.from_numpy(w["router_bias"]).cuda()
    layer = moe.MoeLayer(cfg, routed, shared, rw, rb, max_tokens=T)
    xb = synth.make_tokens(cfg, 7, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out = layer.forward(x).float().cpu().numpy()
    assert layer.check() == 0
    r = layer.routing(T)
    rc = cfg.router
    osel, ow = oracle.router_topk(r["logits"], w["router_bias"], rc.n_used, rc.n_group, rc.topk_group, rc.score_fn, rc.route_scale, rc.weight_eps)
    assert np.array_equal(r["selected"], osel) and np.array_equal(r["weights"].view(np.uint32), ow.view(np.uint32))
    ref = oracle.moe_layer_f32(FMT_MXFP4, synth.bf16_bits_to_f32(xb), osel, ow, w["gate"], w["up"], w["down"],
                               shared=((sg[0][0], sg[1][0]), (su[0][0], su[1][0]), (sd[0][0], sd[1][0])), shared_fmt=FMT_Q8_0,
                               clamp=cfg.clamp, n_expert=rc.n_expert)
    assert rel_l2(out, ref) <= REL_L2_TOL
    # and the shared rows really are in the sum: without them the result is far off
    no_shared = oracle.moe_layer_f32(FMT_MXFP4, synth.bf16_bits_to_f32(xb), osel, ow, w["gate"], w["up"], w["down"], clamp=cfg.clamp,
                                     n_expert=rc.n_expert)
    assert rel_l2(out, no_shared) > 5 * REL_L2_TOL
    layer.close()


@pytest.mark.parametrize("T", [16, 200])
def test_forward_remap_interleaved_ownership_sums_to_full(torch_cuda, moe, oracle, T):
    """The reference's ownership table (het/weights.rs:1357-1381): three owners hold interleaved, unequal, unordered
    subsets of the experts (no contiguous range could describe them); each returns its weighted partial sum for the
    picks it owns, a sentinel pick (id n_expert) and a NO_PICK belong to nobody, and the partial sums add up to the
    full layer.  Both kernel families (16 tokens: grouped GEMV; 200: tensor cores)."""
    torch = torch_cuda
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[0]
    E, k = cfg.router.n_expert, cfg.router.n_used
    w = synth.make_layer(cfg, 0)
    full = moe.build_layer_from_host(cfg, w, max_tokens=T)
    xb = synth.make_tokens(cfg, 0, T)
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    out_full = full.forward(x).float().cpu().numpy()
    r = full.routing(T)
    rng = np.random.default_rng(31)
    owner_of = rng.integers(0, 3, size=E)
    owner_of[::7] = 0                                   # unequal shares
    rw = torch.from_numpy(w["router_w"]).cuda()
    shared = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.shared_ffn, w["shared_gate"], w["shared_up"], w["shared_down"])
    sel = r["selected"].copy()
    wt = r["weights"].copy()
    acc = np.zeros_like(out_full)
    for owner in range(3):
        mine = rng.permutation(np.nonzero(owner_of == owner)[0])       # slot order unrelated to expert order
        remap = np.zeros(E, np.int32)                                   # >= 0: someone else's
        for slot, e in enumerate(mine):
            remap[e] = -(slot + 1)
        store = moe.RoutedExpertWeights.from_host(cfg.fmt, cfg.hidden, cfg.ffn, tuple(a[mine] for a in w["gate"]), tuple(a[mine] for a in w["up"]),
                                                  tuple(a[mine] for a in w["down"]))
        layer = moe.MoeLayer(cfg, store, shared, rw, None, max_tokens=T)
        got = layer.forward_remap(x, torch.from_numpy(sel).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(remap).cuda(),
                                  with_shared=(owner == 0))
        assert layer.check() == 0
        acc += got.float().cpu().numpy()
        layer.close()
    assert rel_l2(acc, out_full) < 8e-3                 # bf16 rounding of three partial results instead of one
    # a sentinel id and a NO_PICK in place of two real picks: their contribution disappears, nothing else changes
    sel2 = sel.copy()
    sel2[0, 0], sel2[1, 1] = E, -1
    remap_all = -(np.arange(E, dtype=np.int32) + 1)
    a = full.forward_remap(x, torch.from_numpy(sel2).cuda(), torch.from_numpy(wt).cuda(), torch.from_numpy(remap_all).cuda()).float().cpu().numpy()
    shared_t = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))
    wt2 = wt.copy()
    wt2[0, 0] = wt2[1, 1] = 0.0
    sel_ref = np.where((sel2 < 0) | (sel2 >= E), 0, sel2)
    ref = oracle.moe_layer_f32(cfg.fmt, synth.bf16_bits_to_f32(xb), sel_ref, wt2, w["gate"], w["up"], w["down"], shared=shared_t,
                               clamp=cfg.clamp, n_expert=E)
    assert rel_l2(a, ref) <= REL_L2_TOL
    full.close()


@pytest.mark.parametrize("T", [3, 16, 80])
def test_layer_v41_widths(torch_cuda, moe, oracle, T):
    """The reference model's own widths (hidden 5120, expert FFN 2304, top-6, sqrt-softplus scores, no
    group limit; 32 of its 384 experts to keep the test small): the 5120-long reduction does not fit
    the two-warps-per-row-tile form of the decode kernel, so batches below 8 tokens take 256-row units."""
    from deepstrix_b200.config import CONFIGS, RouterConfig
    cfg = CONFIGS[1].with_(hidden=5120, ffn=2304, shared_ffn=2304,
                           router=RouterConfig(n_expert=32, n_used=6, n_group=1, topk_group=1, score_fn=0, route_scale=1.5))
    out, ref, layer, w, x, routing = _layer_case(torch_cuda, moe, oracle, cfg, 1, T, max_tokens=80)
    assert rel_l2(out, ref) <= REL_L2_TOL
    layer.close()


@pytest.mark.parametrize("T,n", [(1, 4096), (37, 5120), (3, 512), (2, 10000)])
def test_rms_norm_rows_bitexact(torch_cuda, moe, oracle, T, n):
    """The norm that produces the layer's input rows: f32 result bit-exact with the oracle's restatement of
    rms_norm.hip (double partials per thread, f32 tree), bf16 result = that value rounded to nearest even."""
    rng = np.random.Generator(np.random.PCG64(900 + n))
    x = (rng.standard_normal((T, n)) * 3.0).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    o32, o16 = moe.RmsNorm.launch_weighted_batched(torch_cuda.from_numpy(x).cuda(), torch_cuda.from_numpy(w).cuda(), 1e-6, want_f32=True)
    ref = oracle.rms_norm_rows(x, w, 1e-6)
    assert np.array_equal(o32.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    want16 = torch_cuda.from_numpy(ref).to(torch_cuda.bfloat16)
    assert torch_cuda.equal(o16.cpu(), want16)


@pytest.mark.parametrize("bf16_in,n_hc", [(True, 4), (False, 4), (True, 3)])
def test_hc_post_bitexact(torch_cuda, moe, oracle, bf16_in, n_hc):
    """The residual mix that consumes the layer's output (hc_post.hip), reading it as bf16 or f32."""
    rng = np.random.Generator(np.random.PCG64(911))
    T, n = 9, 4096
    bo = rng.standard_normal((T, n)).astype(np.float32)
    rh = rng.standard_normal((T, n_hc, n)).astype(np.float32)
    post = rng.standard_normal((T, n_hc)).astype(np.float32)
    comb = rng.standard_normal((T, n_hc * n_hc)).astype(np.float32)
    bo_t = torch_cuda.from_numpy(bo).cuda()
    if bf16_in:
        bo_t = bo_t.to(torch_cuda.bfloat16)
        bo = bo_t.float().cpu().numpy()
    out = moe.HcPost.launch_batched(bo_t, torch_cuda.from_numpy(rh).cuda(), torch_cuda.from_numpy(post).cuda(), torch_cuda.from_numpy(comb).cuda())
    ref = oracle.hc_post(bo, rh, post, comb)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_empty_batches(torch_cuda, moe, oracle):
    """Zero tokens is a valid call everywhere (the reference's wrappers return early on an empty batch,
    src/moe_group_builder.rs:144-150): nothing is launched, nothing is written, no error."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    from deepstrix_b200.ep import PeerMemoryComm
    cfg = CONFIGS[0]
    r = cfg.router
    w = synth.make_layer(cfg, 0)
    layer = moe.build_layer_from_host(cfg, w, max_tokens=16)
    x0 = torch_cuda.empty((0, cfg.hidden), dtype=torch_cuda.bfloat16, device="cuda")
    out = layer.forward(x0)
    assert out.shape == (0, cfg.hidden) and layer.check() == 0
    sel0 = torch_cuda.empty((0, r.n_used), dtype=torch_cuda.int32, device="cuda")
    w0 = torch_cuda.empty((0, r.n_used), dtype=torch_cuda.float32, device="cuda")
    assert layer.forward_picks(x0, sel0, w0).shape == (0, cfg.hidden)
    router = moe.RouterTopk(r)
    rw = torch_cuda.from_numpy(w["router_w"]).cuda()
    assert router.logits(x0, rw).shape == (0, r.n_expert)
    # an empty batch after a real one leaves the layer usable
    x = torch_cuda.from_numpy(synth.make_tokens(cfg, 0, 4).view(np.int16)).cuda().view(torch_cuda.bfloat16)
    a = layer.forward(x).clone()
    layer.forward(x0)
    assert torch_cuda.equal(layer.forward(x), a)
    # a rank with nothing to send still takes part in the exchange
    comm = PeerMemoryComm(1, 0, 8, cfg.hidden, r.n_used)
    comm.connect_local([comm])
    comm.dispatch(x0, sel0, w0, r.n_expert)
    rows, sel, wt = comm.prepare()
    torch_cuda.cuda.synchronize()
    assert int(comm.counts().cpu()[0]) == 0 and bool((sel == -1).all())
    comm.close()
    layer.close()


def test_launcher_validation(torch_cuda, moe):
    torch = torch_cuda
    from deepstrix_b200.config import RouterConfig
    with pytest.raises(moe.DsxError):
        moe.RoutedExpertWeights(0, 2, 500, 256)          # hidden not a multiple of 256
    r = moe.RouterTopk(RouterConfig(n_expert=250, n_used=8, n_group=1, topk_group=1))
    with pytest.raises(moe.DsxError):
        r.launch_batched(torch.zeros((2, 250), device="cuda"), None)
    st = moe.RoutedExpertWeights(0, 1, 256, 256)
    with pytest.raises(moe.DsxError):
        st.load(moe.MAT_GATE, moe.SRC_Q8_0_SPLIT, np.zeros((256, 256), np.int8), np.zeros((256, 8), np.float16), slot=0)
