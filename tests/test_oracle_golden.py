"""The CPU oracle against the reference's own known answers (no GPU)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_mxfp4_dequant_matches_reference_selftest_bits(oracle):
    # external/ds4-dump/quants_selftest_expected.inc:93-137 (llama.cpp dequant bit patterns)
    g = np.load(os.path.join(GOLD, "mxfp4_selftest.npz"))
    got = oracle.mxfp4_dequant_ggml(g["blocks"]).view(np.uint32)
    assert np.array_equal(got, g["expected"])


def test_mxfp4_layouts_agree(oracle):
    g = np.load(os.path.join(GOLD, "mxfp4_selftest.npz"))
    blocks = g["blocks"]  # one row of 256 elements
    packed, scales = oracle.mxfp4_repack_ggml_to_hf(blocks, 1, 256)
    ref = oracle.mxfp4_dequant_ggml(blocks)
    assert np.array_equal(oracle.mxfp4_dequant_hf(packed, scales).ravel().view(np.uint32), ref.view(np.uint32))
    sb2 = oracle.mxfp4_repack_hf_to_sb2(packed, scales)
    assert np.array_equal(oracle.mxfp4_dequant_sb2(sb2).view(np.uint32), ref.view(np.uint32))
    p2, s2 = oracle.mxfp4_repack_sb2_to_hf(sb2, 1, 256)
    assert np.array_equal(p2, packed) and np.array_equal(s2, scales)


def test_repack_nibble_placement_literal(oracle):
    # crates/v4flash-core/src/hf_v41.rs:1358-1382: elements k = 0..31 with value k & 0xF
    packed = np.array([((2 * i) & 0xF) | (((2 * i + 1) & 0xF) << 4) for i in range(16)], np.uint8)
    packed = np.tile(packed, 8)[None, :]            # one row, 8 blocks = one super-block
    scales = np.full((1, 8), 0x7F, np.uint8)
    sup = oracle.mxfp4_repack_hf_to_sb2(packed, scales)[0]
    for i in range(16):
        assert sup[i] & 0xF == i & 0xF
        assert sup[i] >> 4 == (16 + i) & 0xF
    assert sup[128] == 0x7F


def test_e4m3_e8m0_literals(oracle):
    # crates/v4flash-core/src/hf_v41.rs:1321-1339
    assert oracle.e4m3(0x38) == 1.0
    assert oracle.e4m3(0x7E) == 448.0
    assert oracle.e4m3(0x08) == 2.0 ** -6
    assert oracle.e4m3(0x01) == 2.0 ** -9
    assert oracle.e4m3(0xB8) == -1.0
    assert np.signbit(oracle.e4m3(0x80)) and oracle.e4m3(0x80) == 0.0
    assert np.isnan(oracle.e4m3(0x7F)) and np.isnan(oracle.e4m3(0xFF))
    assert oracle.e8m0(127) == 1.0
    assert oracle.e8m0(0) == 2.0 ** -127
    assert oracle.e8m0(254) == 2.0 ** 127
    assert np.isnan(oracle.e8m0(255))
    # mxfp4_tables.rs:37-45: 2^(e-128), denormal for e < 2
    for e in (0, 1, 2, 100, 127, 200, 254):
        assert oracle.e8m0_half(e) == 2.0 ** (e - 128)


def test_q8_0_block_literal(oracle):
    # crates/v4flash-core/src/hf_v41.rs:1341-1356
    x = np.zeros(32, np.float32)
    x[:4] = [254.0, -1.0, 0.75, -0.75]
    o = oracle.q8_0_quantize_block(x)
    d = np.frombuffer(o[:2].tobytes(), np.float16)[0]
    assert float(d) == 2.0
    q = o[2:].view(np.int8)
    assert q[0] == 127 and q[1] == -1 and q[2] == 0 and q[3] == 0
    assert not oracle.q8_0_quantize_block(np.zeros(32, np.float32)).any()


def test_bytes_per_expert_and_wi_bound_literals(oracle):
    # src/weight_contract.rs:363-366 and het/dispatch.rs:746-748
    assert 2048 * (4096 // 32) * 17 == 4_456_448
    assert oracle.wi_upper_bound(12, 384, 32) == 12
    assert oracle.wi_upper_bound(3072, 384, 32) == 480
    assert oracle.wi_upper_bound(3072, 384, 32, 100) == 100


def test_against_reference_kernel_py(oracle):
    # outputs of scripts/v41_oracle/kernel.py (dequant_fp4, q8_0_roundtrip, fp4_gemm)
    g = np.load(os.path.join(GOLD, "kernelpy_vectors.npz"))
    deq = oracle.mxfp4_dequant_hf(g["packed"], g["scales"])
    # kernel.py keeps -0.0 for code 8; the engine's integer table gives +0: compare values
    assert np.array_equal(deq, g["dequant"])
    # fp4_gemm = f32 matmul of dequantised operands
    ref = g["x_fp8_dequant"] @ deq.T
    assert np.allclose(ref, g["fp4_gemm"], rtol=1e-5, atol=1e-4)
    # Q8_0 round trip = quantise block + dequant
    w = g["q8_in"]
    rt = np.empty_like(w)
    for r in range(w.shape[0]):
        for b in range(w.shape[1] // 32):
            blk = oracle.q8_0_quantize_block(w[r, b * 32:(b + 1) * 32])
            rt[r, b * 32:(b + 1) * 32] = oracle.q8_0_dequant(blk)
    assert np.array_equal(rt, g["q8_roundtrip"])


def test_dot_mxfp4_q8k_consistency(oracle):
    # external/ds4-dump/quants_selftest.c:120-171: vec_dot == dot of dequantised operands within 1e-4
    rng = np.random.default_rng(5)
    K = 1024
    packed = rng.integers(0, 256, (1, K // 2), dtype=np.uint8)
    scales = rng.integers(118, 134, (1, K // 32), dtype=np.uint8)
    x = rng.standard_normal(K).astype(np.float32)
    xq = oracle.q8_k_quantize(x)
    sb2 = oracle.mxfp4_repack_hf_to_sb2(packed, scales)
    got = oracle.dot_mxfp4_q8k(sb2, xq)
    w = oracle.mxfp4_dequant_hf(packed, scales)[0].astype(np.float64)
    blocks = xq.reshape(-1, 292)
    xd = np.concatenate([b[:4].view(np.float32)[0] * b[4:260].view(np.int8).astype(np.float64) for b in blocks])
    want = float(w @ xd)
    assert abs(got - want) <= 1e-4 * max(abs(want), 1.0)
    # bsums consistent with quants (needed by the reference's matrix-core arm)
    for b in blocks:
        q = b[4:260].view(np.int8).astype(np.int32).reshape(16, 16).sum(1)
        assert np.array_equal(q, b[260:].view(np.int16))


def test_q8_k_tie_takes_the_sign_the_reduction_tree_picks(oracle):
    # kernels/q8_k_quantize.hip:50-62: stride 128..1, the upper element only when strictly larger -- of two equal
    # |x| at indices 1 and 128, index 128 reaches slot 0 in the first round and keeps it
    x = np.full(256, 0.25, np.float32)
    x[1], x[128] = 2.0, -2.0
    b = oracle.q8_k_quantize(x)
    d = b[:4].view(np.float32)[0]
    q = b[4:260].view(np.int8)
    assert d == np.float32(1.0) / (np.float32(-127.0) / np.float32(-2.0)) and q[128] == -127 and q[1] == 127
    assert np.array_equal(b[260:].view(np.int16), q.astype(np.int32).reshape(16, 16).sum(1))
    assert not oracle.q8_k_quantize(np.zeros(256, np.float32)).any()


def test_swiglu_clamp_weighted_oracle(oracle):
    # kernels/swiglu_clamp_weighted.hip:16-37 -- one-sided clamp on gate, two-sided on up, times the expert's weight
    gate = np.array([[20.0, -20.0, 1.0, 0.0], [3.0, 3.0, 3.0, 3.0]], np.float32)
    up = np.array([[20.0, -20.0, -2.0, 5.0], [1.0, -1.0, 11.0, -11.0]], np.float32)
    w = np.array([0.5, 2.0], np.float32)
    for det in (True, False):
        m = oracle.swiglu_clamp_weighted(gate, up, w, 10.0, use_det=det)
        sil = lambda g: g / (1.0 + np.exp(-np.float64(g)))
        want = np.array([[sil(10.0) * 10 * 0.5, sil(-20.0) * -10 * 0.5, sil(1.0) * -2 * 0.5, 0.0],
                         [sil(3.0) * 2, -sil(3.0) * 2, sil(3.0) * 10 * 2, -sil(3.0) * 10 * 2]])
        assert np.allclose(m, want, rtol=1e-6, atol=1e-12)
    unclamped = oracle.swiglu_clamp_weighted(gate, up, w, 0.0)
    assert np.isclose(unclamped[0, 0], 20.0 * 20.0 * 0.5, rtol=1e-6)
    rng = np.random.default_rng(3)
    g, u = (rng.standard_normal((5, 64)) * 8).astype(np.float32), (rng.standard_normal((5, 64)) * 8).astype(np.float32)
    ww = rng.random(5).astype(np.float32)
    assert np.allclose(oracle.swiglu_clamp_weighted(g, u, ww, 10.0), oracle.swiglu_clamp_weighted(g, u, ww, 10.0, use_det=False), rtol=1e-6, atol=1e-30)


def test_det_math_close_to_libm(oracle):
    xs = np.linspace(-30, 30, 2001).astype(np.float32)
    for x in xs[::7]:
        a = oracle.lib().dsxo_det_expf(float(x))
        assert abs(a - np.exp(np.float64(x))) <= 4e-7 * np.exp(np.float64(x))
    for y in np.exp(np.linspace(-20, 20, 301)).astype(np.float32):
        a = oracle.lib().dsxo_det_log1pf(float(y))
        assert abs(a - np.log1p(np.float64(y))) <= 1e-6 * np.log1p(np.float64(y))


def _router_f64(logits, bias, k, n_group, topk_group, score_fn, scale, eps):
    lg = logits.astype(np.float64)
    if score_fn == 1:
        p = 1.0 / (1.0 + np.exp(-lg))
    else:
        p = np.sqrt(np.where(lg > 20, lg, np.where(lg < -20, np.exp(lg), np.log1p(np.exp(lg)))))
    s = p + (0 if bias is None else bias.astype(np.float64))
    T, E = s.shape
    if n_group > 1:
        per = E // n_group
        gs = np.sort(s.reshape(T, n_group, per), axis=2)[:, :, -2:].sum(2)
        order = np.argsort(-gs, axis=1, kind="stable")[:, :topk_group]
        keep = np.zeros((T, n_group), bool)
        np.put_along_axis(keep, order, True, axis=1)
        s = np.where(np.repeat(keep, per, axis=1), s, -np.inf)
    sel = np.argsort(-s, axis=1, kind="stable")[:, :k]
    ps = np.take_along_axis(p, sel, 1)
    w = ps / np.maximum(ps.sum(1, keepdims=True), eps) * scale
    return sel, w


@pytest.mark.parametrize("score_fn,n_group,topk_group,k,E", [(1, 8, 4, 8, 256), (0, 1, 1, 6, 256), (1, 8, 4, 6, 64), (1, 1, 1, 10, 256)])
def test_router_against_f64(oracle, score_fn, n_group, topk_group, k, E):
    rng = np.random.default_rng(11)
    logits = (rng.standard_normal((64, E)) * 1.3).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    sel, w = oracle.router_topk(logits, bias, k, n_group, topk_group, score_fn, 2.5)
    rsel, rw = _router_f64(logits, bias, k, n_group, topk_group, score_fn, 2.5, oracle.ROUTER_EPS)
    # selections identical except where f32 rounding reorders near-ties (tests/router_topk_alts.rs:97-133)
    same = (sel == rsel).all(1)
    assert same.mean() > 0.95
    assert np.abs(w[same] - rw[same]).max() < 5e-5  # tests/router_learned.rs:200-204
    assert np.allclose(w.sum(1), 2.5, atol=1e-4)
    for t in range(sel.shape[0]):
        assert len(set(sel[t])) == k


def test_router_group_limit_one_group_is_reference(oracle):
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((32, 256)).astype(np.float32)
    a = oracle.router_topk(logits, None, 6, 1, 1, 0, 1.5)
    b = oracle.router_topk(logits, None, 6, 0, 0, 0, 1.5)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_router_ties_lower_index(oracle):
    logits = np.zeros((2, 256), np.float32)
    logits[1, 200:] = 1.0
    sel, w = oracle.router_topk(logits, None, 8, 1, 1, 1, 1.0)
    assert list(sel[0]) == list(range(8))
    assert list(sel[1]) == list(range(200, 208))
    assert np.allclose(w, 1 / 8)
    # with 8 groups of 32: all group scores tie -> groups 0..3 kept
    sel, _ = oracle.router_topk(logits[:1], None, 8, 8, 4, 1, 1.0)
    assert list(sel[0]) == list(range(8))


def test_group_build_properties(oracle):
    rng = np.random.default_rng(7)
    T, k, E = 37, 6, 64
    sel = np.stack([rng.choice(E, k, replace=False) for _ in range(T)]).astype(np.int32)
    sel[3, 2] = -1          # NO_PICK is dropped
    sel[5, 0] = E + 3       # ids past the bound are dropped
    hist, offs, perm = oracle.group_build(sel, E)
    flat = sel.ravel()
    valid = (flat >= 0) & (flat < E)
    assert hist.sum() == valid.sum() == offs[-1] == perm.size
    assert np.array_equal(hist, np.bincount(flat[valid], minlength=E))
    assert np.array_equal(offs[1:], np.cumsum(hist))
    for e in range(E):
        seg = perm[offs[e]:offs[e + 1]]
        assert (flat[seg] == e).all() and (np.diff(seg) > 0).all()
    items, n = oracle.work_items(hist, 8)
    assert n == sum((h + 7) // 8 for h in hist) <= oracle.wi_upper_bound(T * k, E, 8)
    assert (np.diff(items >> 16) >= 0).all()


def test_moe_layer_slot_order_and_reference_int_path(oracle):
    """Dequantised-f32 layer vs the reference's int8 (Q8_K) arithmetic on one pick:
    through both products and the Q8_K re-quantisation of mid the two agree to the
    tolerance of the reference's routed-MoE test (max < 5e-2, mean < 1e-3 relative to
    the largest output, tests/routed_moe.rs:335-344)."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import MoeConfig, RouterConfig
    cfg = MoeConfig(hidden=512, ffn=256, shared_ffn=0, router=RouterConfig(n_expert=4, n_used=2, n_group=1, topk_group=1))
    w = synth.make_layer(cfg, 0)
    x = synth.bf16_bits_to_f32(synth.make_tokens(cfg, 0, 3))
    sel = np.array([[1, 3], [0, 1], [2, 0]], np.int32)
    wt = np.array([[0.7, 0.3], [0.5, 0.5], [1.0, 0.25]], np.float32)
    out, partials = oracle.moe_layer_f32(cfg.fmt, x, sel, wt, w["gate"], w["up"], w["down"], n_expert=4, return_partials=True)
    assert np.array_equal(out[0], (np.float32(0) + partials[0]) + partials[1])
    e = 3
    ref_int = oracle.expert_ref_int_mxfp4((w["gate"][0][e], w["gate"][1][e]), (w["up"][0][e], w["up"][1][e]),
                                          (w["down"][0][e], w["down"][1][e]), cfg.hidden, cfg.ffn, x[0], 0.3)
    d = np.abs(ref_int - partials[1]) / np.abs(partials[1]).max()
    assert d.max() < 5e-2 and d.mean() < 5e-3


def test_glue_restatements_match_plain_formulas(oracle):
    """RMSNorm and the residual mix: the order-preserving restatements agree with the textbook formulas
    in float64 (no golden vector exists for these two in the reference: parity unpinned beyond this)."""
    rng = np.random.Generator(np.random.PCG64(31))
    x = (rng.standard_normal((6, 5120)) * 2.0).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(5120)).astype(np.float32)
    got = oracle.rms_norm_rows(x, w, 1e-6)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6) * w
    assert np.abs(got - ref).max() < 2e-6 * np.abs(ref).max()
    bo = rng.standard_normal((3, 64)).astype(np.float32)
    rh = rng.standard_normal((3, 4, 64)).astype(np.float32)
    post = rng.standard_normal((3, 4)).astype(np.float32)
    comb = rng.standard_normal((3, 16)).astype(np.float32)
    got = oracle.hc_post(bo, rh, post, comb)
    ref = bo[:, None, :].astype(np.float64) * post[:, :, None] + np.einsum("tsd,tsk->tkd", rh.astype(np.float64), comb.reshape(3, 4, 4))
    assert np.abs(got - ref).max() < 1e-5


def test_activation_quantisers_match_reference_kernel_py(oracle):
    """The two activation quantisers the tensor-core path is judged with, against outputs of the reference's
    scripts/v41_oracle/kernel.py: act_quant (E4M3, block 32, ue8m0 scales; :85-106) bit for bit, and the three
    MXFP4 terms (fp4_act_quant, :129-147, applied to x and then to what each term left over) term by term."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kernelpy_vectors.npz"))
    x = g["x"]
    got = np.stack([oracle.act_quant_e4m3(r) for r in x])
    assert np.array_equal(got.view(np.uint32), g["x_fp8_dequant"].view(np.uint32))
    e2m1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    for i in range(x.shape[0]):
        codes, scales, total = oracle.act_terms_mxfp4(x[i], 3)
        acc = np.zeros_like(x[i])
        for t in range(3):
            vals = np.stack([e2m1[codes[t] & 15], e2m1[codes[t] >> 4]], 1).reshape(-1)
            term = vals * np.repeat(np.exp2(scales[t].astype(np.float32) - 127.0), 32).astype(np.float32)
            assert np.array_equal(term, g["x_fp4_terms"][t, i])      # -0.0 == 0.0: values, not sign of zero
            acc += term
        assert np.array_equal(acc, total)
    # three terms leave about 2^-9 of the row
    left = x - g["x_fp4_terms"].sum(0)
    assert np.linalg.norm(left) / np.linalg.norm(x) < 2.5e-3


def test_operand_mix_error_measured_on_config0(oracle):
    """What each tensor-core operand format costs on the layer output, measured on configuration 0 against the
    dequantised-f32 oracle (the 1e-2 target): one E4M3 term per activation (the model's own FP8 numerics) and
    one or two MXFP4 terms miss it; two E4M3 terms or three MXFP4 terms meet it with room to spare."""
    from deepstrix_b200 import synth
    from deepstrix_b200.config import CONFIGS
    cfg = CONFIGS[0]
    r = cfg.router
    w = synth.make_layer(cfg, 0)
    x = synth.bf16_bits_to_f32(synth.make_tokens(cfg, 0, 16))
    sel, wt = oracle.router_topk(oracle.router_logits(x, w["router_w"]), w["router_bias"], r.n_used, r.n_group, r.topk_group, r.score_fn,
                                 r.route_scale, r.weight_eps)
    shared = tuple((w[f"shared_{n}"][0][0], w[f"shared_{n}"][1][0]) for n in ("gate", "up", "down"))

    def run(mode):
        return oracle.moe_layer_f32(cfg.fmt, x, sel, wt, w["gate"], w["up"], w["down"], shared=shared, clamp=cfg.clamp, n_expert=r.n_expert,
                                    act_mode=mode)
    ref = run(oracle.ACT_EXACT).astype(np.float64)
    err = {name: float(np.linalg.norm(run(mode) - ref) / np.linalg.norm(ref))
           for name, mode in (("e4m3", oracle.ACT_E4M3), ("e4m3x2", oracle.ACT_E4M3_X2), ("mxfp4x1", oracle.act_mxfp4(1)),
                              ("mxfp4x2", oracle.act_mxfp4(2)), ("mxfp4x3", oracle.act_mxfp4(3)))}
    print("rel-L2 vs dequantised-f32 oracle:", {k: f"{v:.2e}" for k, v in err.items()})
    assert err["e4m3"] > 1e-2 and err["mxfp4x1"] > 1e-1 and err["mxfp4x2"] > 1e-2
    assert err["e4m3x2"] < 3e-3 and err["mxfp4x3"] < 5e-3
