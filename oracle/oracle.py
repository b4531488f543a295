"""ctypes front end of the CPU oracle (``dsx_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline / reference arm, never by the shipped
package.  Each wrapper names the reference file:line restated by the C function
it calls (see the C file for the full citations).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libdsx_oracle.so")

SCORE_SQRT_SOFTPLUS = 0  # kernels/router_topk.hip:71
SCORE_SIGMOID = 1        # kernels/laguna_ops.hip:59
FMT_MXFP4 = 0
FMT_Q8_0 = 1
ROUTER_EPS = 6.103515625e-5  # het/forward_layer.rs:36


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "dsx_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libdsx_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.dsxo_e8m0_half.restype = C.c_float
        _lib.dsxo_e8m0_half.argtypes = [C.c_uint8]
        _lib.dsxo_e8m0.restype = C.c_float
        _lib.dsxo_e8m0.argtypes = [C.c_uint8]
        _lib.dsxo_e4m3.restype = C.c_float
        _lib.dsxo_e4m3.argtypes = [C.c_uint8]
        _lib.dsxo_f16_to_f32.restype = C.c_float
        _lib.dsxo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.dsxo_f32_to_f16.restype = C.c_uint16
        _lib.dsxo_f32_to_f16.argtypes = [C.c_float]
        _lib.dsxo_det_expf.restype = C.c_float
        _lib.dsxo_det_expf.argtypes = [C.c_float]
        _lib.dsxo_det_log1pf.restype = C.c_float
        _lib.dsxo_det_log1pf.argtypes = [C.c_float]
        _lib.dsxo_router_prob.restype = C.c_float
        _lib.dsxo_router_prob.argtypes = [C.c_float, C.c_int]
        _lib.dsxo_dot_mxfp4_q8k.restype = C.c_float
        _lib.dsxo_group_build.restype = C.c_int64
        _lib.dsxo_work_items.restype = C.c_int32
        _lib.dsxo_wi_upper_bound.restype = C.c_uint32
        _lib.dsxo_wi_upper_bound.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64]
        _lib.dsxo_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().dsxo_num_threads())


# ----------------------------------------------------------------- scalars
def e8m0_half(e: int) -> float:
    return float(lib().dsxo_e8m0_half(int(e)))


def e8m0(e: int) -> float:
    return float(lib().dsxo_e8m0(int(e)))


def e4m3(b: int) -> float:
    return float(lib().dsxo_e4m3(int(b)))


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().dsxo_f32_to_bf16(_p(x), _p(y), C.c_int64(x.size))
    return y


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.uint16)
    y = np.empty(x.shape, np.float32)
    lib().dsxo_bf16_to_f32(_p(x), _p(y), C.c_int64(x.size))
    return y


# ------------------------------------------------------------ MXFP4 / Q8_0
def mxfp4_dequant_ggml(blocks: np.ndarray) -> np.ndarray:
    blocks = _c(blocks, np.uint8).reshape(-1)
    nb = blocks.size // 17
    out = np.empty(nb * 32, np.float32)
    lib().dsxo_mxfp4_dequant_ggml(_p(blocks), C.c_int64(nb), _p(out))
    return out


def mxfp4_dequant_sb2(sb: np.ndarray) -> np.ndarray:
    sb = _c(sb, np.uint8).reshape(-1)
    ns = sb.size // 136
    out = np.empty(ns * 256, np.float32)
    lib().dsxo_mxfp4_dequant_sb2(_p(sb), C.c_int64(ns), _p(out))
    return out


def mxfp4_dequant_hf(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    packed = _c(packed, np.uint8)
    scales = _c(scales, np.uint8)
    rows, half = packed.shape
    out = np.empty((rows, half * 2), np.float32)
    lib().dsxo_mxfp4_dequant_hf(_p(packed), _p(scales), C.c_int64(rows), C.c_int64(half * 2), _p(out))
    return out


def mxfp4_repack_hf_to_sb2(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    packed = _c(packed, np.uint8)
    scales = _c(scales, np.uint8)
    rows, half = packed.shape
    K = half * 2
    dst = np.empty((rows, K // 32 * 17), np.uint8)
    lib().dsxo_mxfp4_repack_hf_to_sb2(_p(packed), _p(scales), C.c_int64(rows), C.c_int64(K), _p(dst))
    return dst


def mxfp4_repack_ggml_to_hf(blocks: np.ndarray, rows: int, K: int):
    blocks = _c(blocks, np.uint8).reshape(-1)
    packed = np.empty((rows, K // 2), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    lib().dsxo_mxfp4_repack_ggml_to_hf(_p(blocks), C.c_int64(rows), C.c_int64(K), _p(packed), _p(scales))
    return packed, scales


def mxfp4_repack_sb2_to_hf(sb: np.ndarray, rows: int, K: int):
    sb = _c(sb, np.uint8).reshape(-1)
    packed = np.empty((rows, K // 2), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    lib().dsxo_mxfp4_repack_sb2_to_hf(_p(sb), C.c_int64(rows), C.c_int64(K), _p(packed), _p(scales))
    return packed, scales


def q8_0_quantize_block(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(34, np.uint8)
    lib().dsxo_q8_0_quantize_block(_p(x), _p(out))
    return out


def q8_0_dequant(blocks: np.ndarray) -> np.ndarray:
    blocks = _c(blocks, np.uint8).reshape(-1)
    nb = blocks.size // 34
    out = np.empty(nb * 32, np.float32)
    lib().dsxo_q8_0_dequant(_p(blocks), C.c_int64(nb), _p(out))
    return out


def q8_0_quantize_act(x: np.ndarray):
    x = _c(x, np.float32).reshape(-1)
    nb = x.size // 32
    xq = np.empty(nb * 32, np.int8)
    xs = np.empty(nb, np.float32)
    lib().dsxo_q8_0_quantize_act(_p(x), C.c_int64(nb), _p(xq), _p(xs))
    return xq, xs


def q8_k_quantize(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1)
    nb = x.size // 256
    out = np.empty(nb * 292, np.uint8)
    lib().dsxo_q8_k_quantize(_p(x), C.c_int64(nb), _p(out))
    return out


def swiglu_clamp_weighted(gate: np.ndarray, up: np.ndarray, expert_w: np.ndarray, clamp: float, use_det: bool = True) -> np.ndarray:
    """[n_experts, ff_exp] f32.  use_det: the exponential from IEEE add / mul / fma only (what the CUDA operator evaluates);
    False: libm's expf, as the reference source reads."""
    g, u, w = _c(gate, np.float32), _c(up, np.float32), _c(expert_w, np.float32).reshape(-1)
    n, ff = g.shape
    out = np.empty((n, ff), np.float32)
    lib().dsxo_swiglu_clamp_weighted(_p(out), _p(g), _p(u), _p(w), C.c_float(clamp), C.c_int64(ff), C.c_int64(n), C.c_int(1 if use_det else 0))
    return out


def dot_mxfp4_q8k(w_sb2: np.ndarray, y_q8k: np.ndarray) -> float:
    w = _c(w_sb2, np.uint8).reshape(-1)
    y = _c(y_q8k, np.uint8).reshape(-1)
    return float(lib().dsxo_dot_mxfp4_q8k(C.c_int64(w.size // 136), _p(w), _p(y)))


def dequant_matrix(fmt: int, q: np.ndarray, s: np.ndarray, rows: int, K: int) -> np.ndarray:
    q = np.ascontiguousarray(q).view(np.uint8)
    s = np.ascontiguousarray(s).view(np.uint8)
    out = np.empty((rows, K), np.float32)
    lib().dsxo_dequant_matrix(C.c_int(fmt), _p(q), _p(s), C.c_int64(rows), C.c_int64(K), _p(out))
    return out


# ----------------------------------------------------------------- router
def router_prob(logit: float, score_fn: int) -> float:
    return float(lib().dsxo_router_prob(C.c_float(logit), score_fn))


def router_logits(x: np.ndarray, W: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    W = _c(W, np.float32)
    T, H = x.shape
    E = W.shape[0]
    out = np.empty((T, E), np.float32)
    lib().dsxo_router_logits(_p(x), _p(W), C.c_int64(T), C.c_int(E), C.c_int64(H), _p(out))
    return out


def router_topk(logits, bias, n_used, n_group=1, topk_group=1, score_fn=SCORE_SIGMOID,
                scale=1.0, eps=ROUTER_EPS):
    logits = _c(logits, np.float32)
    T, E = logits.shape
    b = None if bias is None else _c(bias, np.float32)
    sel = np.empty((T, n_used), np.int32)
    w = np.empty((T, n_used), np.float32)
    lib().dsxo_router_topk(_p(logits), _p(b), C.c_int64(T), C.c_int(E), C.c_int(n_used),
                           C.c_int(n_group), C.c_int(topk_group), C.c_int(score_fn),
                           C.c_float(scale), C.c_float(eps), _p(sel), _p(w))
    return sel, w


def router_topk_ex(logits, bias, n_used, n_alt, n_group=1, topk_group=1, score_fn=SCORE_SIGMOID,
                   scale=1.0, eps=ROUTER_EPS):
    """router_topk plus the alternatives (ranks n_used+1 .. n_used+n_alt), their weights and the score range."""
    logits = _c(logits, np.float32)
    T, E = logits.shape
    b = None if bias is None else _c(bias, np.float32)
    sel = np.empty((T, n_used), np.int32)
    w = np.empty((T, n_used), np.float32)
    alts = np.empty((T, max(n_alt, 1)), np.int32)
    alt_w = np.empty((T, max(n_alt, 1)), np.float32)
    rng = np.empty((T,), np.float32)
    lib().dsxo_router_topk_ex(_p(logits), _p(b), C.c_int64(T), C.c_int(E), C.c_int(n_used),
                              C.c_int(n_group), C.c_int(topk_group), C.c_int(score_fn),
                              C.c_float(scale), C.c_float(eps), _p(sel), _p(w), C.c_int(n_alt), _p(alts), _p(alt_w), _p(rng))
    return sel, w, alts[:, :n_alt], alt_w[:, :n_alt], rng


def router_topk_prior(logits, bias, n_used, n_alt, prior, n_protect, prior_dry=False, score_fn=SCORE_SIGMOID, scale=1.0, eps=ROUTER_EPS):
    """Top-k with the reference's cache prior: (selected, weights, alts, alt_weights, orig_sel)."""
    logits = _c(logits, np.float32)
    T, E = logits.shape
    b = None if bias is None else _c(bias, np.float32)
    pr = _c(prior, np.float32)
    sel = np.empty((T, n_used), np.int32)
    w = np.empty((T, n_used), np.float32)
    alts = np.empty((T, max(n_alt, 1)), np.int32)
    alt_w = np.empty((T, max(n_alt, 1)), np.float32)
    orig = np.empty((T, n_used), np.int32)
    lib().dsxo_router_topk_prior(_p(logits), _p(b), C.c_int64(T), C.c_int(E), C.c_int(n_used), C.c_int(score_fn), C.c_float(scale),
                                 C.c_float(eps), _p(sel), _p(w), C.c_int(n_alt), _p(alts), _p(alt_w), _p(pr), C.c_int(n_protect),
                                 C.c_int(1 if prior_dry else 0), _p(orig))
    return sel, w, alts[:, :n_alt], alt_w[:, :n_alt], orig


def rms_norm_rows(x, weight, eps=1e-6):
    x = _c(x, np.float32)
    w = _c(weight, np.float32)
    T, n = x.shape
    out = np.empty((T, n), np.float32)
    lib().dsxo_rms_norm_rows(_p(x), _p(w), C.c_int64(T), C.c_int64(n), C.c_float(eps), _p(out))
    return out


def hc_post(block_out, residual_hc, post, comb):
    bo = _c(block_out, np.float32)
    rh = _c(residual_hc, np.float32)
    T, n_hc, n = rh.shape
    out = np.empty((T, n_hc, n), np.float32)
    lib().dsxo_hc_post(_p(bo), _p(rh), _p(_c(post, np.float32)), _p(_c(comb, np.float32)), C.c_int64(T), C.c_int64(n), C.c_int(n_hc), _p(out))
    return out


def group_build(selected: np.ndarray, n_expert: int):
    selected = _c(selected, np.int32)
    T, k = selected.shape
    hist = np.empty(n_expert, np.int32)
    offs = np.empty(n_expert + 1, np.int32)
    perm = np.full(max(T * k, 1), -1, np.int32)
    n = lib().dsxo_group_build(_p(selected), C.c_int64(T), C.c_int(k), C.c_int(n_expert),
                               _p(hist), _p(offs), _p(perm))
    return hist, offs, perm[:n]


def work_items(hist: np.ndarray, chunk: int, cap: int | None = None) -> np.ndarray:
    hist = _c(hist, np.int32)
    cap = int(cap if cap is not None else hist.sum() + hist.size)
    items = np.empty(max(cap, 1), np.int32)
    n = lib().dsxo_work_items(_p(hist), C.c_int(hist.size), C.c_int(chunk), _p(items), C.c_int32(cap))
    return items[:min(n, cap)], int(n)


def wi_upper_bound(members: int, groups: int, chunk: int, cap: int = 2**62) -> int:
    return int(lib().dsxo_wi_upper_bound(members, groups, chunk, cap))


# -------------------------------------------------------------- MoE layer
ACT_EXACT, ACT_E4M3, ACT_E4M3_X2 = 0, 1, 2


def act_mxfp4(n_terms: int) -> int:
    """act_mode of ``moe_layer_f32``: activations as a sum of n_terms MXFP4 rows."""
    return 10 + n_terms


def act_quant_e4m3(x: np.ndarray) -> np.ndarray:
    """scripts/v41_oracle/kernel.py:85-106 (act_quant, block 32, ue8m0 scales): the dequantised result."""
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().dsxo_act_quant_e4m3(_p(x), C.c_int64(x.size), _p(out))
    return out


def act_terms_mxfp4(x: np.ndarray, n_terms: int = 3):
    """One row -> (codes uint8 [n_terms, n/2], E8M0 scales uint8 [n_terms, n/32], sum of the terms f32 [n]);
    term t is kernel.py's fp4_act_quant (:129-147) of what the earlier terms left over."""
    x = _c(x, np.float32).reshape(-1)
    n = x.size
    codes = np.zeros((n_terms, n // 2), np.uint8)
    scales = np.zeros((n_terms, n // 32), np.uint8)
    total = np.empty(n, np.float32)
    lib().dsxo_act_terms_mxfp4(_p(x), C.c_int64(n), C.c_int(n_terms), _p(codes), _p(scales), _p(total))
    return codes, scales, total


def moe_layer_f32(fmt, x, selected, weights, gate, up, down, shared=None, shared_fmt=None,
                  clamp=10.0, mid_round=0, n_expert=None, return_partials=False, act_mode=0):
    """Dequantised-f32 MoE layer.  gate/up/down are ``(q, s)`` pairs holding all
    experts back to back; ``shared`` is ``((gq,gs),(uq,us),(dq,ds))`` or None.
    act_mode: how the two products see their activation rows (0 exact -- the tolerance target;
    ACT_E4M3 / ACT_E4M3_X2 / act_mxfp4(k), see apply_act_mode in the C file)."""
    x = _c(x, np.float32)
    T, H = x.shape
    selected = _c(selected, np.int32)
    weights = _c(weights, np.float32)
    k = selected.shape[1]
    gq, gs = (np.ascontiguousarray(a).view(np.uint8) for a in gate)
    uq, us = (np.ascontiguousarray(a).view(np.uint8) for a in up)
    dq, ds = (np.ascontiguousarray(a).view(np.uint8) for a in down)
    E = int(n_expert)
    per_q = gq.size // E
    F = (per_q * 2 // H) if fmt == FMT_MXFP4 else (per_q // H)
    sh = [None] * 6
    Fs = 0
    sfmt = fmt if shared_fmt is None else shared_fmt
    if shared is not None:
        sh = [np.ascontiguousarray(a).view(np.uint8) for pair in shared for a in pair]
        Fs = (sh[0].size * 2 // H) if sfmt == FMT_MXFP4 else (sh[0].size // H)
    out = np.empty((T, H), np.float32)
    partials = np.empty((T * k + T, H), np.float32) if return_partials else None
    lib().dsxo_moe_layer_act(
        C.c_int(fmt), C.c_int64(T), C.c_int64(H), C.c_int64(F), C.c_int(E), C.c_int(k),
        _p(x), _p(selected), _p(weights), _p(gq), _p(gs), _p(uq), _p(us), _p(dq), _p(ds),
        C.c_int(sfmt), C.c_int64(Fs), *[_p(a) for a in sh],
        C.c_float(clamp), C.c_int(mid_round), C.c_int(act_mode), _p(out), _p(partials))
    return (out, partials) if return_partials else out


def expert_ref_int_mxfp4(gate, up, down, H, F, x, w, clamp=10.0) -> np.ndarray:
    """One routed pick through the reference's int8 (Q8_K) arithmetic."""
    gq, gs = (_c(a, np.uint8) for a in gate)
    uq, us = (_c(a, np.uint8) for a in up)
    dq, ds = (_c(a, np.uint8) for a in down)
    x = _c(x, np.float32)
    out = np.empty(H, np.float32)
    lib().dsxo_expert_ref_int_mxfp4(_p(gq), _p(gs), _p(uq), _p(us), _p(dq), _p(ds), C.c_int64(H),
                                    C.c_int64(F), C.c_float(clamp), _p(x), C.c_float(w), _p(out))
    return out
