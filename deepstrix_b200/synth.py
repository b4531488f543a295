"""Seeded synthetic workloads with the shapes and value distributions of the
benchmark configurations (there is no dataset behind this path; the reference
benchmarks also run on generated weights and random distinct picks,
crates/v4flash-kernels/tests/bench_v41_kernel_roofline.rs:604-658)."""
from __future__ import annotations

import numpy as np

from .config import FMT_MXFP4, MoeConfig, SEED_BASE


def rng_for(config_id: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([SEED_BASE + config_id, stream]))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_matrix(rng, fmt: int, n: int, rows: int, k: int):
    """n matrices [rows, k] in the canonical host layout.
    MXFP4: (codes uint8 [n, rows, k/2] uniform over the 16 codes, E8M0 uint8
    [n, rows, k/32] = 127 + u, u uniform in [-8, -4]).
    Q8_0: (int8 [n, rows, k] uniform in [-127, 127], f16 [n, rows, k/32] ~ U(1e-3, 1e-2))."""
    if fmt == FMT_MXFP4:
        q = rng.integers(0, 256, size=(n, rows, k // 2), dtype=np.uint8)
        s = rng.integers(119, 124, size=(n, rows, k // 32), dtype=np.uint8)
        return q, s
    q = rng.integers(-127, 128, size=(n, rows, k), dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, size=(n, rows, k // 32)).astype(np.float16)
    return q, s


def make_layer(cfg: MoeConfig, config_id: int, layer: int = 0, n_expert: int | None = None):
    """Weights of one layer: dict with gate/up/down (q, s) for all routed
    experts, shared_* for the shared expert, router_w f32 N(0, 0.02), router_bias
    f32 N(0, 0.01)."""
    rng = rng_for(config_id, 1000 + layer)
    E = cfg.router.n_expert if n_expert is None else n_expert
    out = {
        "gate": make_matrix(rng, cfg.fmt, E, cfg.ffn, cfg.hidden),
        "up": make_matrix(rng, cfg.fmt, E, cfg.ffn, cfg.hidden),
        "down": make_matrix(rng, cfg.fmt, E, cfg.hidden, cfg.ffn),
    }
    if cfg.shared_ffn:
        out["shared_gate"] = make_matrix(rng, cfg.fmt, 1, cfg.shared_ffn, cfg.hidden)
        out["shared_up"] = make_matrix(rng, cfg.fmt, 1, cfg.shared_ffn, cfg.hidden)
        out["shared_down"] = make_matrix(rng, cfg.fmt, 1, cfg.hidden, cfg.shared_ffn)
    out["router_w"] = rng.normal(0.0, 0.02, size=(cfg.router.n_expert, cfg.hidden)).astype(np.float32)
    out["router_bias"] = rng.normal(0.0, 0.01, size=(cfg.router.n_expert,)).astype(np.float32)
    return out


def make_tokens(cfg: MoeConfig, config_id: int, T: int, stream: int = 0) -> np.ndarray:
    """N(0,1) activations as bf16 bit patterns, uint16 [T, hidden]."""
    rng = rng_for(config_id, 2000 + stream)
    return f32_to_bf16_bits(rng.standard_normal((T, cfg.hidden), dtype=np.float32))


def uniform_logits(cfg: MoeConfig, config_id: int, T: int) -> np.ndarray:
    """Logits that make routing uniform-random (k distinct experts per token)."""
    rng = rng_for(config_id, 3000)
    return rng.standard_normal((T, cfg.router.n_expert), dtype=np.float32)


def _route_numpy(logits: np.ndarray, bias: np.ndarray, cfg: MoeConfig) -> np.ndarray:
    """Plain numpy restatement of the router's selection (sigmoid or sqrt-softplus scores + bias,
    optional group limit, top-k), used only to calibrate synthetic biases: returns picks [T, k]."""
    r = cfg.router
    lg = logits.astype(np.float64)
    p = 1.0 / (1.0 + np.exp(-lg)) if r.score_fn == 1 else np.sqrt(np.log1p(np.exp(lg)))
    s = p + bias.astype(np.float64)
    T, E = s.shape
    if r.n_group > 1:
        per = E // r.n_group
        gs = np.sort(s.reshape(T, r.n_group, per), axis=2)[:, :, -2:].sum(2)
        keep = np.zeros((T, r.n_group), bool)
        np.put_along_axis(keep, np.argsort(-gs, axis=1, kind="stable")[:, : r.topk_group], True, axis=1)
        s = np.where(np.repeat(keep, per, axis=1), s, -np.inf)
    return np.argsort(-s, axis=1, kind="stable")[:, : r.n_used]


def zipf_bias(cfg: MoeConfig, logits: np.ndarray | None = None, s: float = 1.1, seed: int = 3) -> np.ndarray:
    """Router bias that skews expert popularity towards a Zipf(s) profile (expert e has rank e+1).
    bias = c * (log p_e - mean), with the single strength c found by bisection so that the 32
    most popular experts receive the share of picks the (capped) Zipf profile gives them; one
    pick per token caps an expert's share at 1/k.  A per-expert fit is not attempted: with a
    group limit the experts' popularities are coupled and such a fit does not converge.
    Calibrated on a sample of router logits (default: N(0, 1.28), the logit distribution of
    N(0, 0.02) router weights on N(0, 1) activations of width 4096)."""
    E, k = cfg.router.n_expert, cfg.router.n_used
    if logits is None:
        logits = np.random.Generator(np.random.PCG64([SEED_BASE + seed, 77])).normal(0.0, 1.28, size=(2048, E)).astype(np.float32)
    target = 1.0 / np.arange(1, E + 1, dtype=np.float64) ** s
    target /= target.sum()
    shape = np.log(target) - np.log(target).mean()
    for _ in range(8):                       # cap at one pick per token, renormalise the rest
        over = target > 1.0 / k
        if not over.any():
            break
        target[over] = 1.0 / k
        target[~over] *= (1.0 - over.sum() / k) / target[~over].sum()
    head = min(32, E // 2)
    want = target[:head].sum()
    lo, hi = 0.0, 1.0
    for _ in range(14):
        c = 0.5 * (lo + hi)
        sel = _route_numpy(logits, c * shape, cfg)
        got = (sel < head).mean()
        lo, hi = (c, hi) if got < want else (lo, c)
    return (0.5 * (lo + hi) * shape).astype(np.float32)
