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


def zipf_bias(cfg: MoeConfig, s: float = 1.1, strength: float = 0.25) -> np.ndarray:
    """Router bias that skews expert popularity towards a Zipf(s) profile:
    bias_e grows with log of the target probability of rank e."""
    E = cfg.router.n_expert
    p = 1.0 / np.arange(1, E + 1, dtype=np.float64) ** s
    p /= p.sum()
    b = strength * (np.log(p) - np.log(p).mean())
    return b.astype(np.float32)
