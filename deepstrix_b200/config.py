"""Layer shapes and router settings (plain data, no device code).

The numbered configurations are the benchmark's five workloads; reference
defaults they derive from: crates/v4flash-kernels/src/config.rs:10,65-76,104-105
(hidden 4096, 256 experts, top-6, ffn 2048, scale 1.5, clamp 10) and
het/forward_layer.rs:36 (weight eps).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

FMT_MXFP4 = 0
FMT_Q8_0 = 1
SCORE_SQRT_SOFTPLUS = 0
SCORE_SIGMOID = 1
ROUTER_EPS = 6.103515625e-5


@dataclass(frozen=True)
class RouterConfig:
    n_expert: int = 256
    n_used: int = 8
    n_group: int = 8
    topk_group: int = 4
    score_fn: int = SCORE_SIGMOID
    route_scale: float = 2.5
    weight_eps: float = ROUTER_EPS


@dataclass(frozen=True)
class MoeConfig:
    hidden: int = 4096
    ffn: int = 2048
    shared_ffn: int = 2048          # 0 = no shared expert
    fmt: int = FMT_MXFP4
    clamp: float = 10.0
    router: RouterConfig = field(default_factory=RouterConfig)
    name: str = "full"

    def with_(self, **kw) -> "MoeConfig":
        return replace(self, **kw)

    # bytes of one matrix / one expert in HBM (17 or 34 bytes per 32 weights)
    def matrix_bytes(self, rows=None, k=None) -> int:
        rows = self.ffn if rows is None else rows
        k = self.hidden if k is None else k
        return rows * (k // 32) * (17 if self.fmt == FMT_MXFP4 else 34)

    def expert_bytes(self) -> int:
        return 3 * self.matrix_bytes()

    def algorithmic_bytes(self, tokens: int, distinct_experts: int) -> int:
        """Weights of every distinct expert touched once + shared expert +
        router weights + bf16 token rows in and out."""
        shared = 3 * self.matrix_bytes(self.shared_ffn) if self.shared_ffn else 0
        return (distinct_experts * self.expert_bytes() + shared + self.router.n_expert * self.hidden * 4
                + tokens * self.hidden * 4)

    def flops(self, tokens: int) -> float:
        routed = 2.0 * 3 * tokens * self.router.n_used * self.ffn * self.hidden
        shared = 2.0 * 3 * tokens * self.shared_ffn * self.hidden
        router = 2.0 * tokens * self.router.n_expert * self.hidden
        return routed + shared + router


_SMALL = MoeConfig(hidden=2048, ffn=1024, shared_ffn=1024, name="small",
                   router=RouterConfig(n_expert=64, n_used=6, n_group=8, topk_group=4))
_FULL = MoeConfig(name="full")

CONFIGS = {
    0: _SMALL,                                          # 16 fp32 tokens, CPU-runnable
    1: _FULL.with_(name="decode"),                      # T in {1, 8, 32, 64}
    2: _FULL.with_(name="prefill"),                     # T = 8192, uniform-random routing
    3: _FULL.with_(name="q8_0_zipf", fmt=FMT_Q8_0),     # T = 2048, Zipf(1.1) expert popularity
    4: _FULL.with_(name="ep_stack"),                    # 8 layers, experts sharded over the GPUs
}
SEED_BASE = 0xD5EE0000
