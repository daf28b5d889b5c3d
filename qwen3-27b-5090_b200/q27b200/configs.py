"""Seeded synthetic inputs for the five benchmark configurations (shapes, distributions and seeds only; no model
checkpoint or dataset is involved). Activations use seed = configuration index, weights seed = 1000 + index
(configuration 3: 1000 * (layer + 1) + projection index); all draws are torch.randn on the CPU generator, so the
same tensors can be rebuilt anywhere. The activation tensor scale is amax(x) / (6 * 448), the static-calibration
stand-in the reference derives the same way for its own weights (engine/src/weights.cc:484).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

HIDDEN, INTER, KV = 5120, 17408, 1024
LAYERS = 64
SWEEP_M = (1, 2, 4, 8, 16, 32, 64, 128)
# name, N (weight rows), K, fused SiLU*mul epilogue
LAYER_PROJECTIONS = (("q", HIDDEN, HIDDEN, False), ("k", KV, HIDDEN, False), ("v", KV, HIDDEN, False),
                     ("o", HIDDEN, HIDDEN, False), ("gate_up", 2 * INTER, HIDDEN, True), ("down", HIDDEN, INTER, False))


@dataclass(frozen=True)
class GemmConfig:
    index: int
    name: str
    M: int
    N: int        # weight rows (gate and up together for glu)
    K: int
    glu: bool
    x_std: float = 1.0
    w_std: float = 0.02

    @property
    def n_out(self) -> int:
        return self.N // 2 if self.glu else self.N

    def algorithmic_bytes(self, M: int | None = None) -> int:
        M = self.M if M is None else M
        return self.N * self.K // 2 + self.N * self.K // 16 + 2 * M * self.K + 2 * M * self.n_out

    def flops(self, M: int | None = None) -> int:
        return 2 * (self.M if M is None else M) * self.N * self.K


CONFIGS = {
    0: GemmConfig(0, "cfg0 decode GEMV 1x5120x5120", 1, HIDDEN, HIDDEN, False),
    1: GemmConfig(1, "cfg1 verify gate_up 16x34816x5120 SiLU*mul", 16, 2 * INTER, HIDDEN, True),
    2: GemmConfig(2, "cfg2 verify down 128x5120x17408", 128, HIDDEN, INTER, False, x_std=0.5),
    4: GemmConfig(4, "cfg4 prefill gate_up 4096x34816x5120 SiLU*mul", 4096, 2 * INTER, HIDDEN, True),
}


def layer_weight_bytes() -> int:
    return sum(n * k // 2 + n * k // 16 for _, n, k, _ in LAYER_PROJECTIONS)


def sweep_algorithmic_bytes(M: int, layers: int = LAYERS) -> int:
    per_layer = 0
    for _, n, k, glu in LAYER_PROJECTIONS:
        per_layer += n * k // 2 + n * k // 16 + 2 * M * k + 2 * M * (n // 2 if glu else n)
    return per_layer * layers


def make_x(cfg: GemmConfig, M: int | None = None, seed: int | None = None) -> torch.Tensor:
    g = torch.Generator().manual_seed(cfg.index if seed is None else seed)
    x = torch.randn(cfg.M if M is None else M, cfg.K, generator=g, dtype=torch.float32) * cfg.x_std
    return x.to(torch.bfloat16)


def make_w(N: int, K: int, seed: int, std: float = 0.02, rows: slice | None = None) -> torch.Tensor:
    """fp32 [N][K] ~ N(0, std); `rows` returns only that slice of the same matrix (generated in full on the CPU)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g, dtype=torch.float32) * std
    return w if rows is None else w[rows].contiguous()


def input_scale_of(x: torch.Tensor) -> float:
    return float(torch.div(x.float().abs().amax(), torch.tensor(6.0 * 448.0, device=x.device)))
