"""Seeded synthetic inputs for the benchmark workloads (host side, numpy only).

The reference names no dataset; every workload runs on tensors drawn from these generators: activations ~ N(0, 1),
weights ~ N(0, sigma), bias ~ N(0, 0.1), and MoE token counts ~ Multinomial(tokens, Dirichlet(alpha)).  The seed of a
tensor is the triple (0, config number, tensor id), so the parity tests and the benchmark see the same data.
"""
import numpy as np


def rng_for(cfg: int, tensor_id: int) -> np.random.Generator:
    return np.random.default_rng(np.random.SeedSequence([0, cfg, tensor_id]))


def normal_f32(cfg: int, tensor_id: int, shape, sigma: float) -> np.ndarray:
    x = rng_for(cfg, tensor_id).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x


def moe_group_rows(cfg: int = 4, groups: int = 128, tokens: int = 32768, alpha: float = 0.5) -> np.ndarray:
    """Rows of A owned by each expert; some experts get none, a few get thousands."""
    r = rng_for(cfg, 4)
    p = r.dirichlet(np.full(groups, alpha))
    return r.multinomial(tokens, p).astype(np.int64)
