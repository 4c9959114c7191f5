"""Seeded synthetic inputs for the benchmark workloads (CPU generators, so every rank and the
CPU baseline see the same batch)."""
from __future__ import annotations

import torch


def zipf_logits(T: int, E: int, s: float = 1.1, seed: int = 0, noise_seed=None) -> torch.Tensor:
    """fp32 router logits [T,E] whose top-k routing follows a Zipf(s) expert popularity:
    log p[pi(e)] + Gumbel(0,1) noise with p_r proportional to r^-s and pi a seeded permutation
    of the expert ids (sampling without replacement under the popularity law).  `seed` fixes
    the popularity permutation; `noise_seed` (default: continue the same stream) draws another
    batch under the same popularity."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    ranks = torch.arange(1, E + 1, dtype=torch.float64)
    p = ranks.pow(-s)
    p = p / p.sum()
    pi = torch.randperm(E, generator=g)
    logp = torch.empty(E, dtype=torch.float64)
    logp[pi] = p.log()
    if noise_seed is not None:
        g = torch.Generator(device="cpu")
        g.manual_seed(noise_seed)
    u = torch.rand(T, E, generator=g, dtype=torch.float64).clamp_(1e-12, 1 - 1e-12)
    gumbel = -(-(u.log())).log()
    return (logp[None, :] + gumbel).to(torch.float32)


def activations(T: int, H: int, seed: int = 0) -> torch.Tensor:
    """bf16 activations [T,H] ~ N(0,1)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return torch.randn(T, H, generator=g, dtype=torch.float32).bfloat16()
