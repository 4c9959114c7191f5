"""Router GEMM + top-k + softmax in one call, behind the reference's factory names.

The reference (kernels/router_gemm_topk_softmax.py) builds one TileLang kernel per algorithm and shape and hands
out a callable ``kernel(X[T,H], W[H,E]) -> (scores[T,K] float32, indices[T,K])`` with the top-k taken on the logits
and the softmax over the k selected (:1169-1203, and the six factories :149-1166 used by
tests/test_router_fusion_correctness.py).  Here every algorithm name is the same operator,
``ops.router_topk_softmax``: the tcgen05 GEMM with the selection in its epilogue (or its few-token / few-expert
forms), fp32-accumulated logits, indices int64 sorted by value with the lowest index first among equals.

The reference's weight is [H, E]; the library reads the router weight as [E, H] (K contiguous, the layout of the
fused layer), so the callable transposes it once per weight tensor and remembers the result.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch

from .. import ops as _ops

ALGORITHMS = ("cpasync_selection", "cpasync_bitonic", "tma_selection", "tma_bitonic", "tma_auto_selection",
              "tma_auto_bitonic")
_transposed: Dict[tuple, torch.Tensor] = {}


def _next_pow2(n: int) -> int:
    """Smallest power of two >= n (reference :60-66: the width it pads the expert dimension to; nothing is padded here)."""
    p = 1
    while p < n:
        p *= 2
    return p


def _weight_eh(W: torch.Tensor, E: int) -> torch.Tensor:
    key = (W.data_ptr(), W._version, tuple(W.shape), W.device, E)
    t = _transposed.get(key)
    if t is None:
        if len(_transposed) > 64:
            _transposed.clear()
        t = W[:, :E].t().contiguous()          # a padded [H, E_padded] weight is accepted: the padding is dropped
        _transposed[key] = t
    return t


def _make(num_tokens: int, H: int, E: int, top_k: int) -> Callable[[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]:
    def kernel(X: torch.Tensor, W: torch.Tensor):
        if X.shape != (num_tokens, H) or W.shape[0] != H or W.shape[1] < E:
            raise ValueError(f"built for X [{num_tokens},{H}] and W [{H},>={E}], got {tuple(X.shape)} and {tuple(W.shape)}")
        return _ops.router_topk_softmax(X, _weight_eh(W, E), top_k, mode="B")
    return kernel


def get_fused_router_kernel(algo: str, num_tokens: int, H: int, E: int, top_k: int, dtype=None, block_M: int = 64,
                            block_K: int = 64, num_stages: int = 2, threads: int = 256):
    """Callable(X, W[H,E]) -> (scores, indices); arguments as the reference's (:1169-1203).  The tuning arguments
    of the TileLang kernels are accepted and have no meaning here."""
    if algo not in ALGORITHMS:
        raise ValueError(f"Unknown algorithm: {algo}. Valid: {list(ALGORITHMS)}")
    return _make(num_tokens, H, E, top_k)


def get_router_gemm_kernel(num_tokens: int, H: int, E: int, dtype=None):
    """Callable(X[T,H], W[H,E]) -> fp32 logits [T,E]: the stand-alone router GEMM (reference :79-146), here
    ``ops.router_logits`` with fp32 accumulation."""
    def kernel(X: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
        if X.shape != (num_tokens, H) or W.shape[0] != H or W.shape[1] < E:
            raise ValueError(f"built for X [{num_tokens},{H}] and W [{H},>={E}], got {tuple(X.shape)} and {tuple(W.shape)}")
        return _ops.router_logits(X, _weight_eh(W, E))
    return kernel


def _factory(num_tokens, H, E, E_padded, top_k, block_M=64, block_K=64, num_stages=2, threads=256, dtype=None):
    """The reference's per-algorithm factories take the padded expert count as well (:149, :270, :487, :639, :858, :971)."""
    return _make(num_tokens, H, E, top_k)


fused_router_cpasync_selection_kernel = _factory
fused_router_cpasync_bitonic_kernel = _factory
fused_router_tma_selection_kernel = _factory
fused_router_tma_bitonic_kernel = _factory
fused_router_tma_auto_selection_kernel = _factory
fused_router_tma_auto_bitonic_kernel = _factory
