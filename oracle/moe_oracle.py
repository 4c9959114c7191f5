"""CPU oracle for the MoE-layer hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU, what the reference's PyTorch
baseline path computes.  It exists to check the CUDA library; it is never part
of the shipped path.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it.

The arithmetic of the reference baseline lives in PyTorch itself (``torch.topk``,
``F.softmax``, ``@``, ``scatter_reduce_``; reference ``requirements.txt:3``,
``torch>=2.0.0``).  The oracle therefore calls the same torch primitives on CPU,
with two canonicalisations that make bit-exact comparison possible:

* ``torch.topk`` leaves the order of equal values unspecified.  The oracle uses a
  stable descending sort, so equal values come out lowest index first.
* "fp32-accumulated reference" for bf16 GEMM / MoE outputs means: the same
  operations evaluated on ``.float()`` copies of the bf16-rounded inputs.

Pinning: ``oracle/pin_against_reference.py`` runs the reference's own
``kernels/*_baseline.py`` side by side with this module and writes the fixtures
under ``tests/golden/``; ``tests/test_oracle.py`` replays them.  The reference
ships no golden vectors of its own for this path, so those fixtures (outputs of
the reference code itself) are the pin.

Reference citations use paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

MODE_B = 0          # topk on logits, softmax over the k selected
MODE_A = 1          # softmax over all N, then pick k (scores sum < 1)
MODE_A_RENORM = 2   # as MODE_A, then renormalise the k scores to sum 1

_MODE_NAMES = {"B": MODE_B, "A": MODE_A, "A_norenorm": MODE_A, "A_renorm": MODE_A_RENORM}


def _mode(mode) -> int:
    if isinstance(mode, str):
        return _MODE_NAMES[mode]
    return int(mode)


# --------------------------------------------------------------------------- routing
def stable_topk(values: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k along the last dim, sorted descending, equal values lowest index first.

    Replaces ``torch.topk`` (kernels/topk_softmax_baseline.py:31,61) whose tie
    order is unspecified.  -0.0 and +0.0 compare equal; NaN sorts as the largest
    value (torch's sort convention).
    """
    sv, si = torch.sort(values, dim=-1, descending=True, stable=True)
    return sv[..., :k].contiguous(), si[..., :k].contiguous()


def topk_softmax(logits: torch.Tensor, k: int, mode="B") -> Tuple[torch.Tensor, torch.Tensor]:
    """Router op.  Returns (scores fp32 [M,k], indices int64 [M,k]).

    mode B          kernels/topk_softmax_baseline.py:39-66  (topk_softmax_fused)
    mode A          kernels/topk_softmax_baseline.py:15-36  (topk_softmax_separate);
                    also the FusedMoE router, kernels/fusedmoe_baseline.py:73-76
    mode A_renorm   kernels/topk_softmax_baseline.py:223-236

    Selection is always made on the logits.  For modes A / A_renorm the reference
    selects on the softmax scores; softmax is monotone non-decreasing in the
    logit, so the two selections agree except where rounding maps two different
    logits to one score (see ``selection_is_score_stable``).
    """
    m = _mode(mode)
    logits = logits.to(torch.float32)
    if m == MODE_B:
        vals, idx = stable_topk(logits, k)
        return F.softmax(vals, dim=-1, dtype=torch.float32), idx
    probs = F.softmax(logits, dim=-1, dtype=torch.float32)
    _, idx = stable_topk(logits, k)
    sc = torch.gather(probs, -1, idx)
    if m == MODE_A_RENORM:
        sc = sc / sc.sum(dim=-1, keepdim=True)
    return sc, idx


def selection_is_score_stable(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Per row: True where top-k by stable sort of the softmax scores equals top-k
    by stable sort of the logits (the reference's literal mode-A selection)."""
    probs = F.softmax(logits.float(), dim=-1, dtype=torch.float32)
    _, i_p = stable_topk(probs, k)
    _, i_l = stable_topk(logits.float(), k)
    return (i_p == i_l).all(dim=-1)


def rows_with_ties(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Per row: True if any two of the top-(k+1) values are equal (so the
    reference's unmodified ``torch.topk`` may legally order them either way)."""
    kk = min(k + 1, logits.shape[-1])
    sv, _ = torch.sort(logits.float(), dim=-1, descending=True, stable=True)
    sv = sv[..., :kk]
    return (sv[..., 1:] == sv[..., :-1]).any(dim=-1)


def route_histogram(topk_indices: torch.Tensor, n_experts: int):
    """Permutation / histogram stage, kernels/fusedmoe_baseline.py:123-134.

    Returns (counts int32 [E], offsets int32 [E+1] exclusive, perm int32 [T*k],
    inv int32 [T*k]).  ``offsets[1:]`` equals the reference's inclusive
    ``counts.cumsum()``; ``perm`` is the stable argsort of the flattened expert
    ids (the canonical form of the reference's unstable ``argsort``); ``inv`` is
    its inverse (sorted position of every flat (token, slot) entry).
    """
    flat = topk_indices.reshape(-1).to(torch.int64)
    perm = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n_experts)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=torch.int64)
    return counts.to(torch.int32), offsets.to(torch.int32), perm.to(torch.int32), inv.to(torch.int32)


# --------------------------------------------------------------------------- grouped GEMM
def grouped_gemm(X: torch.Tensor, W: torch.Tensor, expert_indices: torch.Tensor,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Y[i] = X[i] @ W[expert_indices[i]].T, kernels/grouped_gemm_baseline.py:14-57.

    X [T,H], W [E,I,H], expert_indices [T] (or [T,k] -> Y [T,k,I]).  Computed on
    fp32 copies (fp32 accumulate); ``out_dtype`` None keeps fp32, else the result
    is rounded once to that dtype like the reference's matmul output.
    """
    two_d = expert_indices.dim() == 2
    if two_d:
        k = expert_indices.shape[1]
        Xr = X.repeat_interleave(k, dim=0)
        idx = expert_indices.reshape(-1)
    else:
        Xr, idx = X, expert_indices
    E, I, H = W.shape
    Xf = Xr.float()
    Y = torch.zeros(Xr.shape[0], I, dtype=torch.float32)
    for e in range(E):
        rows = (idx == e).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        Y[rows] = Xf[rows] @ W[e].float().T
    if out_dtype is not None:
        Y = Y.to(out_dtype)
    if two_d:
        Y = Y.view(expert_indices.shape[0], k, I)
    return Y


# --------------------------------------------------------------------------- FusedMoE
def expert_ffn(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """(SiLU(x Wg^T) * (x Wu^T)) Wd^T, kernels/fusedmoe_baseline.py:93-103."""
    return (F.silu(x @ gate.T) * (x @ up.T)) @ down.T


def router_logits(x_flat: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """fp32-accumulated logits from (bf16-rounded) x and Wr, kernels/fusedmoe_baseline.py:72."""
    return x_flat.float() @ router_weight.float().T


def routed_experts(x_flat: torch.Tensor, topk_indices: torch.Tensor, topk_scores: torch.Tensor,
                   routed_gate: torch.Tensor, routed_up: torch.Tensor, routed_down: torch.Tensor,
                   compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Routed-expert loop with scatter-sum combine, kernels/fusedmoe_baseline.py:105-168.

    Visits experts in ascending id, skips empty ones, scales each expert output
    by the routing score and sums it into a [T,H] cache of ``compute_dtype``.
    """
    T, H = x_flat.shape
    E = routed_gate.shape[0]
    k = topk_indices.shape[1]
    x = x_flat.to(compute_dtype)
    flat_scores = topk_scores.reshape(-1, 1).to(compute_dtype)
    _, offsets, perm, _ = route_histogram(topk_indices, E)
    perm = perm.long()
    token_of = perm // k
    cache = torch.zeros(T, H, dtype=compute_dtype)
    for e in range(E):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if s == t:
            continue
        tok = token_of[s:t]
        out = expert_ffn(x[tok], routed_gate[e].to(compute_dtype), routed_up[e].to(compute_dtype),
                         routed_down[e].to(compute_dtype))
        out = out * flat_scores[perm[s:t]]
        cache.index_add_(0, tok, out)
    return cache


def fusedmoe(x: torch.Tensor, router_weight: torch.Tensor,
             shared_gate: Optional[torch.Tensor], shared_up: Optional[torch.Tensor],
             shared_down: Optional[torch.Tensor],
             routed_gate: torch.Tensor, routed_up: torch.Tensor, routed_down: torch.Tensor,
             n_experts_per_token: int, compute_dtype: torch.dtype = torch.float32,
             logits: Optional[torch.Tensor] = None, return_routing: bool = False):
    """Shared + routed MoE forward, kernels/fusedmoe_baseline.py:46-91,171-203.

    Router: fp32 logits (given, or x Wr^T on fp32 copies), softmax over all
    experts, top-k without renormalisation (mode A).  ``compute_dtype`` float32
    gives the fp32-accumulated oracle; bfloat16 reproduces the baseline's own
    rounding between ops.
    """
    shape = x.shape
    H = shape[-1]
    x_flat = x.reshape(-1, H)
    if logits is None:
        logits = router_logits(x_flat, router_weight)
    scores, idx = topk_softmax(logits, n_experts_per_token, MODE_A)
    xc = x_flat.to(compute_dtype)
    routed = routed_experts(x_flat, idx, scores, routed_gate, routed_up, routed_down, compute_dtype)
    if shared_gate is not None and shared_gate.numel() > 0:
        shared = expert_ffn(xc, shared_gate.to(compute_dtype), shared_up.to(compute_dtype),
                            shared_down.to(compute_dtype))
        out = shared + routed
    else:
        out = routed
    out = out.view(*shape)
    if return_routing:
        return out, scores, idx
    return out


# --------------------------------------------------------------------------- seeded inputs
def make_fusedmoe_inputs(batch_size: int, seq_len: int, d_hidden: int, d_expert: int,
                         n_routed_experts: int, n_shared_experts: int, n_experts_per_token: int,
                         dtype: torch.dtype = torch.bfloat16, seed: int = 42
                         ) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Seeded CPU inputs with the tensor names, shapes, draw order and 1/sqrt(fan_in)
    scaling of kernels/fusedmoe_baseline.py:311-375 (always on the CPU generator)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)

    def rn(*shape):
        return torch.randn(*shape, dtype=dtype, generator=g)

    x = rn(batch_size, seq_len, d_hidden).contiguous()
    sd = d_expert * n_shared_experts
    w = {}
    w["router_weight"] = rn(n_routed_experts, d_hidden) / math.sqrt(d_hidden)
    w["shared_gate"] = rn(sd, d_hidden) / math.sqrt(d_hidden)
    w["shared_up"] = rn(sd, d_hidden) / math.sqrt(d_hidden)
    w["shared_down"] = rn(d_hidden, sd) / math.sqrt(max(sd, 1))
    w["routed_gate"] = rn(n_routed_experts, d_expert, d_hidden) / math.sqrt(d_hidden)
    w["routed_up"] = rn(n_routed_experts, d_expert, d_hidden) / math.sqrt(d_hidden)
    w["routed_down"] = rn(n_routed_experts, d_hidden, d_expert) / math.sqrt(d_expert)
    return x, w


def zipf_logits(T: int, E: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """Router logits with Zipf(s) expert popularity: log p[pi(e)] + Gumbel(0,1) noise,
    p_r ~ r^-s, pi a seeded permutation of expert ids.  fp32 [T,E]."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    ranks = torch.arange(1, E + 1, dtype=torch.float64)
    p = ranks.pow(-s)
    p = p / p.sum()
    pi = torch.randperm(E, generator=g)
    logp = torch.empty(E, dtype=torch.float64)
    logp[pi] = p.log()
    u = torch.rand(T, E, generator=g, dtype=torch.float64).clamp_(1e-12, 1 - 1e-12)
    gumbel = -(-(u.log())).log()
    return (logp[None, :] + gumbel).to(torch.float32)


# ----------------------------------------------------------------------------- mHC pre / post blocks
def sinkhorn(x: torch.Tensor, repeat: int, eps: float) -> torch.Tensor:
    """Row softmax + eps, a column normalisation, then (repeat-1) x [row normalisation, column normalisation],
    every divisor with + eps (reference kernels/mhc_baseline.py:18-43).  x fp32 [..., hc, hc]."""
    x = torch.softmax(x, dim=-1) + eps
    x = x / (x.sum(dim=-2, keepdim=True) + eps)
    for _ in range(repeat - 1):
        x = x / (x.sum(dim=-1, keepdim=True) + eps)
        x = x / (x.sum(dim=-2, keepdim=True) + eps)
    return x


def mhc_pre(residual: torch.Tensor, fn: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor,
            rms_eps: float = 1e-6, hc_pre_eps: float = 1e-6, hc_sinkhorn_eps: float = 1e-6,
            hc_post_mult_value: float = 1.0, sinkhorn_repeat: int = 10, accumulate=torch.float32):
    """mHC pre block (reference kernels/mhc_baseline.py:48-128).  residual bf16 [T, hc, hidden], fn fp32
    [2hc+hc*hc, hc*hidden], hc_scale fp32 [3], hc_base fp32 [2hc+hc*hc] ->
    post_mix fp32 [T,hc,1], comb_mix fp32 [T,hc,hc], layer_input bf16 [T,hidden].
    ``accumulate=torch.float64`` evaluates the dot products and the sum of squares in double precision (the
    yardstick the GPU tests use; the default follows the reference's fp32 evaluation)."""
    T, hc, hidden = residual.shape
    flat = residual.reshape(T, hc * hidden).to(accumulate)
    sqrsum = flat.square().sum(-1)
    rms = (sqrsum / fn.shape[-1] + rms_eps).rsqrt()
    mixes = ((flat @ fn.to(accumulate).T) * rms.unsqueeze(-1)).float()
    scale = torch.cat([hc_scale[0].expand(hc), hc_scale[1].expand(hc), hc_scale[2].expand(hc * hc)])
    mixes = mixes * scale + hc_base
    pre = mixes[:, :hc].sigmoid().unsqueeze(-1) + hc_pre_eps
    post = (mixes[:, hc:2 * hc].sigmoid() * hc_post_mult_value).unsqueeze(-1)
    comb = sinkhorn(mixes[:, 2 * hc:].reshape(T, hc, hc), sinkhorn_repeat, hc_sinkhorn_eps)
    layer_input = (residual * pre).sum(-2).bfloat16()
    return post, comb, layer_input


def mhc_post(x: torch.Tensor, residual: torch.Tensor, post_layer_mix: torch.Tensor, comb_res_mix: torch.Tensor):
    """mHC post block (reference kernels/mhc_baseline.py:136-163): x bf16 [T,hidden], residual bf16 [T,hc,hidden],
    post_layer_mix fp32 [T,hc,1], comb_res_mix fp32 [T,hc,hc] -> bf16 [T,hc,hidden] =
    x * post_layer_mix + comb_res_mix^T @ residual, evaluated in fp32."""
    term1 = x.float().unsqueeze(-2) * post_layer_mix
    term2 = torch.bmm(comb_res_mix.transpose(1, 2), residual.float())
    return (term1 + term2).bfloat16()


def make_mhc_inputs(num_tokens: int, hidden: int, hc: int = 4, seed: int = 42):
    """Seeded mHC inputs with the value distributions of the reference benchmark
    (benchmarks/benchmark_mhc.py:79-108): residual ~ N(0,1)*(1+0.01*m) in bf16, fn ~ 1e-4*N(0,1)*(1+0.01*m) in fp32,
    hc_scale, hc_base ~ 0.1*N(0,1); post-block inputs ~ N(0,1).  Drawn on the CPU."""
    g = torch.Generator().manual_seed(seed)
    r3 = 2 * hc + hc * hc
    ramp = (1 + torch.arange(hc).mul(0.01)).view(1, -1, 1)
    residual = (torch.randn(num_tokens, hc, hidden, generator=g) * ramp).bfloat16()
    fn = (torch.randn(r3, hc, hidden, generator=g) * 1e-4 * ramp).flatten(1, 2).contiguous()
    hc_scale = torch.randn(3, generator=g) * 0.1
    hc_base = torch.randn(r3, generator=g) * 0.1
    x = torch.randn(num_tokens, hidden, generator=g).bfloat16()
    post_layer_mix = torch.randn(num_tokens, hc, 1, generator=g)
    comb_res_mix = torch.randn(num_tokens, hc, hc, generator=g)
    return dict(residual=residual, fn=fn, hc_scale=hc_scale, hc_base=hc_base, x=x, post_layer_mix=post_layer_mix,
                comb_res_mix=comb_res_mix)
