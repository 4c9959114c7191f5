"""Drop-in for the hot path of the reference's ``kernels`` package.

Same names, argument order and return types as the reference's public API
(reference kernels/__init__.py:4-101) for the MoE-layer path:

    topk_softmax(logits, k)                       kernels/topk_softmax_tilelang.py:1103-1135
    grouped_gemm(X, W, expert_indices)            kernels/grouped_gemm_tilelang.py:859-895
    fusedmoe_tilelang(x, router_weight, ...)      kernels/fusedmoe_tilelang.py:605-647
    FusedMoETileLang(...).forward(...)            kernels/fusedmoe_tilelang.py:241-417
    generate_fusedmoe_inputs(...)                 kernels/fusedmoe_baseline.py:311-375
    mhc_pre(residual, fn, hc_scale, hc_base, ...) kernels/mhc_tilelang.py:494-545
    mhc_post(x, residual, post_mix, comb_mix)     kernels/mhc_tilelang.py:575-582

Everything runs on the CUDA library behind ``include/moe_b200.h``; there is no
strategy auto-selection between back ends and no CPU path.  Deliberate
differences from the reference's GPU path, all towards its PyTorch baseline:
indices are int64 and sorted (value descending, ties lowest index first), the
router of the fused layer accumulates logits in fp32, and both float16 (the
reference's default) and bfloat16 are computed natively with fp32 accumulation.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from .. import layer as _layer
from .. import ops as _ops

__all__ = [
    "topk_softmax", "topk_softmax_best", "grouped_gemm", "grouped_gemm_best", "fusedmoe_tilelang", "fusedmoe",
    "FusedMoETileLang", "FusedMoE", "generate_fusedmoe_inputs", "route_histogram", "mhc_pre", "mhc_post",
    # the reference's other public names (its strategy variants and its PyTorch baselines): the same operator each
    "topk_softmax_fused", "topk_softmax_selection", "topk_softmax_sonic", "topk_softmax_bitonic",
    "topk_softmax_separate", "topk_softmax_separate_compiled", "topk_softmax_tilelang_separate", "topk_radix_tilelang",
    "grouped_gemm_loop", "grouped_gemm_loop_compiled", "grouped_gemm_padded", "grouped_gemm_tilelang",
    "grouped_gemm_pytorch", "fusedmoe_pytorch", "fusedmoe_pytorch_compiled", "fusedmoe_tilelang_streams", "fusedmoe_best",
    "FusedMoETileLangStreams", "topk_softmax_conv_a_renorm", "topk_softmax_conv_b_unfused",
    "topk_softmax_conv_b_radix_unfused", "topk_softmax_bitonic_v2", "topk_softmax_bitonic_v3", "grouped_gemm_tilelang_v2",
    "grouped_gemm_tilelang_v3",
    "mhc_pre_pytorch", "mhc_pre_pytorch_compiled", "mhc_pre_tilelang_official", "mhc_pre_tilelang_optimized",
    "mhc_pre_tilelang_splitk", "mhc_post_pytorch", "mhc_post_pytorch_compiled", "mhc_post_tilelang_official",
]


def topk_softmax(logits: torch.Tensor, k: int, mode: str = "B") -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k of the logits, softmax over the k selected (convention B).

    logits (num_tokens, num_experts) float32 -> (scores float32 (num_tokens, k),
    indices int64 (num_tokens, k)).  ``mode`` "A" / "A_renorm" give the other two
    conventions of the reference baseline (softmax over all experts first).
    """
    return _ops.topk_softmax(logits, k, mode=mode, index_dtype=torch.int64)


topk_softmax_best = topk_softmax


def route_histogram(topk_indices: torch.Tensor, n_experts: int):
    """counts, exclusive offsets, stable permutation and inverse of the flattened expert ids."""
    return _ops.route_histogram(topk_indices, n_experts)


def grouped_gemm(X: torch.Tensor, W: torch.Tensor, expert_indices: torch.Tensor,
                 w_layout: str = "EIH") -> torch.Tensor:
    """Y[i] = X[i] @ W[expert_indices[i]].T.

    X (total_tokens, H) bfloat16 or float16; W (E, I, H); expert_indices (total_tokens,) int64
    -> Y (total_tokens, I).  With 2-D expert_indices (T, k) every token row is used
    by its k experts and Y is (T, k, I), without materialising a repeated X on the
    host side.  ``w_layout="EHI"`` accepts the kernel-level layout the reference's
    benchmark allocates (it is transposed once here).
    """
    if w_layout == "EHI":
        W = W.transpose(1, 2).contiguous()
    elif w_layout != "EIH":
        raise ValueError("w_layout must be 'EIH' or 'EHI'")
    if X.dtype not in _ops.DTYPE_CODE or W.dtype != X.dtype:
        raise ValueError("grouped_gemm computes in bfloat16 or float16 (X and W of the same type)")
    if expert_indices.dim() not in (1, 2) or expert_indices.shape[0] != X.shape[0]:
        raise ValueError("expert_indices must be (total_tokens,) or (total_tokens, k)")
    E, I, H = W.shape
    k = expert_indices.shape[1] if expert_indices.dim() == 2 else 1
    n = X.shape[0] * k
    _, offsets, perm, _ = _ops.route_histogram(expert_indices, E, want_inv=False)
    Y = torch.empty(n, I, dtype=X.dtype, device=X.device)
    if H % 64 == 0:     # the GEMM fetches the rows of X through the permutation itself
        _ops.grouped_gemm_sorted(_ops.GEMM_PLAIN, X.contiguous(), W.contiguous(), offsets, dst_rows=perm, out=Y,
                                 gather=perm, gather_div=k)
    else:
        xs = _ops.gather_rows(X.contiguous(), perm, div=k)
        _ops.grouped_gemm_sorted(_ops.GEMM_PLAIN, xs, W.contiguous(), offsets, dst_rows=perm, out=Y)
    return Y.view(X.shape[0], k, I) if expert_indices.dim() == 2 else Y


grouped_gemm_best = grouped_gemm


class FusedMoETileLang:
    """Shared + routed SiLU-gated MoE layer with persistent scratch for one shape.

    Constructor arguments as in the reference (kernels/fusedmoe_tilelang.py:248-260);
    ``block_token`` is accepted and ignored (the tile shape is fixed by the kernel).
    """

    def __init__(self, d_hidden: int, d_expert: int, n_routed_experts: int, n_shared_experts: int,
                 n_experts_per_token: int, batch_size: int, seq_len: int, dtype: torch.dtype = torch.float16,
                 block_token: int = 128, device: Optional[torch.device] = None):
        if dtype not in _ops.DTYPE_CODE:
            raise ValueError("moe_b200 computes in bfloat16 or float16")
        self.d_hidden, self.d_expert = d_hidden, d_expert
        self.n_routed_experts, self.n_shared_experts = n_routed_experts, n_shared_experts
        self.n_experts_per_token = n_experts_per_token
        self.batch_size, self.seq_len = batch_size, seq_len
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.ws = _layer.SingleCallWorkspace(batch_size * seq_len, n_experts_per_token, d_hidden, d_expert,
                                             n_routed_experts, d_expert * n_shared_experts, dev, dtype)

    # A single shared expert of the routed experts' width can run as expert E of the routed grouped GEMMs (five
    # launches for the whole layer, no second stream): the library does so when the shared weights lie directly behind
    # the routed ones in memory.  The layer object keeps such stacked copies of the weights it is called with, as the
    # reference's layer keeps its stacked expert tensors (kernels/fusedmoe_tilelang.py:296-307), as long as they stay
    # below this size; larger layers keep the side-stream form and their weights where they are.
    STACK_LIMIT_BYTES = 2 << 30

    def _stacked(self, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down):
        ws = (shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down)
        E, I, H = routed_gate.shape
        if (self.n_shared_experts != 1 or H % 64 or any(w is None for w in ws)
                or 3 * (E + 1) * I * H * routed_gate.element_size() > self.STACK_LIMIT_BYTES):
            return None
        key = tuple((w.data_ptr(), w._version) for w in ws)
        if getattr(self, "_stack_key", None) != key:
            def stack(routed, shared, shape):
                out = torch.empty(E + 1, *shape, dtype=routed.dtype, device=routed.device)
                out[:E].copy_(routed)
                out[E].copy_(shared.reshape(shape))
                return out
            self._stack = (stack(routed_gate, shared_gate, (I, H)), stack(routed_up, shared_up, (I, H)),
                           stack(routed_down, shared_down, (H, I)))
            self._stack_key = key
        return self._stack

    def forward(self, x, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down,
                logits: Optional[torch.Tensor] = None):
        """One library call (``moe_layer_forward``) enqueues the whole layer."""
        st = self._stacked(shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down) \
            if self.n_shared_experts else None
        if st is not None:
            E = routed_gate.shape[0]
            g, u, d = st
            return _layer.moe_forward_single_call(x, router_weight, g[E], u[E], d[E], g[:E], u[:E], d[:E],
                                                  self.n_experts_per_token, ws=self.ws, logits=logits)
        return _layer.moe_forward_single_call(x, router_weight, shared_gate if self.n_shared_experts else None,
                                              shared_up, shared_down, routed_gate, routed_up, routed_down,
                                              self.n_experts_per_token, ws=self.ws, logits=logits)

    __call__ = forward

    def capture(self, x, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down,
                logits: Optional[torch.Tensor] = None, warmup: int = 2):
        """Record the whole forward (about a dozen launches, no host synchronisation anywhere) into a CUDA graph.

        The tensors passed here become the graph's static inputs: write new activations into ``x`` (and
        ``logits``) in place, call the returned function, read the returned output tensor.  Small layers are
        bound by launch latency rather than by the kernels; replaying one graph removes it (the reference gets
        a similar effect from its two-stream variant, kernels/fusedmoe_tilelang.py:428-553)."""
        args = (x, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down)
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):      # first calls set kernel attributes and build cached tables
                self.forward(*args, logits=logits)
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.forward(*args, logits=logits)

        def replay():
            graph.replay()
            return out

        replay.graph, replay.output = graph, out
        return replay


FusedMoE = FusedMoETileLang
_layer_cache: Dict[tuple, FusedMoETileLang] = {}


def fusedmoe_tilelang(x, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down,
                      n_experts_per_token: int) -> torch.Tensor:
    """Functional form; caches one layer object per shape like the reference
    (kernels/fusedmoe_tilelang.py:628-640).  Output: shape of x."""
    B, S, H = x.shape
    E, I, _ = routed_gate.shape
    n_shared = shared_gate.shape[0] // I if shared_gate is not None else 0
    key = (H, I, E, n_shared, n_experts_per_token, B, S, x.dtype, x.device)
    m = _layer_cache.get(key)
    if m is None:
        m = FusedMoETileLang(H, I, E, n_shared, n_experts_per_token, B, S, x.dtype, device=x.device)
        _layer_cache[key] = m
    return m.forward(x, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down)


fusedmoe = fusedmoe_tilelang


def generate_fusedmoe_inputs(batch_size: int, seq_len: int, d_hidden: int, d_expert: int, n_routed_experts: int,
                             n_shared_experts: int, n_experts_per_token: int, dtype: torch.dtype = torch.float16,
                             device: str = "cuda", seed: int = 42):
    """Seeded layer inputs: x ~ N(0,1) and weights ~ N(0, 1/fan_in), drawn in the order x,
    router, shared gate/up/down, routed gate/up/down from one generator on ``device``
    (same contract as reference kernels/fusedmoe_baseline.py:311-375)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)

    def draw(*shape):
        return torch.randn(*shape, device=device, dtype=dtype, generator=gen)

    x = draw(batch_size, seq_len, d_hidden).contiguous()
    sd = d_expert * n_shared_experts
    weights = {
        "router_weight": draw(n_routed_experts, d_hidden) / math.sqrt(d_hidden),
        "shared_gate": draw(sd, d_hidden) / math.sqrt(d_hidden),
        "shared_up": draw(sd, d_hidden) / math.sqrt(d_hidden),
        "shared_down": draw(d_hidden, sd) / math.sqrt(max(sd, 1)),
        "routed_gate": draw(n_routed_experts, d_expert, d_hidden) / math.sqrt(d_hidden),
        "routed_up": draw(n_routed_experts, d_expert, d_hidden) / math.sqrt(d_hidden),
        "routed_down": draw(n_routed_experts, d_hidden, d_expert) / math.sqrt(d_expert),
    }
    return x, weights


_mhc_split_cache: Dict[tuple, torch.Tensor] = {}


def mhc_pre(residual: torch.Tensor, fn: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor,
            rms_eps: float = 1e-6, hc_pre_eps: float = 1e-6, hc_sinkhorn_eps: float = 1e-6,
            hc_post_mult_value: float = 1.0, sinkhorn_repeat: int = 10):
    """mHC pre block, arguments and results as the reference's ``mhc_pre`` (kernels/mhc_tilelang.py:494-545):
    residual bf16 (num_tokens, hc_mult, hidden), fn fp32 (2*hc+hc*hc, hc*hidden), hc_scale fp32 (3,), hc_base fp32
    (2*hc+hc*hc,) -> (post_mix fp32 (T,hc,1), comb_mix fp32 (T,hc,hc), layer_input bf16 (T,hidden)).
    The bf16 split of ``fn`` is built on first use and cached per weight tensor (and its version counter)."""
    key = (fn.data_ptr(), fn._version, tuple(fn.shape), fn.device)
    fn3 = _mhc_split_cache.get(key)
    if fn3 is None:
        if len(_mhc_split_cache) > 64:
            _mhc_split_cache.clear()
        fn3 = _ops.mhc_split_weights(fn)
        _mhc_split_cache[key] = fn3
    return _ops.mhc_pre(residual, fn3, hc_scale, hc_base, rms_eps, hc_pre_eps, hc_sinkhorn_eps, hc_post_mult_value,
                        sinkhorn_repeat)


def mhc_post(x: torch.Tensor, residual: torch.Tensor, post_layer_mix: torch.Tensor,
             comb_res_mix: torch.Tensor) -> torch.Tensor:
    """mHC post block (reference kernels/mhc_tilelang.py:575-582): bf16 (T, hc_mult, hidden)."""
    return _ops.mhc_post(x, residual, post_layer_mix, comb_res_mix)


# ---------------------------------------------------------------------------------------------------------------
# The reference exports every strategy variant and every PyTorch baseline of an operator under its own name
# (reference kernels/__init__.py:4-101).  Here each operator has one implementation, so the other names are the same
# function with the variant's convention: code written against any of them keeps working.
# ---------------------------------------------------------------------------------------------------------------
def topk_softmax_fused(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k first, softmax over the k selected (reference kernels/topk_softmax_baseline.py:39-68)."""
    return topk_softmax(logits, k, mode="B")


topk_softmax_selection = topk_softmax_fused     # reference kernels/topk_softmax_tilelang.py:983-1001
topk_softmax_sonic = topk_softmax_fused         # its alias, :1005
topk_softmax_bitonic = topk_softmax_fused       # :895-921


def topk_softmax_separate(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax over all experts, then top-k (reference kernels/topk_softmax_baseline.py:15-36)."""
    return topk_softmax(logits, k, mode="A")


def topk_softmax_conv_a_renorm(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax over all experts, top-k, then renormalised to sum 1 (reference kernels/topk_softmax_baseline.py:223-236)."""
    return topk_softmax(logits, k, mode="A_renorm")


topk_softmax_conv_b_unfused = topk_softmax_fused            # reference kernels/topk_softmax_baseline.py:241
topk_softmax_conv_b_radix_unfused = topk_softmax_fused      # reference kernels/topk_softmax_tilelang.py:1139-1159
topk_softmax_bitonic_v2 = topk_softmax_fused                # :924-951
topk_softmax_bitonic_v3 = topk_softmax_fused                # :954-980
topk_softmax_separate_compiled = topk_softmax_separate
topk_softmax_tilelang_separate = topk_softmax_separate     # reference kernels/topk_softmax_tilelang.py:1013-1040


def topk_radix_tilelang(logits: torch.Tensor, topk: int = 6) -> torch.Tensor:
    """Indices of the top-k logits only (reference kernels/topk_softmax_tilelang.py:205-240); int64 here."""
    return topk_softmax(logits, int(topk), mode="B")[1]


grouped_gemm_loop = grouped_gemm               # reference kernels/grouped_gemm_baseline.py:14-57
grouped_gemm_loop_compiled = grouped_gemm
grouped_gemm_padded = grouped_gemm             # :60-118
grouped_gemm_tilelang = grouped_gemm           # reference kernels/grouped_gemm_tilelang.py:606-680
grouped_gemm_pytorch = grouped_gemm            # :542-603
grouped_gemm_tilelang_v2 = grouped_gemm        # :682-768
grouped_gemm_tilelang_v3 = grouped_gemm        # :771-856
fusedmoe_tilelang_streams = fusedmoe_tilelang  # reference kernels/fusedmoe_tilelang.py:559-602 (its two-stream variant)
fusedmoe_best = fusedmoe_tilelang              # :654-690
FusedMoETileLangStreams = FusedMoETileLang     # :428-556
fusedmoe_pytorch = fusedmoe_tilelang           # reference kernels/fusedmoe_baseline.py:171-203
fusedmoe_pytorch_compiled = fusedmoe_tilelang  # :285-308
mhc_pre_pytorch = mhc_pre                      # reference kernels/mhc_baseline.py:48-127
mhc_pre_pytorch_compiled = mhc_pre
mhc_pre_tilelang_official = mhc_pre            # reference kernels/mhc_tilelang.py:363-403
mhc_pre_tilelang_optimized = mhc_pre           # :406-446
mhc_pre_tilelang_splitk = mhc_pre              # :449-491
mhc_post_pytorch = mhc_post                    # reference kernels/mhc_baseline.py:130-170
mhc_post_pytorch_compiled = mhc_post
mhc_post_tilelang_official = mhc_post          # reference kernels/mhc_tilelang.py:548-572
