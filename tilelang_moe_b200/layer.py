"""The MoE layer forward as a fixed sequence of launches on one stream.

    logits -> top-k + softmax -> histogram / offsets / permutation
           -> up GEMM (row gather fused into its operand pipeline, SiLU gate fused into its epilogue)
           -> down GEMM (routing-weight scale + scatter fused) -> combine (k-way sum + shared expert)

(for a hidden size that is not a multiple of 64 the rows are gathered by a separate kernel first).

No step reads anything back to the host: tile tables are derived on the device
from the expert offsets, and scratch is sized from T, k, H, I alone, so one
``MoEWorkspace`` serves every routing pattern of a given shape.

Mirrors ``FusedMoEPyTorch.forward`` (reference kernels/fusedmoe_baseline.py:46-91)
and ``FusedMoETileLang.forward`` (reference kernels/fusedmoe_tilelang.py:309-417).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, ops


@dataclass
class MoEWorkspace:
    """Persistent scratch for one (T, k, H, I, E) shape on one device."""
    T: int
    k: int
    H: int
    I: int
    E: int
    SI: int
    device: torch.device
    dtype: torch.dtype = torch.bfloat16

    def __post_init__(self):
        dev, bf16 = self.device, self.dtype
        n = self.T * self.k
        self.logits = torch.empty(self.T, self.E, dtype=torch.float32, device=dev)
        # the up GEMM fetches the activation rows itself (MOE_B200_FUSED_GATHER=0: separate gather pass, for measurement)
        self.fused_gather = self.H % 64 == 0 and os.environ.get("MOE_B200_FUSED_GATHER", "1") != "0"
        if not self.fused_gather:
            self.xs = torch.empty(n, self.H, dtype=bf16, device=dev)      # expert-sorted activations
            self.ws = torch.empty(n, dtype=torch.float32, device=dev)     # routing weight per sorted row
        self.act = torch.empty(n, self.I, dtype=bf16, device=dev)         # SiLU(gate)*up per sorted row
        self.yk = torch.empty(n, self.H, dtype=bf16, device=dev)          # scaled expert output per (token, slot)
        need = _lib.load().moe_route_histogram_workspace(n, self.E)
        self.hist_ws = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
        if self.SI > 0:
            self.act_s = torch.empty(self.T, self.SI, dtype=bf16, device=dev)
            self.y_s = torch.empty(self.T, self.H, dtype=bf16, device=dev)
            self.offs_s = torch.tensor([0, self.T], dtype=torch.int32, device=dev)
        self.out = torch.empty(self.T, self.H, dtype=bf16, device=dev)


_side_streams = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _side_streams.get(key)
    if st is None:
        st = torch.cuda.Stream(device=device)
        _side_streams[key] = st
    return st


class _Stage:
    """Records a CUDA event pair around a stage when a timers dict is given (else does nothing)."""

    def __init__(self, timers, name):
        self.timers, self.name = timers, name

    def __enter__(self):
        if self.timers is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.a.record()

    def __exit__(self, *exc):
        if self.timers is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            self.timers[self.name] = (self.a, b)


def routed_forward(x_flat: torch.Tensor, scores: torch.Tensor, idx32: torch.Tensor, routed_gate: torch.Tensor,
                   routed_up: torch.Tensor, routed_down: torch.Tensor, ws: MoEWorkspace,
                   shared_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   timers: Optional[dict] = None, shared_ready: Optional[torch.cuda.Event] = None) -> torch.Tensor:
    """Routed experts + combine for routing already decided (scores fp32 [T,k], idx32 int32 [T,k]).
    ``timers``: optional dict that receives a CUDA event pair per stage."""
    E = routed_gate.shape[0]
    k = idx32.shape[1]
    with _Stage(timers, "histogram"):
        counts, offsets, perm, _ = ops.route_histogram(idx32, E, want_inv=False, workspace=ws.hist_ws)
    if ws.fused_gather:
        with _Stage(timers, "up_gemm"):
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x_flat, routed_gate, offsets, B2=routed_up, out=ws.act,
                                    gather=perm, gather_div=k)
        with _Stage(timers, "down_gemm"):   # the weight of sorted row r is scores.flat[perm[r]]: read at the destination
            ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER_DSTW, ws.act, routed_down, offsets, dst_rows=perm,
                                    row_w=scores.reshape(-1), out=ws.yk)
    else:
        with _Stage(timers, "gather"):
            ops.gather_rows(x_flat, perm, div=k, out=ws.xs, w_src=scores, w_out=ws.ws)
        with _Stage(timers, "up_gemm"):
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, ws.xs, routed_gate, offsets, B2=routed_up, out=ws.act)
        with _Stage(timers, "down_gemm"):
            ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, ws.act, routed_down, offsets, dst_rows=perm,
                                    row_w=ws.ws, out=ws.yk)
    if shared_ready is not None:      # the shared expert ran on another stream: join before it is read
        torch.cuda.current_stream(x_flat.device).wait_event(shared_ready)
    with _Stage(timers, "combine"):
        y = ops.combine(ws.yk, k, shared=shared_out, out=ws.out if out is None else out)
    return y


def shared_forward(x_flat: torch.Tensor, shared_gate: torch.Tensor, shared_up: torch.Tensor,
                   shared_down: torch.Tensor, ws: MoEWorkspace) -> torch.Tensor:
    """The shared experts as one dense SiLU-gated FFN of width S*I (reference fusedmoe_baseline.py:93-103)."""
    ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x_flat, shared_gate.unsqueeze(0), ws.offs_s,
                            B2=shared_up.unsqueeze(0), out=ws.act_s)
    return ops.grouped_gemm_sorted(ops.GEMM_PLAIN, ws.act_s, shared_down.unsqueeze(0), ws.offs_s, out=ws.y_s)


def moe_forward(x: torch.Tensor, router_weight: Optional[torch.Tensor], shared_gate, shared_up, shared_down,
                routed_gate: torch.Tensor, routed_up: torch.Tensor, routed_down: torch.Tensor, k: int,
                ws: Optional[MoEWorkspace] = None, logits: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, return_routing: bool = False):
    """Full layer.  x [..., H] bf16.  Router: fp32 logits (given, or x.Wr^T), softmax over all
    experts, top-k without renormalisation (reference fusedmoe_baseline.py:72-76)."""
    if x.dtype not in ops.DTYPE_CODE:
        raise ValueError("moe_b200 computes in bfloat16 or float16; cast the activations and weights")
    shape = x.shape
    H = shape[-1]
    x_flat = x.reshape(-1, H)
    if not x_flat.is_contiguous():
        x_flat = x_flat.contiguous()
    T = x_flat.shape[0]
    E, I, _ = routed_gate.shape
    SI = 0 if shared_gate is None else shared_gate.shape[0]
    if (ws is None or (ws.T, ws.k, ws.H, ws.I, ws.E, ws.SI, ws.dtype) != (T, k, H, I, E, SI, x.dtype)
            or ws.device != x.device):
        ws = MoEWorkspace(T, k, H, I, E, SI, x.device, x.dtype)
    shared_out, shared_ready = None, None
    if SI > 0:
        # The shared expert depends on x only: it runs on a second stream beside router -> permutation -> routed
        # GEMMs and is joined before the combine (reference kernels/fusedmoe_tilelang.py:428-553 does the same with
        # its two kernels).  Under graph capture the fork / join become parallel branches of the graph.
        cur = torch.cuda.current_stream(x.device)
        side = _side_stream(x.device)
        fork = torch.cuda.Event()
        fork.record(cur)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            shared_out = shared_forward(x_flat, shared_gate, shared_up, shared_down, ws)
            shared_ready = torch.cuda.Event()
            shared_ready.record(side)
    if logits is None:     # router GEMM + top-k + softmax: one kernel when the shape allows, logits never stored
        scores, idx32 = ops.router_topk_softmax(x_flat, router_weight, k, mode="A", index_dtype=torch.int32)
    else:
        scores, idx32 = ops.topk_softmax(logits, k, mode="A", index_dtype=torch.int32)
    y = routed_forward(x_flat, scores, idx32, routed_gate, routed_up, routed_down, ws, shared_out=shared_out,
                       out=None if out is None else out.view(T, H), shared_ready=shared_ready)
    y = y.view(*shape)
    if return_routing:
        return y, scores, idx32
    return y


class SingleCallWorkspace:
    """Device scratch of ``moe_layer_forward`` for one (T, k, H, I, E, SI) shape: one buffer, laid out by the library."""

    def __init__(self, T: int, k: int, H: int, I: int, E: int, SI: int, device: torch.device,
                 dtype: torch.dtype = torch.bfloat16):
        self.key = (T, k, H, I, E, SI, dtype, device)
        need = _lib.load().moe_layer_workspace(T, k, H, I, E, SI)
        self.buf = torch.empty(need + 256, dtype=torch.uint8, device=device)
        self.offset = (-self.buf.data_ptr()) % 256
        self.bytes = need
        self.out = torch.empty(T, H, dtype=dtype, device=device)


def moe_forward_single_call(x: torch.Tensor, router_weight: Optional[torch.Tensor], shared_gate, shared_up, shared_down,
                            routed_gate: torch.Tensor, routed_up: torch.Tensor, routed_down: torch.Tensor, k: int,
                            ws: Optional[SingleCallWorkspace] = None, logits: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The layer through ``moe_layer_forward``: one library call enqueues every kernel (the shared expert on the
    side stream), instead of one Python-level call per stage.  Same kernels, same results as ``moe_forward``."""
    if x.dtype not in ops.DTYPE_CODE:
        raise ValueError("moe_b200 computes in bfloat16 or float16; cast the activations and weights")
    shape = x.shape
    H = shape[-1]
    x_flat = x.reshape(-1, H)
    if not x_flat.is_contiguous():
        x_flat = x_flat.contiguous()
    T = x_flat.shape[0]
    E, I, _ = routed_gate.shape
    SI = 0 if shared_gate is None else shared_gate.shape[0]
    tensors = [x_flat, router_weight, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down]
    for t in tensors:
        if t is not None and (not t.is_cuda or t.dtype != x.dtype or not t.is_contiguous()):
            raise ValueError("all layer tensors must be contiguous CUDA tensors of the activation dtype")
    if logits is not None and (logits.dtype != torch.float32 or tuple(logits.shape) != (T, E) or not logits.is_contiguous()):
        raise ValueError("logits must be a contiguous float32 [T, E] tensor")
    if logits is None and router_weight is None:
        raise ValueError("either router_weight or logits is needed")
    dev = x.device
    key = (T, k, H, I, E, SI, x.dtype, dev)
    if ws is None or ws.key != key:
        ws = SingleCallWorkspace(T, k, H, I, E, SI, dev, x.dtype)
    y = ws.out if out is None else out.view(T, H)
    side = _side_stream(dev) if SI > 0 else None
    p = ops._ptr
    with torch.cuda.device(dev):
        rc = _lib.load().moe_layer_forward(
            p(x_flat), p(router_weight) if logits is None else None, p(logits), p(shared_gate), p(shared_up), p(shared_down),
            p(routed_gate), p(routed_up), p(routed_down), T, H, I, E, k, SI, ops.DTYPE_CODE[x.dtype],
            ws.buf.data_ptr() + ws.offset, ws.bytes, p(y), p(ops.status_buffer(dev)), ops._stream(),
            side.cuda_stream if side is not None else None)
    _lib.check(rc, "moe_layer_forward")
    ops._after(dev)
    return y.view(*shape)
