"""Torch-tensor front end of the C ABI: argument checks, output allocation, launch.

PyTorch is used here for device memory and streams only.  Every function enqueues
on the current CUDA stream and returns without synchronising.  Kernels report
device-side give-ups (a bounded wait that expired, an expert id out of range)
in a per-device status word; ``check_status()`` reads it (one D2H sync), and it is
read after every call when ``MOE_B200_DEBUG=1``.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _lib

MODE_B, MODE_A, MODE_A_RENORM = 0, 1, 2
GEMM_PLAIN, GEMM_SILU_GATE, GEMM_SCALE_SCATTER, GEMM_PLAIN_F32, GEMM_SCALE_SCATTER_DSTW = 0, 1, 2, 3, 4
_MODES = {"B": MODE_B, "A": MODE_A, "A_norenorm": MODE_A, "A_renorm": MODE_A_RENORM,
          0: MODE_B, 1: MODE_A, 2: MODE_A_RENORM}

DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1}   # MOE_DTYPE_* of include/moe_b200.h


def _dtype_code(*ts: torch.Tensor) -> int:
    dt = ts[0].dtype
    if dt not in DTYPE_CODE:
        raise ValueError("moe_b200 computes in bfloat16 or float16")
    for t in ts[1:]:
        if t is not None and t.dtype != dt:
            raise ValueError(f"mixed element types: {dt} and {t.dtype}")
    return DTYPE_CODE[dt]


_DEBUG = os.environ.get("MOE_B200_DEBUG", "0") not in ("", "0")
_status = {}
_STATUS_TEXT = {1: "expert id outside [0,E)", 2: "a bounded barrier wait expired", 3: "internal selection count mismatch"}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("moe_b200 operates on CUDA tensors only (no CPU path)")


def status_buffer(device: torch.device) -> torch.Tensor:
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = buf
    return buf


def check_status(device=None, reset: bool = True) -> None:
    """Raise if a kernel recorded a device-side failure since the last check."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = status_buffer(dev)
    vals = buf.tolist()
    if vals[0] != 0:
        if reset:
            buf.zero_()
        raise _lib.MoeLibraryError(
            f"device status {vals}: {_STATUS_TEXT.get(vals[0], 'unknown')}")


def _after(dev) -> None:
    if _DEBUG:
        check_status(dev)


# ----------------------------------------------------------------------------- router
def topk_softmax(logits: torch.Tensor, k: int, mode="B", index_dtype: torch.dtype = torch.int64,
                 also_int32: bool = False):
    """Fused top-k + softmax.  Returns (scores fp32 [M,k], indices [M,k]) sorted by value
    descending, ties lowest index first.  With ``also_int32`` a third tensor carries the
    same indices as int32 (feeds route_histogram without a cast)."""
    _need_cuda(logits)
    if logits.dim() != 2 or logits.dtype != torch.float32:
        raise ValueError("logits must be a 2-D float32 tensor")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    M, N = logits.shape
    if not (1 <= k <= N):
        raise ValueError(f"k={k} must be in [1, N={N}]")
    if index_dtype not in (torch.int64, torch.int32):
        raise ValueError("index_dtype must be int64 or int32")
    lib = _lib.load()
    scores = torch.empty(M, k, dtype=torch.float32, device=logits.device)
    idx64 = torch.empty(M, k, dtype=torch.int64, device=logits.device) if index_dtype == torch.int64 else None
    idx32 = torch.empty(M, k, dtype=torch.int32, device=logits.device) if (also_int32 or idx64 is None) else None
    with torch.cuda.device(logits.device):
        rc = lib.moe_topk_softmax(_ptr(logits), M, N, logits.stride(0), k, _MODES[mode], _ptr(scores), _ptr(idx64),
                                  _ptr(idx32), _ptr(status_buffer(logits.device)), _stream())
    _lib.check(rc, "moe_topk_softmax")
    _after(logits.device)
    if idx64 is None:
        return scores, idx32
    if also_int32:
        return scores, idx64, idx32
    return scores, idx64


# ----------------------------------------------------------------------------- permutation
def route_histogram(topk_idx: torch.Tensor, n_experts: int, want_perm: bool = True, want_inv: bool = True,
                    workspace: Optional[torch.Tensor] = None, id_map: Optional[torch.Tensor] = None):
    """counts [E], exclusive offsets [E+1], stable permutation perm [n] and its inverse inv [n]
    (all int32) of the flattened expert ids."""
    _need_cuda(topk_idx)
    if topk_idx.dtype not in (torch.int64, torch.int32):
        raise ValueError("expert ids must be int64 or int32")
    ids = topk_idx.contiguous().view(-1)
    n = ids.numel()
    dev = ids.device
    lib = _lib.load()
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(n, dtype=torch.int32, device=dev) if want_perm else None
    inv = torch.empty(n, dtype=torch.int32, device=dev) if want_inv else None
    need = lib.moe_route_histogram_workspace(n, n_experts)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.moe_route_histogram(_ptr(ids), int(ids.dtype == torch.int64), n, n_experts, _ptr(id_map), _ptr(counts),
                                     _ptr(offsets), _ptr(perm), _ptr(inv), _ptr(workspace),
                                     workspace.numel() * workspace.element_size(), _ptr(status_buffer(dev)), _stream())
    _lib.check(rc, "moe_route_histogram")
    _after(dev)
    return counts, offsets, perm, inv


def gather_rows(src: torch.Tensor, perm: Optional[torch.Tensor], div: int = 1, out: Optional[torch.Tensor] = None,
                w_src: Optional[torch.Tensor] = None, w_out: Optional[torch.Tensor] = None, n_rows: Optional[int] = None):
    """out[p] = src[perm[p] // div]; optionally w_out[p] = w_src[perm[p]]."""
    _need_cuda(src, perm)
    if src.dim() != 2 or src.dtype not in DTYPE_CODE or not src.is_contiguous():
        raise ValueError("src must be a contiguous 2-D bfloat16 / float16 tensor")
    n = (perm.numel() if perm is not None else src.shape[0]) if n_rows is None else n_rows
    cols = src.shape[1]
    if out is None:
        out = torch.empty(n, cols, dtype=src.dtype, device=src.device)
    if w_src is not None:
        if w_src.dtype != torch.float32:
            raise ValueError("routing weights must be float32")
        w_src = w_src.contiguous().view(-1)
        if w_out is None:
            w_out = torch.empty(n, dtype=torch.float32, device=src.device)
    with torch.cuda.device(src.device):
        rc = _lib.load().moe_gather_rows(_ptr(src), _ptr(perm), div, n, cols, _ptr(out), _ptr(w_src), _ptr(w_out), _stream())
    _lib.check(rc, "moe_gather_rows")
    return (out, w_out) if w_src is not None else out


# ----------------------------------------------------------------------------- expert GEMM
def grouped_gemm_sorted(epilogue: int, A: torch.Tensor, B: torch.Tensor, offsets: torch.Tensor,
                        B2: Optional[torch.Tensor] = None, dst_rows: Optional[torch.Tensor] = None,
                        row_w: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                        out_rows: Optional[int] = None, max_rows: Optional[int] = None,
                        expected_rows: int = 0, gather: Optional[torch.Tensor] = None,
                        gather_div: int = 1) -> torch.Tensor:
    """Expert GEMM over expert-sorted rows.  A [rows,K] bf16, B (and B2) [E,N,K] bf16,
    offsets int32 [E+1] on the device.  See include/moe_b200.h for the epilogues.

    With ``gather`` (int32 [rows], the ``perm`` of route_histogram) A is the un-permuted
    matrix and sorted row r is A[gather[r] // gather_div]: the kernel fetches the rows itself
    (K must be a multiple of 64)."""
    _need_cuda(A, B, offsets)
    dt = _dtype_code(A, B, B2)
    if A.dim() != 2 or B.dim() != 3 or not A.is_contiguous() or not B.is_contiguous():
        raise ValueError("A must be contiguous [rows,K], B contiguous [E,N,K]")
    rows, K = A.shape
    E, N, K2 = B.shape
    if K2 != K:
        raise ValueError(f"inner dimensions differ: A has K={K}, B has K={K2}")
    if B2 is not None and (B2.shape != B.shape or B2.dtype != B.dtype or not B2.is_contiguous()):
        raise ValueError("B2 must match B")
    if offsets.dtype != torch.int32 or offsets.numel() != E + 1:
        raise ValueError("offsets must be int32 [E+1]")
    if gather is not None:
        _need_cuda(gather)
        if gather.dtype != torch.int32 or gather.dim() != 1 or not gather.is_contiguous():
            raise ValueError("gather must be a contiguous int32 vector")
        if K % 64:
            raise ValueError("a fused row gather needs K to be a multiple of 64")
        x_rows, rows = rows, gather.numel()
    if max_rows is None:
        max_rows = rows
    if out is None:
        odt = torch.float32 if epilogue == GEMM_PLAIN_F32 else A.dtype
        out = torch.empty(rows if out_rows is None else out_rows, N, dtype=odt, device=A.device)
    with torch.cuda.device(A.device):
        if gather is not None:
            name = "moe_grouped_gemm_gathered"
            rc = _lib.load().moe_grouped_gemm_gathered(
                epilogue, _ptr(A), x_rows, _ptr(gather), gather_div, _ptr(B), _ptr(B2), _ptr(offsets), _ptr(dst_rows),
                _ptr(row_w), _ptr(out), out.stride(0), max_rows, expected_rows, K, N, E, dt,
                _ptr(status_buffer(A.device)), _stream())
        else:
            name = "moe_grouped_gemm"
            rc = _lib.load().moe_grouped_gemm(epilogue, _ptr(A), _ptr(B), _ptr(B2), _ptr(offsets), _ptr(dst_rows),
                                              _ptr(row_w), _ptr(out), out.stride(0), max_rows, expected_rows, K, N, E,
                                              dt, _ptr(status_buffer(A.device)), _stream())
    _lib.check(rc, name)
    _after(A.device)
    return out


def combine(Yk: torch.Tensor, k: int, shared: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            row_of: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
            T: Optional[int] = None) -> torch.Tensor:
    """out[t] = shared[t] + sum_s scale[t*k+s] * Yk[row_of[t*k+s]] (fp32 sum, one bf16 rounding);
    row_of defaults to the identity and scale to 1."""
    _need_cuda(Yk, shared)
    n, H = Yk.shape
    if T is None:
        T = (row_of.numel() if row_of is not None else n) // k
    dt = _dtype_code(Yk, shared)
    if out is None:
        out = torch.empty(T, H, dtype=Yk.dtype, device=Yk.device)
    with torch.cuda.device(Yk.device):
        rc = _lib.load().moe_combine(_ptr(Yk), _ptr(shared), _ptr(row_of), _ptr(scale), T, k, H, dt, _ptr(out), _stream())
    _lib.check(rc, "moe_combine")
    return out


_dense_offsets = {}


def _offsets_0_T(T: int, device: torch.device) -> torch.Tensor:
    """Device tensor [0, T] (int32): the group table of a dense, single-group GEMM."""
    key = (T, device.index)
    t = _dense_offsets.get(key)
    if t is None:
        t = torch.tensor([0, T], dtype=torch.int32, device=device)
        _dense_offsets[key] = t
    return t


def router_logits(x: torch.Tensor, router_weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 logits [T,E] = x [T,H] . Wr[E,H]^T from 16-bit inputs, fp32 accumulate.
    Few experts (E <= 32, weight within 200 KB): one warp per token on CUDA cores.  Otherwise the tcgen05 GEMM with fp32 output
    (the router weight is one dense group [1,E,H])."""
    _need_cuda(x, router_weight)
    dt = _dtype_code(x, router_weight)
    T, H = x.shape
    E = router_weight.shape[0]
    if out is None:
        out = torch.empty(T, E, dtype=torch.float32, device=x.device)
    x = x.contiguous()
    router_weight = router_weight.contiguous()
    small = E <= 32 and E * H * 2 <= 200 * 1024        # the whole router weight fits one CTA's shared memory
    if not small and E % 8 == 0 and T > 0:
        return grouped_gemm_sorted(GEMM_PLAIN_F32, x, router_weight.unsqueeze(0), _offsets_0_T(T, x.device), out=out)
    with torch.cuda.device(x.device):
        rc = _lib.load().moe_router_logits(_ptr(x), _ptr(router_weight), T, H, E, dt, _ptr(out),
                                           _ptr(status_buffer(x.device)), _stream())
    _lib.check(rc, "moe_router_logits")
    return out


def router_topk_fused_supported(H: int, E: int, k: int) -> bool:
    """Shapes the one-kernel router (moe_router_topk) takes; others run as router_logits + topk_softmax."""
    if H % 8 or k < 1 or k > E:
        return False
    if E <= 32 and E * H * 2 <= 200 * 1024:
        return True
    return E % 8 == 0 and 8 <= E <= 256 and k <= 8


def router_splits(T: int, H: int) -> int:
    """K slices the few-token router GEMM is cut into (the library's rule, restated for the dispatch below)."""
    row_tiles = (T + 127) // 128
    S = 1
    while S < 16 and row_tiles * S * 2 <= 148 and H % (64 * S * 2) == 0 and H // (S * 2) >= 256:
        S *= 2
    return S


def _router_topk_splitk(x, router_weight, k, mode, index_dtype, logits_out):
    T, H = x.shape
    E = router_weight.shape[0]
    dt = _dtype_code(x, router_weight)
    if index_dtype not in (torch.int64, torch.int32):
        raise ValueError("index_dtype must be int64 or int32")
    x = x.contiguous()
    router_weight = router_weight.contiguous()
    lib = _lib.load()
    need = lib.moe_router_topk_splitk_workspace(T, H, E)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    scores = torch.empty(T, k, dtype=torch.float32, device=x.device)
    idx = torch.empty(T, k, dtype=index_dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.moe_router_topk_splitk(_ptr(x), _ptr(router_weight), T, H, E, k, _MODES[mode], dt, _ptr(scores),
                                        _ptr(idx) if index_dtype == torch.int64 else None,
                                        _ptr(idx) if index_dtype == torch.int32 else None, _ptr(logits_out), _ptr(ws),
                                        ws.numel(), _ptr(status_buffer(x.device)), _stream())
    _lib.check(rc, "moe_router_topk_splitk")
    _after(x.device)
    return scores, idx


def router_topk_softmax(x: torch.Tensor, router_weight: torch.Tensor, k: int, mode="B",
                        index_dtype: torch.dtype = torch.int64, logits_out: Optional[torch.Tensor] = None,
                        fused: Optional[bool] = None):
    """scores, indices of top-k + softmax over the router logits x . Wr^T (reference
    kernels/router_gemm_topk_softmax.py computes the same pair in one kernel).  One launch when the shape allows
    (CUDA cores for E <= 32, else the tcgen05 GEMM with the selection in its epilogue): the [T,E] logits are only
    written if ``logits_out`` is given.  Other shapes: router GEMM, then topk_softmax on its fp32 logits.
    ``fused``: None = pick by shape, True / False = force the one-kernel / two-kernel path, "splitk" = force the
    few-token path (GEMM split along K, then a kernel that adds the slices and selects)."""
    _need_cuda(x, router_weight)
    T, H = x.shape
    E = router_weight.shape[0]
    small_e = E <= 32 and E * H * 2 <= 200 * 1024
    if fused is None:
        # Measured on B200: with few row tiles the selection in the epilogue is not hidden behind another tile's
        # main loop, and the separate top-k kernel (all SMs) is quicker; from about 32 tokens per expert the single
        # kernel wins (T=16384: 93 vs 124 us at E=256, 44 vs 48 us at E=64).  Few experts: always one kernel.
        # Few tokens (at most a quarter of the SMs would get a row tile): the GEMM is split along K instead.
        if not small_e and router_splits(T, H) >= 4 and E % 8 == 0 and 8 <= E <= 256 and k <= 32:
            fused = "splitk"
        else:
            fused = E <= 64 or T >= 32 * E
    if fused == "splitk":
        return _router_topk_splitk(x, router_weight, k, mode, index_dtype, logits_out)
    if not fused or not router_topk_fused_supported(H, E, k) or T == 0:
        return topk_softmax(router_logits(x, router_weight, out=logits_out), k, mode=mode, index_dtype=index_dtype)
    dt = _dtype_code(x, router_weight)
    if index_dtype not in (torch.int64, torch.int32):
        raise ValueError("index_dtype must be int64 or int32")
    x = x.contiguous()
    router_weight = router_weight.contiguous()
    if logits_out is not None and (logits_out.shape != (T, E) or logits_out.dtype != torch.float32
                                   or not logits_out.is_contiguous()):
        raise ValueError("logits_out must be a contiguous fp32 [T,E] tensor")
    scores = torch.empty(T, k, dtype=torch.float32, device=x.device)
    idx = torch.empty(T, k, dtype=index_dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().moe_router_topk(_ptr(x), _ptr(router_weight), T, H, E, k, _MODES[mode], dt,
                                         _ptr(scores), _ptr(idx) if index_dtype == torch.int64 else None,
                                         _ptr(idx) if index_dtype == torch.int32 else None, _ptr(logits_out),
                                         _ptr(status_buffer(x.device)), _stream())
    _lib.check(rc, "moe_router_topk")
    _after(x.device)
    return scores, idx


# ----------------------------------------------------------------------------- mHC pre / post blocks
def mhc_split_weights(fn: torch.Tensor) -> torch.Tensor:
    """fn fp32 [R, K] -> bf16 [3R, K] (hi, mid, lo; hi + mid + lo == fn to 24 bits).  Once per weight."""
    _need_cuda(fn)
    if fn.dtype != torch.float32 or fn.dim() != 2:
        raise ValueError("fn must be a 2-D float32 tensor")
    fn = fn.contiguous()
    R, K = fn.shape
    fn3 = torch.empty(3 * R, K, dtype=torch.bfloat16, device=fn.device)
    with torch.cuda.device(fn.device):
        rc = _lib.load().moe_mhc_split_weights(_ptr(fn), R, K, _ptr(fn3), _stream())
    _lib.check(rc, "moe_mhc_split_weights")
    return fn3


def mhc_pre(residual: torch.Tensor, fn3: torch.Tensor, hc_scale: torch.Tensor, hc_base: torch.Tensor,
            rms_eps: float = 1e-6, hc_pre_eps: float = 1e-6, hc_sinkhorn_eps: float = 1e-6,
            hc_post_mult_value: float = 1.0, sinkhorn_repeat: int = 10, workspace: Optional[torch.Tensor] = None):
    """mHC pre block on split weights (mhc_split_weights(fn)).  residual bf16 [T, hc, hidden] ->
    (post_mix fp32 [T,hc,1], comb_mix fp32 [T,hc,hc], layer_input bf16 [T,hidden])."""
    _need_cuda(residual, fn3, hc_scale, hc_base)
    if residual.dtype != torch.bfloat16 or residual.dim() != 3:
        raise ValueError("residual must be bfloat16 [T, hc_mult, hidden]")
    T, hc, hidden = residual.shape
    R = 2 * hc + hc * hc
    if fn3.dtype != torch.bfloat16 or tuple(fn3.shape) != (3 * R, hc * hidden) or not fn3.is_contiguous():
        raise ValueError("fn3 must be the contiguous bfloat16 [3*(2hc+hc^2), hc*hidden] output of mhc_split_weights")
    if hc_scale.dtype != torch.float32 or hc_scale.numel() != 3 or hc_base.dtype != torch.float32 or hc_base.numel() != R:
        raise ValueError("hc_scale must be float32 [3] and hc_base float32 [2hc+hc^2]")
    residual = residual.contiguous()
    dev = residual.device
    lib = _lib.load()
    need = lib.moe_mhc_pre_workspace(T, hc, hidden)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    post = torch.empty(T, hc, 1, dtype=torch.float32, device=dev)
    comb = torch.empty(T, hc, hc, dtype=torch.float32, device=dev)
    layer_input = torch.empty(T, hidden, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        rc = lib.moe_mhc_pre(_ptr(residual), _ptr(fn3), _ptr(hc_scale.contiguous()), _ptr(hc_base.contiguous()), T, hc,
                             hidden, rms_eps, hc_pre_eps, hc_sinkhorn_eps, hc_post_mult_value, sinkhorn_repeat,
                             _ptr(workspace), workspace.numel() * workspace.element_size(), _ptr(post), _ptr(comb),
                             _ptr(layer_input), _ptr(status_buffer(dev)), _stream())
    _lib.check(rc, "moe_mhc_pre")
    _after(dev)
    return post, comb, layer_input


def mhc_post(x: torch.Tensor, residual: torch.Tensor, post_layer_mix: torch.Tensor,
             comb_res_mix: torch.Tensor) -> torch.Tensor:
    """out bf16 [T, hc, hidden] = x * post_layer_mix + comb_res_mix^T @ residual (fp32 arithmetic)."""
    _need_cuda(x, residual, post_layer_mix, comb_res_mix)
    if x.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or residual.dim() != 3:
        raise ValueError("x and residual must be bfloat16, residual [T, hc_mult, hidden]")
    T, hc, hidden = residual.shape
    if tuple(x.shape) != (T, hidden) or post_layer_mix.numel() != T * hc or comb_res_mix.numel() != T * hc * hc:
        raise ValueError("shape mismatch between x, residual and the mixing coefficients")
    if post_layer_mix.dtype != torch.float32 or comb_res_mix.dtype != torch.float32:
        raise ValueError("mixing coefficients must be float32")
    out = torch.empty(T, hc, hidden, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().moe_mhc_post(_ptr(x.contiguous()), _ptr(residual.contiguous()), _ptr(post_layer_mix.contiguous()),
                                      _ptr(comb_res_mix.contiguous()), T, hc, hidden, _ptr(out), _stream())
    _lib.check(rc, "moe_mhc_post")
    return out


def ep_regroup(recv_counts: torch.Tensor, n_recv_bound: int):
    """recv_counts int32 [G, E_local] -> (offsets int32 [E_local+1], src_row int32 [n_recv_bound])."""
    _need_cuda(recv_counts)
    G, El = recv_counts.shape
    dev = recv_counts.device
    offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
    src_row = torch.empty(max(n_recv_bound, 1), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().moe_ep_regroup(_ptr(recv_counts.contiguous()), G, El, _ptr(offsets), _ptr(src_row), _stream())
    _lib.check(rc, "moe_ep_regroup")
    return offsets, src_row


# ----------------------------------------------------------------------------- expert parallelism over peer memory
def _ptr_array(ptrs):
    import ctypes
    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr


def ep_plan(cnt_all: torch.Tensor, G: int, e_local: int, rank: int, cap_rows: int, out: Optional[dict] = None):
    """cnt_all int32 [G, G*e_local] -> (offsets [e_local+1], dst_base [G*e_local], ret_rank [cap], ret_row [cap])."""
    _need_cuda(cnt_all)
    dev = cnt_all.device
    out = {} if out is None else out
    if "offsets" not in out:
        out["offsets"] = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
        out["dst_base"] = torch.empty(G * e_local, dtype=torch.int32, device=dev)
        out["ret_rank"] = torch.empty(cap_rows, dtype=torch.int32, device=dev)
        out["ret_row"] = torch.empty(cap_rows, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().moe_ep_plan(_ptr(cnt_all), G, e_local, rank, _ptr(out["offsets"]), _ptr(out["dst_base"]),
                                     _ptr(out["ret_rank"]), _ptr(out["ret_row"]), _stream())
    _lib.check(rc, "moe_ep_plan")
    return out["offsets"], out["dst_base"], out["ret_rank"], out["ret_row"]


def ep_dispatch(x: torch.Tensor, perm: torch.Tensor, idx32: torch.Tensor, id_map: torch.Tensor, offsets: torch.Tensor,
                dst_base: torch.Tensor, k: int, e_local: int, peer_recv_ptrs, slot_lo: int = 0,
                slot_hi: Optional[int] = None) -> None:
    """Copy the routed rows of x bound for local expert slots [slot_lo, slot_hi) into the destination ranks'
    receive buffers (peer stores)."""
    _need_cuda(x, perm)
    n = perm.numel()
    arr = peer_recv_ptrs if not isinstance(peer_recv_ptrs, (list, tuple)) else _ptr_array(peer_recv_ptrs)
    with torch.cuda.device(x.device):
        rc = _lib.load().moe_ep_dispatch(_ptr(x), _ptr(perm), _ptr(idx32), _ptr(id_map), _ptr(offsets), _ptr(dst_base),
                                         k, e_local, slot_lo, e_local if slot_hi is None else slot_hi, n, x.shape[1],
                                         arr, len(arr), _stream())
    _lib.check(rc, "moe_ep_dispatch")


def ep_unique(idx32: torch.Tensor, id_map: torch.Tensor, e_local: int, G: int, out: Optional[dict] = None):
    """(urank int32 [Tl, G], ucount int32 [G]): per token and destination rank, how many earlier tokens of this rank
    also go there (or -1 if the token has no expert there), and the number of tokens per destination."""
    _need_cuda(idx32, id_map)
    Tl, k = idx32.shape
    out = {} if out is None else out
    if "urank" not in out or out["urank"].shape[0] != Tl:
        out["urank"] = torch.empty(Tl, G, dtype=torch.int32, device=idx32.device)
        out["ucount"] = torch.empty(G, dtype=torch.int32, device=idx32.device)
    with torch.cuda.device(idx32.device):
        rc = _lib.load().moe_ep_unique(_ptr(idx32), _ptr(id_map), Tl, k, e_local, G, _ptr(out["urank"]), _ptr(out["ucount"]),
                                       _stream())
    _lib.check(rc, "moe_ep_unique")
    return out["urank"], out["ucount"]


def ep_plan_dedup(cnt_all: torch.Tensor, G: int, e_local: int, rank: int, cap_rows: int, out: Optional[dict] = None):
    """ep_plan on the [G, E+G] table (counts, then tokens per destination) -> (offsets, dst_base, ret_rank, ret_row,
    u_base [G])."""
    _need_cuda(cnt_all)
    dev = cnt_all.device
    out = {} if out is None else out
    if "offsets" not in out:
        out["offsets"] = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
        out["dst_base"] = torch.empty(G * e_local, dtype=torch.int32, device=dev)
        out["ret_rank"] = torch.empty(cap_rows, dtype=torch.int32, device=dev)
        out["ret_row"] = torch.empty(cap_rows, dtype=torch.int32, device=dev)
    if "u_base" not in out:
        out["u_base"] = torch.empty(G, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().moe_ep_plan_dedup(_ptr(cnt_all), G, e_local, rank, _ptr(out["offsets"]), _ptr(out["dst_base"]),
                                           _ptr(out["ret_rank"]), _ptr(out["ret_row"]), _ptr(out["u_base"]), _stream())
    _lib.check(rc, "moe_ep_plan_dedup")
    return out["offsets"], out["dst_base"], out["ret_rank"], out["ret_row"], out["u_base"]


def ep_dispatch_dedup(x: torch.Tensor, perm: torch.Tensor, idx32: torch.Tensor, id_map: torch.Tensor,
                      offsets: torch.Tensor, dst_base: torch.Tensor, urank: torch.Tensor, u_base: torch.Tensor, k: int,
                      e_local: int, peer_recv_ptrs, peer_gidx_ptrs) -> None:
    """De-duplicated dispatch: every (token, destination rank) row once, plus the received-row number of every
    routed entry into the destination's index list (peer stores)."""
    _need_cuda(x, perm, urank, u_base)
    with torch.cuda.device(x.device):
        rc = _lib.load().moe_ep_dispatch_dedup(_ptr(x), _ptr(perm), _ptr(idx32), _ptr(id_map), _ptr(offsets), _ptr(dst_base),
                                               _ptr(urank), _ptr(u_base), k, e_local, perm.numel(), x.shape[0], x.shape[1],
                                               peer_recv_ptrs, peer_gidx_ptrs, len(peer_recv_ptrs), _stream())
    _lib.check(rc, "moe_ep_dispatch_dedup")


def ep_barrier(peer_flag_ptrs, rank: int, channel: int, epoch: int, device: torch.device,
               timeout_us: int = 1_000_000) -> None:
    """Enqueue the time-limited barrier of the expert-parallel group on the current stream (see the header)."""
    with torch.cuda.device(device):
        rc = _lib.load().moe_ep_barrier(peer_flag_ptrs, len(peer_flag_ptrs), rank, channel, epoch, timeout_us,
                                        _ptr(status_buffer(device)), _stream())
    _lib.check(rc, "moe_ep_barrier")


def ep_share_counts(counts: torch.Tensor, extra: Optional[torch.Tensor], peer_table_ptrs, slot: int, peer_flag_ptrs,
                    rank: int, channel: int, epoch: int, timeout_us: int = 1_000_000) -> None:
    """Store this rank's histogram (counts, then extra) into row [slot][rank] of every rank's table over peer memory
    and run the time-limited barrier behind it: an all-gather of a few hundred ints in one launch."""
    _need_cuda(counts)
    if counts.dtype != torch.int32 or not counts.is_contiguous():
        raise ValueError("counts must be a contiguous int32 vector")
    if extra is not None and (extra.dtype != torch.int32 or not extra.is_contiguous() or extra.device != counts.device):
        raise ValueError("extra must be a contiguous int32 vector on the same device")
    with torch.cuda.device(counts.device):
        rc = _lib.load().moe_ep_share_counts(_ptr(counts), counts.numel(), _ptr(extra), 0 if extra is None else extra.numel(),
                                             peer_table_ptrs, slot, peer_flag_ptrs, len(peer_flag_ptrs), rank, channel,
                                             epoch, timeout_us, _ptr(status_buffer(counts.device)), _stream())
    _lib.check(rc, "moe_ep_share_counts")


def debug_bounds_status(device: torch.device):
    """(checked_build, [code, site, index]): what the index checks of the checked build (libmoe_b200_check.so, loaded
    through MOE_B200_LIBRARY) recorded since the last call; the normal build reports (False, [0, 0, 0])."""
    import ctypes
    out = (ctypes.c_int32 * 3)()
    with torch.cuda.device(device):
        rc = _lib.load().moe_debug_bounds_status(out, _stream())
    if rc < 0:
        _lib.check(rc, "moe_debug_bounds_status")
    return bool(rc), [int(out[0]), int(out[1]), int(out[2])]


def debug_wait_probe(device: torch.device, limit_us: int = 1000) -> int:
    """Run the bounded-wait self-test kernel; returns 1 if the wait succeeded (it cannot), 0 if it ran out."""
    outcome = torch.full((1,), -1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        rc = _lib.load().moe_debug_wait_probe(limit_us, _ptr(status_buffer(device)), _ptr(outcome), _stream())
    _lib.check(rc, "moe_debug_wait_probe")
    return int(outcome.item())


def grouped_gemm_peer_scatter(A: torch.Tensor, B: torch.Tensor, offsets: torch.Tensor, row_rank: torch.Tensor,
                              dst_rows: torch.Tensor, peer_ptrs, ldy: int, max_rows: Optional[int] = None,
                              expected_rows: int = 0) -> None:
    """Expert GEMM whose epilogue stores row r into peer buffer row_rank[r] at row dst_rows[r]."""
    _need_cuda(A, B, offsets)
    rows, K = A.shape
    E, N, _ = B.shape
    arr = peer_ptrs if not isinstance(peer_ptrs, (list, tuple)) else _ptr_array(peer_ptrs)
    with torch.cuda.device(A.device):
        rc = _lib.load().moe_grouped_gemm_peer_scatter(_ptr(A), _ptr(B), _ptr(offsets), _ptr(row_rank), _ptr(dst_rows),
                                                       arr, len(arr), ldy, rows if max_rows is None else max_rows,
                                                       expected_rows, K, N, E, _dtype_code(A, B),
                                                       _ptr(status_buffer(A.device)), _stream())
    _lib.check(rc, "moe_grouped_gemm_peer_scatter")
    _after(A.device)
