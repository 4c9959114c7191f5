"""CPU stand-ins for the device ops, used only to run the expert-parallel host protocol on gloo ranks.
Same call signatures as tilelang_moe_b200.ops; arithmetic in the dtype of the inputs."""
import torch

from oracle import moe_oracle as O

GEMM_PLAIN, GEMM_SILU_GATE, GEMM_SCALE_SCATTER, GEMM_PLAIN_F32 = 0, 1, 2, 3


def topk_softmax(logits, k, mode="B", index_dtype=torch.int64, also_int32=False):
    s, i = O.topk_softmax(logits, k, mode)
    return s, i.to(index_dtype)


def route_histogram(topk_idx, n_experts, want_perm=True, want_inv=True, workspace=None, id_map=None):
    ids = topk_idx.reshape(-1).long()
    if id_map is not None:
        ids = id_map.long()[ids]
    return O.route_histogram(ids, n_experts)


def gather_rows(src, perm, div=1, out=None, w_src=None, w_out=None, n_rows=None):
    n = perm.numel() if n_rows is None else n_rows
    rows = src[(perm[:n].long() // div)]
    if out is not None:
        out[:n] = rows
        rows = out[:n]
    return rows


def ep_regroup(recv_counts, n_recv_bound):
    G, El = recv_counts.shape
    cnt = recv_counts.long()
    in_start = (torch.cumsum(cnt.reshape(-1), 0) - cnt.reshape(-1)).view(G, El)
    offsets = torch.zeros(El + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(cnt.sum(0), 0).int()
    src_row = torch.zeros(max(n_recv_bound, 1), dtype=torch.int32)
    p = 0
    for j in range(El):
        for s in range(G):
            c = int(cnt[s, j])
            src_row[p:p + c] = torch.arange(int(in_start[s, j]), int(in_start[s, j]) + c, dtype=torch.int32)
            p += c
    return offsets, src_row


def grouped_gemm_sorted(epilogue, A, B, offsets, B2=None, dst_rows=None, row_w=None, out=None, out_rows=None,
                        max_rows=None):
    rows = A.shape[0]
    E, N, K = B.shape
    res = torch.zeros(rows if out is None else out.shape[0], N, dtype=A.dtype)
    for e in range(E):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if s == t:
            continue
        y = A[s:t] @ B[e].T
        if epilogue == GEMM_SILU_GATE:
            y = torch.nn.functional.silu(y) * (A[s:t] @ B2[e].T)
        if epilogue == GEMM_SCALE_SCATTER:
            y = y * row_w[s:t, None]
        dst = dst_rows[s:t].long() if dst_rows is not None and epilogue != GEMM_SILU_GATE else torch.arange(s, t)
        res[dst] = y
    if out is not None:
        out.copy_(res)
        return out
    return res


def combine(Yk, k, shared=None, out=None, row_of=None, scale=None, T=None):
    n = row_of.numel() if row_of is not None else Yk.shape[0]
    rows = Yk[row_of.long()] if row_of is not None else Yk
    if scale is not None:
        rows = rows * scale.reshape(-1, 1).to(rows.dtype)
    res = rows.view(n // k, k, -1).sum(1)
    if shared is not None:
        res = res + shared
    return res
