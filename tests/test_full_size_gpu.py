"""The DeepSeek-V3-shaped layer at its full benchmark size (T=8192, H=7168, I=2048, E=256, top-8, Zipf load):
too large for a whole-batch CPU oracle inside a test, so it is checked through size-independent properties and a
sampled-token oracle."""
import pytest
import torch

from oracle import moe_oracle as O
from tilelang_moe_b200 import inputs, layer, ops

pytestmark = pytest.mark.gpu
T, H, I, E, K = 8192, 7168, 2048, 256, 8


@pytest.fixture(scope="module")
def big(cuda):
    free, _ = torch.cuda.mem_get_info(cuda)
    if free < 40 * (1 << 30):
        pytest.skip("needs ~30 GB of free device memory")
    g = torch.Generator(device=cuda)
    g.manual_seed(77)
    Wg = torch.empty(E, I, H, dtype=torch.bfloat16, device=cuda)
    Wu = torch.empty(E, I, H, dtype=torch.bfloat16, device=cuda)
    Wd = torch.empty(E, H, I, dtype=torch.bfloat16, device=cuda)
    for e in range(E):
        Wg[e] = torch.randn(I, H, generator=g, device=cuda).mul_(0.02)
        Wu[e] = torch.randn(I, H, generator=g, device=cuda).mul_(0.02)
        Wd[e] = torch.randn(H, I, generator=g, device=cuda).mul_(0.02)
    x = inputs.activations(T, H, seed=5).to(cuda)
    logits = inputs.zipf_logits(T, E, 1.1, seed=5).to(cuda)
    ws = layer.MoEWorkspace(T, K, H, I, E, 0, cuda)
    return dict(Wg=Wg, Wu=Wu, Wd=Wd, x=x, logits=logits, ws=ws)


def _run(b, x, logits):
    sc, ix = ops.topk_softmax(logits, K, mode="A", index_dtype=torch.int32)
    return layer.routed_forward(x, sc, ix, b["Wg"], b["Wu"], b["Wd"], b["ws"]).clone(), sc, ix


def test_sampled_tokens_against_the_fp32_oracle(cuda, big):
    y, sc, ix = _run(big, big["x"], big["logits"])
    ops.check_status(cuda)
    # routing of the whole batch: bit-exact indices, scores to 1e-6
    s_ref, i_ref = O.topk_softmax(big["logits"].cpu(), K, "A")
    assert torch.equal(ix.cpu().long(), i_ref)
    torch.testing.assert_close(sc.cpu(), s_ref, rtol=1e-6, atol=1e-30)
    # per-expert offsets of the whole batch: bit-exact
    c_ref, o_ref, p_ref, _ = O.route_histogram(i_ref, E)
    c, o, p, _ = ops.route_histogram(ix, E)
    assert torch.equal(c.cpu(), c_ref) and torch.equal(o.cpu(), o_ref) and torch.equal(p.cpu(), p_ref)
    # 256 tokens spread over the batch, end to end against the fp32 CPU oracle: the experts they use (nearly all of
    # them) travel to the host one at a time and each processes its share of the sampled tokens
    toks = torch.linspace(0, T - 1, 256).long()
    xs = big["x"][toks.to(cuda)].float().cpu()
    ref = torch.zeros(toks.numel(), H)
    users = {}
    for i, t in enumerate(toks.tolist()):
        for s in range(K):
            users.setdefault(int(i_ref[t, s]), []).append((i, float(s_ref[t, s])))
    for e, lst in sorted(users.items()):
        rows = torch.tensor([i for i, _ in lst])
        w = torch.tensor([v for _, v in lst]).unsqueeze(1)
        out = O.expert_ffn(xs[rows], big["Wg"][e].float().cpu(), big["Wu"][e].float().cpu(), big["Wd"][e].float().cpu())
        ref.index_add_(0, rows, out * w)
    assert len(users) > 200
    torch.testing.assert_close(y[toks.to(cuda)].float().cpu(), ref, rtol=1e-2, atol=2e-2)


def test_token_permutation_permutes_the_output_bit_exactly(cuda, big):
    """Every output row depends on its own token only, whatever tile it lands in: shuffling the batch must shuffle the
    result and change nothing else (exercises every ragged tile boundary at full size)."""
    y, _, _ = _run(big, big["x"], big["logits"])
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(3)).to(cuda)
    y2, _, _ = _run(big, big["x"][perm].contiguous(), big["logits"][perm].contiguous())
    ops.check_status(cuda)
    assert torch.equal(y2, y[perm])


def test_routing_weight_linearity(cuda, big):
    """Doubling every routing weight doubles the output exactly (a power-of-two scale commutes with every rounding)."""
    sc, ix = ops.topk_softmax(big["logits"], K, mode="A", index_dtype=torch.int32)
    y1 = layer.routed_forward(big["x"], sc, ix, big["Wg"], big["Wu"], big["Wd"], big["ws"]).clone()
    y2 = layer.routed_forward(big["x"], sc * 2.0, ix, big["Wg"], big["Wu"], big["Wd"], big["ws"]).clone()
    assert torch.equal(y2.float(), y1.float() * 2.0)


def test_eight_emulated_ranks_at_full_size_equal_the_single_gpu_layer(cuda, big):
    """The expert-parallel path for 8 ranks at the benchmark's size, the ranks run one after another on this GPU
    (plain torch.stack instead of the histogram exchange, no barriers needed on one stream): placement by row tiles
    with spare expert slots (ranks hold different numbers of experts), de-duplicated dispatch, gathered up GEMM,
    down GEMM scattering into the owners' return buffers, combine.  Must give the single-GPU layer's output to the
    tolerance of the contract (the routing weight meets the bf16 rounding at a different point)."""
    from tilelang_moe_b200 import ep
    G = 8
    Tl = T // G
    y_ref, sc_all, ix_all = _run(big, big["x"], big["logits"])
    calib = inputs.zipf_logits(T, E, 1.1, seed=5, noise_seed=1001).to(cuda)
    _, ixc = ops.topk_softmax(calib, K, mode="A", index_dtype=torch.int32)
    load = ops.route_histogram(ixc, E, want_perm=False, want_inv=False)[0].cpu().tolist()
    slots = E // G + E // G // 4
    e2r = ep.balanced_placement(load, G, cost=ep.tile_cost, max_per_rank=slots)
    plan = ep.EPPlan(E, G, e2r, max(e2r.count(r) for r in range(G)))
    assert len({len(l) for l in plan.local_experts}) > 1
    El, NS = plan.e_local, plan.n_slots
    id_map = torch.tensor(plan.id_map, dtype=torch.int32, device=cuda)
    cap = Tl * K * G
    recv = [torch.empty(cap, H, dtype=torch.bfloat16, device=cuda) for _ in range(G)]
    gidx = [torch.zeros(cap, dtype=torch.int32, device=cuda) for _ in range(G)]
    ret = [torch.zeros(Tl * K, H, dtype=torch.bfloat16, device=cuda) for _ in range(G)]
    recv_ptrs = ops._ptr_array([t.data_ptr() for t in recv])
    gidx_ptrs = ops._ptr_array([t.data_ptr() for t in gidx])
    ret_ptrs = ops._ptr_array([t.data_ptr() for t in ret])
    routed = []
    for s in range(G):
        sl = slice(s * Tl, (s + 1) * Tl)
        scores, idx32 = ops.topk_softmax(big["logits"][sl].contiguous(), K, mode="A", index_dtype=torch.int32)
        counts, offsets, perm, inv = ops.route_histogram(idx32, NS, id_map=id_map)
        urank, ucount = ops.ep_unique(idx32, id_map, El, G)
        routed.append(dict(x=big["x"][sl].contiguous(), scores=scores, idx32=idx32, counts=counts, offsets=offsets, perm=perm,
                           inv=inv, urank=urank, ucount=ucount))
    cnt_all = torch.stack([torch.cat([r["counts"], r["ucount"]]) for r in routed]).contiguous()
    plans = []
    for s in range(G):
        r = routed[s]
        offs_local, dst_base, ret_rank, ret_row, u_base = ops.ep_plan_dedup(cnt_all, G, El, s, cap)
        ops.ep_dispatch_dedup(r["x"], r["perm"], r["idx32"], id_map, r["offsets"], dst_base, r["urank"], u_base, K, El,
                              recv_ptrs, gidx_ptrs)
        plans.append((offs_local, ret_rank, ret_row))
    for d in range(G):
        offs_local, ret_rank, ret_row = plans[d]
        mine = torch.tensor(plan.padded_local_experts(d), device=cuda)
        wg, wu, wd = big["Wg"][mine], big["Wu"][mine], big["Wd"][mine]
        act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, recv[d], wg, offs_local, B2=wu, gather=gidx[d], gather_div=1)
        ops.grouped_gemm_peer_scatter(act, wd, offs_local, ret_rank, ret_row, ret_ptrs, H)
        del wg, wu, wd, act
    for s in range(G):
        r = routed[s]
        out = ops.combine(ret[s], K, row_of=r["inv"], scale=r["scores"].reshape(-1), T=Tl)
        torch.testing.assert_close(out.float(), y_ref[s * Tl:(s + 1) * Tl].float(), rtol=1e-2, atol=2e-2)
    ops.check_status(cuda)
