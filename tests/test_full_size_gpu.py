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
