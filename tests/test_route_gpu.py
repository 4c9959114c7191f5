"""Histogram / offsets / stable permutation, row gather and combine on the GPU (bit-exact)."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O
from tilelang_moe_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _check(idx_cpu, E, dev):
    c_ref, o_ref, p_ref, i_ref = O.route_histogram(idx_cpu, E)
    c, o, p, i = ops.route_histogram(idx_cpu.to(dev), E)
    ops.check_status(dev)
    assert torch.equal(c.cpu(), c_ref) and torch.equal(o.cpu(), o_ref)
    assert torch.equal(p.cpu(), p_ref) and torch.equal(i.cpu(), i_ref)


def test_fixture(cuda, lib):
    g = np.load(GOLDEN / "histogram.npz")
    idx = torch.from_numpy(g["topk_idx"])
    c, o, p, i = ops.route_histogram(idx.to(cuda), int(g["E"]))
    assert np.array_equal(c.cpu().numpy(), g["counts"])
    assert np.array_equal(o.cpu().numpy()[1:], g["offsets_inclusive"])
    assert np.array_equal(p.cpu().numpy(), g["perm_stable"]) and np.array_equal(i.cpu().numpy(), g["inv"])


@pytest.mark.parametrize("T,k,E,dtype", [(1, 1, 1, torch.int64), (1024, 2, 8, torch.int64), (8192, 8, 256, torch.int32),
                                         (4096, 2, 8, torch.int64), (333, 3, 17, torch.int32), (5000, 6, 160, torch.int64),
                                         (100000, 4, 64, torch.int32), (70, 8, 1024, torch.int64),
                                         # three-kernel path: more experts than threads in the scan kernel (two chunks);
                                         # an expert count that leaves scan threads unused (96 -> 10 shares of the
                                         # units); small units with 16 shares; large units right above the switch
                                         (3000, 4, 2048, torch.int32), (9000, 8, 96, torch.int64),
                                         (6000, 8, 40, torch.int32), (8200, 8, 256, torch.int32),
                                         (1030, 4, 300, torch.int32)])
def test_shapes(cuda, lib, T, k, E, dtype):
    g = torch.Generator().manual_seed(T + k + E)
    idx = torch.argsort(torch.rand(T, E, generator=g), dim=1)[:, :k].contiguous().to(dtype) if E >= k and T * E < 5e6 \
        else torch.randint(0, E, (T, k), generator=g, dtype=dtype)
    _check(idx, E, cuda)


def test_skewed_and_empty_experts(cuda, lib):
    lg = O.zipf_logits(8192, 256, 1.1, seed=0)
    _, idx = O.topk_softmax(lg, 8, "A")
    _check(idx, 256, cuda)
    one = torch.full((3000, 2), 5, dtype=torch.int64)
    _check(one, 9, cuda)
    c, o, p, i = ops.route_histogram(torch.zeros(0, 2, dtype=torch.int64, device=cuda), 4)
    assert c.cpu().tolist() == [0, 0, 0, 0] and o.cpu().tolist() == [0] * 5 and p.numel() == 0


def test_out_of_range_id_sets_status(cuda, lib):
    idx = torch.tensor([[0, 3], [7, 1], [2, -1]], dtype=torch.int64, device=cuda)
    c, o, p, i = ops.route_histogram(idx, 4)
    assert c.cpu().tolist() == [1, 1, 1, 1] and int(o[-1]) == 4
    with pytest.raises(_lib.MoeLibraryError):
        ops.check_status(cuda)
    ops.check_status(cuda)  # cleared by the failed check


def test_gather_and_combine(cuda, lib):
    g = torch.Generator().manual_seed(1)
    T, k, H, E = 300, 4, 256, 16
    x = torch.randn(T, H, generator=g).bfloat16()
    idx = torch.argsort(torch.rand(T, E, generator=g), dim=1)[:, :k].contiguous()
    sc = torch.rand(T, k, generator=g)
    _, _, perm, _ = O.route_histogram(idx, E)
    xs, wsrt = ops.gather_rows(x.to(cuda), perm.to(cuda), div=k, w_src=sc.to(cuda))
    assert torch.equal(xs.cpu(), x[(perm.long() // k)]) and torch.equal(wsrt.cpu(), sc.view(-1)[perm.long()])
    yk = torch.randn(T * k, H, generator=g).bfloat16()
    sh = torch.randn(T, H, generator=g).bfloat16()
    ref = (yk.float().view(T, k, H).sum(1) + sh.float()).bfloat16()
    out = ops.combine(yk.to(cuda), k, shared=sh.to(cuda))
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1e-2, atol=2e-2)
    out2 = ops.combine(yk.to(cuda), k)
    # fp32 sum in slot order, rounded once: reproduce exactly
    acc = torch.zeros(T, H)
    for s in range(k):
        acc += yk.float().view(T, k, H)[:, s]
    assert torch.equal(out2.cpu(), acc.bfloat16())


def test_ep_plan_tables(cuda, lib):
    """The expert-parallel plan tables against a direct restatement of their definition."""
    g = torch.Generator().manual_seed(3)
    G, El = 4, 6
    E = G * El
    cnt = torch.randint(0, 40, (G, E), generator=g, dtype=torch.int32)
    cnt[1, 7] = 0
    cnt[:, 13] = 0
    for me in range(G):
        cap = int(cnt[:, me * El:(me + 1) * El].sum()) + 5
        offs, dst_base, ret_rank, ret_row = ops.ep_plan(cnt.to(cuda), G, El, me, cap)
        tot = cnt.sum(0).long()
        # expert-major start of every virtual expert on its destination
        dbase = torch.zeros(E, dtype=torch.long)
        for d in range(G):
            dbase[d * El:(d + 1) * El] = torch.cumsum(tot[d * El:(d + 1) * El], 0) - tot[d * El:(d + 1) * El]
        want_offs = torch.cat([dbase[me * El:(me + 1) * El], tot[me * El:(me + 1) * El].sum().view(1)])
        assert torch.equal(offs.cpu().long(), want_offs)
        want_dst = dbase + cnt[:me].sum(0).long()
        assert torch.equal(dst_base.cpu().long(), want_dst)
        src_off = torch.cumsum(cnt.long(), 1) - cnt.long()           # each source's own sorted order
        rr, rw = ret_rank.cpu(), ret_row.cpu()
        for j in range(El):
            v = me * El + j
            q = int(dbase[v])
            for s_ in range(G):
                c = int(cnt[s_, v])
                assert (rr[q:q + c] == s_).all()
                assert torch.equal(rw[q:q + c].long(), int(src_off[s_, v]) + torch.arange(c))
                q += c
