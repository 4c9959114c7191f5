"""The fused MoE layer on the GPU against the fp32 oracle and the reference fixture."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O
from tilelang_moe_b200 import kernels, layer, ops

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-2
NAMES = ["router_weight", "shared_gate", "shared_up", "shared_down", "routed_gate", "routed_up", "routed_down"]


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _gap_rows(logits, k, eps=1e-5):
    v = torch.sort(logits, dim=-1, descending=True).values
    return (v[:, k - 1] - v[:, k]) < eps


def test_fixture(cuda, lib):
    g = np.load(GOLDEN / "fusedmoe.npz")
    x = _bf16(g["x"]).to(cuda)
    w = [_bf16(g[n]).to(cuda) for n in NAMES]
    y, sc, ix = layer.moe_forward(x, *w, 2, return_routing=True)
    ops.check_status(cuda)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    assert np.array_equal(ix.cpu().numpy(), g["topk_idx"])
    torch.testing.assert_close(sc.cpu(), torch.from_numpy(g["topk_scores"]), rtol=1e-5, atol=1e-8)
    torch.testing.assert_close(y.float().cpu(), torch.from_numpy(g["y_ref_f32"]), rtol=RTOL, atol=ATOL)
    y2 = kernels.fusedmoe_tilelang(x, *w, 2)
    assert torch.equal(y2, y)


def test_config3_small(cuda, lib):
    x, w = O.make_fusedmoe_inputs(1, 1024, 2048, 512, 8, 1, 2, dtype=torch.bfloat16, seed=42)
    logits = O.router_logits(x.view(-1, 2048), w["router_weight"])
    # router GEMM checked to tolerance on its own ...
    lg = ops.router_logits(x.view(-1, 2048).to(cuda), w["router_weight"].to(cuda))
    torch.testing.assert_close(lg.cpu(), logits, rtol=1e-4, atol=1e-5)
    # ... and the layer from one shared fp32 logits tensor, so a last-ulp logit cannot flip an expert
    ref, sc_ref, ix_ref = O.fusedmoe(x, *[w[n] for n in NAMES], 2, logits=logits, return_routing=True)
    m = kernels.FusedMoETileLang(2048, 512, 8, 1, 2, 1, 1024, dtype=torch.bfloat16)
    y = m.forward(x.to(cuda), *[w[n].to(cuda) for n in NAMES], logits=logits.to(cuda))
    ops.check_status(cuda)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=RTOL, atol=ATOL)
    # end to end with the GPU's own logits: identical except on rows with a near-tie at the k-th place
    y_e2e = m.forward(x.to(cuda), *[w[n].to(cuda) for n in NAMES])
    bad = ~torch.isclose(y_e2e.float().cpu(), ref, rtol=RTOL, atol=ATOL).view(1024, -1).all(-1)
    assert (bad & ~_gap_rows(logits, 2)).sum() == 0


def test_no_shared_expert_skewed_routing(cuda, lib):
    g = torch.Generator().manual_seed(3)
    T, H, I, E, k = 512, 512, 256, 32, 4
    x = torch.randn(T, H, generator=g).bfloat16()
    Wg = (torch.randn(E, I, H, generator=g) * 0.02).bfloat16()
    Wu = (torch.randn(E, I, H, generator=g) * 0.02).bfloat16()
    Wd = (torch.randn(E, H, I, generator=g) * 0.02).bfloat16()
    logits = O.zipf_logits(T, E, 1.1, seed=3)
    ref = O.fusedmoe(x, None, None, None, None, Wg, Wu, Wd, k, logits=logits)
    y = layer.moe_forward(x.to(cuda), None, None, None, None, Wg.to(cuda), Wu.to(cuda), Wd.to(cuda), k,
                          logits=logits.to(cuda))
    ops.check_status(cuda)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=RTOL, atol=ATOL)


def test_float16_layer_default_dtype_of_the_reference(cuda, lib):
    x, w = O.make_fusedmoe_inputs(2, 96, 256, 128, 8, 1, 2, dtype=torch.float16, seed=7)
    logits = O.router_logits(x.view(-1, 256), w["router_weight"])
    ref = O.fusedmoe(x, *[w[n] for n in NAMES], 2, logits=logits)
    m = kernels.FusedMoETileLang(256, 128, 8, 1, 2, 2, 96)            # dtype defaults to float16, as in the reference
    y = m.forward(x.to(cuda), *[w[n].to(cuda) for n in NAMES], logits=logits.to(cuda))
    ops.check_status(cuda)
    assert y.dtype == torch.float16 and y.shape == x.shape
    torch.testing.assert_close(y.float().cpu(), ref, rtol=RTOL, atol=ATOL)
    x2, w2 = kernels.generate_fusedmoe_inputs(1, 8, 64, 32, 4, 1, 2, device="cuda")
    assert x2.dtype == torch.float16 and w2["routed_down"].shape == (4, 64, 32)


def test_graph_replay_matches_eager(cuda, lib):
    x, w = O.make_fusedmoe_inputs(1, 256, 512, 256, 8, 1, 2, dtype=torch.bfloat16, seed=11)
    m = kernels.FusedMoETileLang(512, 256, 8, 1, 2, 1, 256, dtype=torch.bfloat16)
    xd = x.to(cuda)
    wd = [w[n].to(cuda) for n in NAMES]
    eager = m.forward(xd, *wd).clone()
    run = m.capture(xd, *wd)
    assert torch.equal(run(), eager)
    # new activations written in place into the static input
    x2 = torch.randn(1, 256, 512, generator=torch.Generator().manual_seed(5)).bfloat16()
    xd.copy_(x2.to(cuda))
    got = run().clone()
    assert torch.equal(got, m.forward(xd, *wd))
    ops.check_status(cuda)


def test_host_pipeline_overlaps_copies_and_keeps_results(cuda, lib):
    from tilelang_moe_b200.pipeline import HostPipeline
    g = torch.Generator().manual_seed(2)
    T, H, I, E, k = 256, 256, 128, 8, 2
    x = torch.randn(T, H, generator=g).bfloat16().pin_memory()
    lg = torch.randn(T, E, generator=g).pin_memory()
    Wg = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16().to(cuda)
    Wu = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16().to(cuda)
    Wd = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().to(cuda)
    ws = layer.MoEWorkspace(T, k, H, I, E, 0, cuda)

    def compute(xd, lgd, outd):
        sc, ix = ops.topk_softmax(lgd, k, mode="A", index_dtype=torch.int32)
        layer.routed_forward(xd, sc, ix, Wg, Wu, Wd, ws, out=outd)

    pipe = HostPipeline(cuda, [x, lg], (T, H), torch.bfloat16, compute)
    last = pipe.run(5)
    torch.cuda.synchronize()
    ref = O.fusedmoe(x, None, None, None, None, Wg.cpu(), Wu.cpu(), Wd.cpu(), k, logits=lg)
    torch.testing.assert_close(last.float(), ref, rtol=RTOL, atol=ATOL)
    assert torch.equal(pipe.out_host[0], pipe.out_host[1])     # every step computed the same batch
    assert pipe.h2d_bytes == T * H * 2 + T * E * 4 and pipe.d2h_bytes == T * H * 2


@pytest.mark.parametrize("B,S,H,I,E,NS,k,dtype", [(1, 300, 512, 256, 8, 1, 2, torch.bfloat16),     # shared expert, few experts
                                                 (2, 128, 256, 128, 64, 0, 6, torch.bfloat16),    # no shared expert
                                                 (1, 200, 200, 72, 16, 2, 4, torch.float16),      # H % 64 != 0: gather pass
                                                 (1, 2304, 1024, 128, 64, 1, 8, torch.bfloat16)]) # enough rows for the one-kernel router
def test_single_call_layer_equals_the_staged_calls(cuda, lib, B, S, H, I, E, NS, k, dtype):
    """moe_layer_forward (one C call) only sequences the library's own entry points: its output must equal, bit for
    bit, the layer issued stage by stage from Python - with the router computed from x and from given logits."""
    x, w = O.make_fusedmoe_inputs(B, S, H, I, E, NS, k, dtype=dtype, seed=B + S)
    xd = x.to(cuda)
    wd = [w[n].to(cuda) for n in NAMES]
    if NS == 0:
        wd[1] = wd[2] = wd[3] = None
    m = kernels.FusedMoETileLang(H, I, E, NS, k, B, S, dtype=dtype)
    y1 = m.forward(xd, *wd).clone()
    y0 = layer.moe_forward(xd, *wd, k).clone()
    ops.check_status(cuda)
    assert y1.shape == x.shape and torch.equal(y1, y0)
    # a single shared expert of the routed width ran as expert E of the routed GEMMs (stacked weights kept by the layer
    # object); the same layer with the stacking switched off takes the side-stream form: all three agree bit for bit
    assert (getattr(m, "_stack", None) is not None) == (NS == 1 and H % 64 == 0)
    if NS == 1:
        m2 = kernels.FusedMoETileLang(H, I, E, NS, k, B, S, dtype=dtype)
        m2.STACK_LIMIT_BYTES = 0
        assert torch.equal(m2.forward(xd, *wd), y0) and getattr(m2, "_stack", None) is None
    lg = ops.router_logits(xd.view(-1, H), wd[0])
    y1l = m.forward(xd, *wd, logits=lg).clone()
    y0l = layer.moe_forward(xd, *wd, k, logits=lg).clone()
    assert torch.equal(y1l, y0l)
    ref = O.fusedmoe(x, *[w[n] for n in NAMES], k, logits=lg.cpu())
    torch.testing.assert_close(y1l.float().cpu(), ref, rtol=RTOL, atol=ATOL)
    # and as one replayed CUDA graph
    replay = m.capture(xd, *wd, logits=lg)
    assert torch.equal(replay(), y0l)
