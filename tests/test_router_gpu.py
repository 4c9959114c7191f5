"""TopK+softmax on the GPU through the C ABI, against the oracle and the reference fixtures."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O
from tilelang_moe_b200 import kernels, ops

pytestmark = pytest.mark.gpu
RTOL = 1e-6  # fp32 softmax scores, relative


def _check(logits_cpu, k, mode, dev, rtol=RTOL, oracle_slack=False):
    s_ref, i_ref = O.topk_softmax(logits_cpu, k, mode)
    s, i = ops.topk_softmax(logits_cpu.to(dev), k, mode=mode)
    ops.check_status(dev)
    assert i.dtype == torch.int64 and s.dtype == torch.float32
    assert torch.equal(i.cpu(), i_ref), f"indices differ (mode {mode}, shape {tuple(logits_cpu.shape)}, k={k})"
    if oracle_slack:
        # quantised inputs repeat the same addend thousands of times, which biases an fp32 running sum:
        # the fp32 oracle itself is then ~1e-6 away from the exact softmax.  Hold the kernel to 1e-6 of the
        # exact (fp64) value, and to 1e-6 plus the oracle's own measured error against the oracle.
        exact = torch.softmax(torch.gather(logits_cpu, 1, i_ref).double(), -1)
        torch.testing.assert_close(s.cpu().double(), exact, rtol=rtol, atol=1e-30)
        rtol = rtol + float(((s_ref.double() - exact).abs() / exact).max())
    torch.testing.assert_close(s.cpu(), s_ref, rtol=rtol, atol=1e-30)
    return s, i


def test_config1_fixture(cuda, lib):
    g = np.load(GOLDEN / "topk_c1.npz")
    logits = torch.from_numpy(g["logits"]).to(cuda)
    for tag, mode in (("B", "B"), ("A", "A"), ("AR", "A_renorm")):
        s, i = kernels.topk_softmax(logits, 6, mode=mode)
        assert np.array_equal(i.cpu().numpy(), g["idx_" + tag].astype(np.int64))
        torch.testing.assert_close(s.cpu(), torch.from_numpy(g["scores_" + tag]), rtol=RTOL, atol=1e-30)


def test_config4_radix_full(cuda, lib):
    big = torch.randn(64, 32768, generator=torch.Generator().manual_seed(0))
    s, i = _check(big, 2048, "B", cuda)
    g = np.load(GOLDEN / "topk_c4_rows8.npz")
    assert np.array_equal(i[:8].cpu().numpy(), g["idx_stable"].astype(np.int64))
    torch.testing.assert_close(s[:8].cpu(), torch.from_numpy(g["scores_ref"]), rtol=RTOL, atol=1e-30)
    # against an fp64 softmax of the selected values as well
    v = torch.gather(big, 1, i.cpu()).double()
    torch.testing.assert_close(s.cpu().double(), torch.softmax(v, -1), rtol=RTOL, atol=1e-30)


def test_ties_fixture(cuda, lib):
    g = np.load(GOLDEN / "topk_ties.npz")
    s, i = kernels.topk_softmax(torch.from_numpy(g["logits"]).to(cuda), 8)
    assert np.array_equal(i.cpu().numpy(), g["idx_stable"].astype(np.int64))
    torch.testing.assert_close(s.cpu(), torch.from_numpy(g["scores_ref"]), rtol=RTOL, atol=1e-30)


@pytest.mark.parametrize("M,N,k", [(1, 8, 2), (7, 16, 4), (33, 31, 5), (64, 64, 8), (512, 128, 8), (100, 160, 6),
                                   (256, 256, 8), (50, 500, 32), (40, 512, 64), (16, 1000, 33), (9, 1024, 64),
                                   (512, 8, 8), (3, 1, 1)])
@pytest.mark.parametrize("mode", ["B", "A", "A_renorm"])
def test_warp_path_shapes(cuda, lib, M, N, k, mode):
    lg = torch.randn(M, N, generator=torch.Generator().manual_seed(M * 131 + N))
    _check(lg, k, mode, cuda)


@pytest.mark.parametrize("M,N,k", [(4, 2048, 2048), (5, 1025, 7), (3, 4096, 100), (2, 32768, 1), (6, 3000, 65),
                                   (8, 512, 128), (2, 65536, 4096), (130, 8192, 256), (1, 131072, 2048),
                                   (300, 2048, 96)])
@pytest.mark.parametrize("mode", ["B", "A", "A_renorm"])
def test_radix_path_shapes(cuda, lib, M, N, k, mode):
    lg = torch.randn(M, N, generator=torch.Generator().manual_seed(M * 7 + N + k))
    _check(lg, k, mode, cuda)


def test_radix_ties_straddling_the_threshold(cuda, lib):
    # heavy quantisation: many equal values exactly at the k-th place, spread over all slices
    g = torch.Generator().manual_seed(5)
    q = torch.round(torch.randn(16, 16384, generator=g) * 4) / 4
    _check(q, 1000, "B", cuda, oracle_slack=True)
    _check(q, 77, "B", cuda, oracle_slack=True)
    const = torch.zeros(3, 5000)
    _check(const, 1234, "B", cuda, oracle_slack=True)


def test_row_stride_and_unaligned(cuda, lib):
    base = torch.randn(20, 300, generator=torch.Generator().manual_seed(2)).to(cuda)
    view = base[:, 3:203]                      # ld=300, offset 3 floats: not 16-byte aligned
    s, i = ops.topk_softmax(view, 5)
    s_ref, i_ref = O.topk_softmax(view.cpu(), 5)
    assert torch.equal(i.cpu(), i_ref)
    big = torch.randn(4, 9001, generator=torch.Generator().manual_seed(3)).to(cuda)
    s, i = ops.topk_softmax(big[:, 1:], 300)
    s_ref, i_ref = O.topk_softmax(big[:, 1:].cpu(), 300)
    assert torch.equal(i.cpu(), i_ref)


def test_signed_zero_nan_and_inf(cuda, lib):
    x = torch.tensor([[0.0, -0.0, 1.0, float("nan"), -0.0, 0.0, float("-inf"), float("inf")]])
    _, i = ops.topk_softmax(x.to(cuda), 8)
    assert i.cpu().tolist() == O.stable_topk(x, 8)[1].tolist() == [[3, 7, 2, 0, 1, 4, 5, 6]]
    wide = torch.zeros(2, 4096)
    wide[0, 100] = float("nan")
    wide[1, 7] = -0.0
    wide[1, 9] = 1.0
    _, i = ops.topk_softmax(wide.to(cuda), 70)
    assert torch.equal(i.cpu(), O.stable_topk(wide, 70)[1])


def test_int32_indices_and_large_m(cuda, lib):
    lg = torch.randn(70000, 128, generator=torch.Generator().manual_seed(9))
    s_ref, i_ref = O.topk_softmax(lg, 6)
    s, i64, i32 = ops.topk_softmax(lg.to(cuda), 6, also_int32=True)
    assert torch.equal(i64.cpu(), i_ref) and torch.equal(i32.cpu().long(), i_ref)
    torch.testing.assert_close(s.cpu(), s_ref, rtol=RTOL, atol=1e-30)


def test_conventions_agree_like_the_reference_test(cuda, lib):
    # reference tests/test_topk_softmax_conventions.py: same expert sets, A-renorm == B to fp32 rounding
    for E, K in ((8, 2), (16, 4), (128, 8), (160, 6), (64, 8)):
        lg = torch.randn(512, E, generator=torch.Generator().manual_seed(42)).to(cuda)
        sb, ib = kernels.topk_softmax(lg, K, mode="B")
        sa, ia = kernels.topk_softmax(lg, K, mode="A")
        sr, ir = kernels.topk_softmax(lg, K, mode="A_renorm")
        assert torch.equal(ib, ia) and torch.equal(ib, ir)
        assert (sb - sr).abs().max().item() < 5e-7
        assert (sa.sum(-1) < 1.0 + 1e-6).all()


@pytest.mark.parametrize("H,E,K", [(3584, 64, 8), (4096, 128, 8), (5120, 160, 6), (2048, 8, 2), (7168, 256, 8)])
def test_router_gemm_then_topk_like_the_reference_fusion_test(cuda, lib, H, E, K):
    """Reference tests/test_router_fusion_correctness.py: T=256, bf16 ~ N(0,1), seed 0; pass = every row selects the
    same expert set as topk(X.float() @ W.float()).  Here also: logits to 1e-4 and, on rows whose k-th / (k+1)-th
    logit gap exceeds 1e-4, identical order and scores."""
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(256, H, generator=g).bfloat16()
    W = torch.randn(E, H, generator=g).bfloat16()
    ref_logits = X.float() @ W.float().T
    lg = ops.router_logits(X.to(cuda), W.to(cuda))
    ops.check_status(cuda)
    torch.testing.assert_close(lg.cpu(), ref_logits, rtol=1e-4, atol=1e-3)
    s, i = ops.router_topk_softmax(X.to(cuda), W.to(cuda), K, fused=True)
    s_ref, i_ref = O.topk_softmax(ref_logits, K, "B")
    sv = torch.sort(ref_logits, dim=-1, descending=True).values
    clear = ((sv[:, :K] - sv[:, 1:K + 1]).min(-1).values > 1e-2)
    assert clear.sum() > 200
    assert torch.equal(torch.sort(i.cpu()[clear], -1).values, torch.sort(i_ref[clear], -1).values)
    assert torch.equal(i.cpu()[clear], i_ref[clear])
    # scores: exact (1e-6) against the softmax of the logits the GPU produced; against the fp32 reference they can
    # only be as close as the logits are (a logit error d moves a score by about d in relative terms)
    s_own, i_own = O.topk_softmax(lg.cpu(), K, "B")
    assert torch.equal(i.cpu(), i_own)
    torch.testing.assert_close(s.cpu(), s_own, rtol=RTOL, atol=1e-30)
    d = float((lg.cpu() - ref_logits).abs().max())
    torch.testing.assert_close(s.cpu()[clear], s_ref[clear], rtol=4 * d + 1e-5, atol=1e-7)


@pytest.mark.parametrize("M,N,k", [(2048, 128, 6), (2500, 8, 2), (2049, 64, 8), (4100, 160, 6), (3000, 256, 8),
                                   (2100, 512, 5), (2050, 1024, 8), (2048, 12, 3), (2200, 300, 7), (2304, 128, 1)])
@pytest.mark.parametrize("mode", ["B", "A", "A_renorm"])
def test_tile_path_shapes(cuda, lib, M, N, k, mode):
    """Thread-per-row tile kernel (M >= 2048, k <= 8, aligned rows): 1, 2, 4 or 8 threads per row."""
    lg = torch.randn(M, N, generator=torch.Generator().manual_seed(M + N + k))
    _check(lg, k, mode, cuda)


def test_tile_path_ties_and_specials(cuda, lib):
    g = torch.Generator().manual_seed(17)
    q = torch.round(torch.randn(2304, 256, generator=g) * 2) / 2          # ties everywhere, across the two halves
    _check(q, 8, "B", cuda, oracle_slack=True)
    # equal values already in the list must keep their order when a larger value arrives later
    y = torch.randn(2048, 128, generator=g)
    y[:, 40] = 1.25; y[:, 45] = 1.25; y[:, 90] = 3.0; y[:, 91] = 1.25
    _check(y, 6, "B", cuda, oracle_slack=True)
    x = torch.randn(2048, 64, generator=g)
    x[5, 10] = float("nan"); x[5, 3] = float("inf"); x[6, :] = 0.0; x[6, 7] = -0.0; x[7, 1] = float("-inf")
    _, i = ops.topk_softmax(x.to(cuda), 4)
    assert torch.equal(i.cpu(), O.stable_topk(x, 4)[1])


@pytest.mark.parametrize("T,H,E,K,dtype", [(300, 512, 64, 8, torch.bfloat16), (1000, 1024, 256, 8, torch.bfloat16),
                                           (129, 256, 160, 6, torch.float16), (77, 2048, 8, 2, torch.bfloat16),
                                           (515, 640, 32, 4, torch.bfloat16), (64, 7168, 256, 1, torch.bfloat16),
                                           (200, 128, 24, 24, torch.bfloat16)])
@pytest.mark.parametrize("mode", ["B", "A", "A_renorm"])
def test_one_kernel_router_equals_gemm_then_topk(cuda, lib, T, H, E, K, dtype, mode):
    """moe_router_topk (selection inside the GEMM's epilogue, or the CUDA-core kernel for few experts) against the
    two separate calls: the same logits bit for bit, hence the same indices; scores to 1e-6.  Inputs are quantised
    so that equal logits occur and the lowest-index rule is exercised."""
    g = torch.Generator().manual_seed(T + E)
    X = (torch.round(torch.randn(T, H, generator=g) * 2) / 2).to(dtype).to(cuda)
    W = (torch.round(torch.randn(E, H, generator=g) * 2) / 8).to(dtype).to(cuda)
    assert ops.router_topk_fused_supported(H, E, K)
    lg = ops.router_logits(X, W)
    s2, i2 = ops.topk_softmax(lg, K, mode=mode)
    lg_out = torch.full((T, E), float("nan"), dtype=torch.float32, device=cuda)
    s1, i1 = ops.router_topk_softmax(X, W, K, mode=mode, logits_out=lg_out, fused=True)
    s32, i32 = ops.router_topk_softmax(X, W, K, mode=mode, index_dtype=torch.int32, fused=True)
    ops.check_status(cuda)
    assert torch.equal(lg_out, lg)
    assert i1.dtype == torch.int64 and i32.dtype == torch.int32
    assert torch.equal(i1, i2) and torch.equal(i32.long(), i2)
    torch.testing.assert_close(s1, s2, rtol=2e-6, atol=1e-30)   # two kernels, each within 1e-6 of the oracle (below)
    assert torch.equal(s32, s1)
    # and against the oracle on those logits (ties lowest index first; scores to the contract's 1e-6)
    s_ref, i_ref = O.topk_softmax(lg.cpu(), K, mode)
    assert torch.equal(i1.cpu(), i_ref)
    torch.testing.assert_close(s1.cpu(), s_ref, rtol=1e-6, atol=1e-30)
    assert (lg.cpu()[:, :-1] == lg.cpu()[:, 1:]).any() or E <= 8     # the quantised inputs do produce equal logits


def test_one_kernel_router_falls_back_for_other_shapes(cuda, lib):
    g = torch.Generator().manual_seed(3)
    X = torch.randn(100, 256, generator=g).bfloat16().to(cuda)
    W = torch.randn(320, 256, generator=g).bfloat16().to(cuda)      # more experts than one accumulator tile holds
    assert not ops.router_topk_fused_supported(256, 320, 4)
    s, i = ops.router_topk_softmax(X, W, 4)
    s2, i2 = ops.topk_softmax(ops.router_logits(X, W), 4)
    assert torch.equal(i, i2) and torch.equal(s, s2)


@pytest.mark.parametrize("T,H,E,K,dtype", [(256, 7168, 256, 8, torch.bfloat16), (1024, 4096, 128, 8, torch.bfloat16),
                                           (77, 5120, 160, 6, torch.float16), (1, 1024, 64, 8, torch.bfloat16),
                                           (300, 3584, 64, 32, torch.bfloat16), (130, 512, 40, 3, torch.bfloat16)])
@pytest.mark.parametrize("mode", ["B", "A", "A_renorm"])
def test_few_token_router_split_along_k(cuda, lib, T, H, E, K, dtype, mode):
    """moe_router_topk_splitk: the logits it reports are the fp32 sums of the K slices (equal to the unsplit GEMM up to
    summation order), and its selection is exactly the oracle's on those logits - ties lowest index first."""
    g = torch.Generator().manual_seed(T + E)
    X = (torch.round(torch.randn(T, H, generator=g) * 2) / 2).to(dtype).to(cuda)
    W = (torch.round(torch.randn(E, H, generator=g) * 2) / 8).to(dtype).to(cuda)
    lg = torch.full((T, E), float("nan"), dtype=torch.float32, device=cuda)
    s, i = ops.router_topk_softmax(X, W, K, mode=mode, logits_out=lg, fused="splitk")
    s32, i32 = ops.router_topk_softmax(X, W, K, mode=mode, index_dtype=torch.int32, fused="splitk")
    ops.check_status(cuda)
    ref_logits = X.float().cpu() @ W.float().cpu().T
    torch.testing.assert_close(lg.cpu(), ref_logits, rtol=1e-4, atol=1e-3)
    s_ref, i_ref = O.topk_softmax(lg.cpu(), K, mode)
    assert torch.equal(i.cpu(), i_ref) and torch.equal(i32.long().cpu(), i_ref)
    torch.testing.assert_close(s.cpu(), s_ref, rtol=1e-6, atol=1e-30)
    assert torch.equal(s32, s)
    if T >= 64:   # with inputs on a coarse grid the split sums are exact, so they equal the unsplit GEMM's logits
        assert torch.equal(lg, ops.router_logits(X, W))


def test_variant_names_of_the_reference_follow_their_conventions(cuda, lib):
    """The reference's other public names: fused / selection / sonic / bitonic select first and normalise over the k
    chosen, separate / tilelang_separate normalise over all experts first, topk_radix_tilelang returns indices only."""
    from tilelang_moe_b200 import kernels as K
    logits = torch.randn(333, 160, generator=torch.Generator().manual_seed(5))
    sB, iB = O.topk_softmax(logits, 6, "B")
    sA, iA = O.topk_softmax(logits, 6, "A")
    d = logits.to(cuda)
    for f in (K.topk_softmax_fused, K.topk_softmax_selection, K.topk_softmax_sonic, K.topk_softmax_bitonic, K.topk_softmax_best):
        s, i = f(d, 6)
        assert torch.equal(i.cpu(), iB)
        torch.testing.assert_close(s.cpu(), sB, rtol=1e-6, atol=1e-30)
    for f in (K.topk_softmax_separate, K.topk_softmax_separate_compiled, K.topk_softmax_tilelang_separate):
        s, i = f(d, 6)
        assert torch.equal(i.cpu(), iA)
        torch.testing.assert_close(s.cpu(), sA, rtol=1e-6, atol=1e-30)
    assert torch.equal(K.topk_radix_tilelang(d, 6).cpu(), iB)


@pytest.mark.parametrize("H,E,K", [(3584, 64, 8), (5120, 160, 6)])
def test_fused_router_factories_of_the_reference_module(cuda, lib, H, E, K):
    """kernels.router_gemm_topk_softmax as the reference's tests/test_router_fusion_correctness.py uses it: a factory
    call per shape, then kernel(X[T,H], W[H,E_padded]); pass = every row selects the expert set of
    topk(X.float() @ W.float())."""
    from tilelang_moe_b200.kernels import router_gemm_topk_softmax as R
    torch.manual_seed(0)
    X = torch.randn(256, H, device=cuda, dtype=torch.bfloat16)
    W = torch.randn(H, E, device=cuda, dtype=torch.bfloat16)
    Ep = R._next_pow2(E)
    Wp = torch.zeros(H, Ep, device=cuda, dtype=torch.bfloat16)
    Wp[:, :E] = W
    logits = X.float() @ W.float()
    vals, ref_i = torch.topk(logits, K, dim=-1)
    ref_s = torch.softmax(vals, dim=-1)
    sv = torch.sort(logits, dim=-1, descending=True).values
    clear = ((sv[:, :K] - sv[:, 1:K + 1]).min(-1).values > 1e-2)          # rows whose order no rounding can change
    for kern in (R.fused_router_tma_auto_bitonic_kernel(256, H, E, Ep, K, block_M=64, block_K=64, num_stages=2, threads=256),
                 R.get_fused_router_kernel("cpasync_selection", 256, H, E, K)):
        scores, idx = kern(X, Wp)
        ops.check_status(cuda)
        assert torch.equal(torch.sort(idx[clear], -1).values, torch.sort(ref_i[clear], -1).values)
        assert (scores[clear] - ref_s[clear]).abs().max().item() < 2e-3
    with pytest.raises(ValueError):
        R.get_fused_router_kernel("no_such_algorithm", 256, H, E, K)
    lg = R.get_router_gemm_kernel(256, H, E)(X, W)                         # the stand-alone router GEMM of the same module
    assert lg.dtype == torch.float32 and lg.shape == (256, E)
    torch.testing.assert_close(lg, logits, rtol=1e-4, atol=1e-3)
