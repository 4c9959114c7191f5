"""mHC pre / post blocks through the C ABI against the oracle and the reference's own outputs (fixture)."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O
from tilelang_moe_b200 import kernels, ops

pytestmark = pytest.mark.gpu
KW = dict(rms_eps=1e-6, hc_pre_eps=1e-6, hc_sinkhorn_eps=1e-6, hc_post_mult_value=1.0, sinkhorn_repeat=10)
# fp32 outputs: the mixes come from a 24-bit-exact tensor-core GEMM with fp32 accumulation; sigmoid / Sinkhorn add a
# few ulps.  bf16 outputs: one rounding of an fp32 value, so at most one bf16 ulp (2^-8 relative) apart.
F32_RTOL, F32_ATOL = 2e-5, 2e-6
BF16_RTOL, BF16_ATOL = 2 ** -7, 1e-6


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _check_pre(d, cuda, kw=KW):
    got = kernels.mhc_pre(d["residual"].to(cuda), d["fn"].to(cuda), d["hc_scale"].to(cuda), d["hc_base"].to(cuda), **kw)
    ops.check_status(cuda)
    ref = O.mhc_pre(d["residual"], d["fn"], d["hc_scale"], d["hc_base"], accumulate=torch.float64, **kw)
    torch.testing.assert_close(got[0].cpu(), ref[0], rtol=F32_RTOL, atol=F32_ATOL)
    torch.testing.assert_close(got[1].cpu(), ref[1], rtol=F32_RTOL, atol=F32_ATOL)
    torch.testing.assert_close(got[2].cpu().float(), ref[2].float(), rtol=BF16_RTOL, atol=BF16_ATOL)
    return got


def test_fixture_pre_and_post(cuda, lib):
    g = np.load(GOLDEN / "mhc.npz")
    d = dict(residual=_bf16(g["residual"]), fn=torch.from_numpy(g["fn"]), hc_scale=torch.from_numpy(g["hc_scale"]),
             hc_base=torch.from_numpy(g["hc_base"]))
    post, comb, li = _check_pre(d, cuda)
    assert post.shape == (24, 4, 1) and comb.shape == (24, 4, 4) and li.shape == (24, 256) and li.dtype == torch.bfloat16
    # the reference's own CPU outputs (fp32 evaluation order differs from ours: tolerance, not equality)
    torch.testing.assert_close(post.cpu(), torch.from_numpy(g["ref_post_mix"]), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(comb.cpu(), torch.from_numpy(g["ref_comb_mix"]), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(li.cpu().float(), _bf16(g["ref_layer_input"]).float(), rtol=BF16_RTOL, atol=1e-5)
    out = kernels.mhc_post(_bf16(g["x"]).to(cuda), d["residual"].to(cuda), torch.from_numpy(g["post_layer_mix"]).to(cuda),
                           torch.from_numpy(g["comb_res_mix"]).to(cuda))
    assert out.shape == (24, 4, 256) and out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().float(), _bf16(g["ref_post_out"]).float(), rtol=BF16_RTOL, atol=1e-5)


@pytest.mark.parametrize("T,hidden,hc", [(512, 1280, 4), (1024, 2560, 4), (300, 4096, 4), (1, 64, 4), (130, 136, 4),
                                         (257, 512, 2), (2048, 1024, 4)])
def test_pre_shapes(cuda, lib, T, hidden, hc):
    """The reference benchmark's shapes (benchmarks/benchmark_mhc.py:66-73; the two 4096-wide ones cut to 300 tokens
    here, their full sizes are run by the benchmark), ragged sizes, and hc_mult = 2; the mixing weights scaled up so
    that the sigmoids and the Sinkhorn iteration see a spread of values."""
    d = O.make_mhc_inputs(T, hidden, hc, seed=T + hidden)
    d["fn"] = d["fn"] * 200.0
    post, comb, li = _check_pre(d, cuda)
    assert (comb.sum(-1) - 1).abs().max() < 1e-3 and (comb.sum(-2) - 1).abs().max() < 1e-3     # doubly stochastic


def test_pre_benchmark_distribution_and_parameters(cuda, lib):
    d = O.make_mhc_inputs(640, 2560, 4, seed=42)           # fn ~ 1e-4 as the benchmark draws it
    _check_pre(d, cuda)
    _check_pre(d, cuda, dict(rms_eps=1e-5, hc_pre_eps=1e-3, hc_sinkhorn_eps=1e-4, hc_post_mult_value=2.0,
                             sinkhorn_repeat=3))
    _check_pre(d, cuda, dict(KW, sinkhorn_repeat=1))


def test_split_weights_cover_24_bits(cuda, lib):
    fn = torch.randn(24, 1024, generator=torch.Generator().manual_seed(1)) * 3e-4
    fn3 = ops.mhc_split_weights(fn.to(cuda)).cpu().float().view(3, 24, 1024)
    back = (fn3[0].double() + fn3[1].double() + fn3[2].double()).float()
    assert ((back - fn).abs() <= fn.abs() * 2.0 ** -23).all()


@pytest.mark.parametrize("T,hidden,hc", [(512, 1280, 4), (77, 2560, 4), (1, 8, 4), (300, 4096, 4), (129, 264, 2)])
def test_post_shapes(cuda, lib, T, hidden, hc):
    d = O.make_mhc_inputs(T, hidden, hc, seed=T)
    out = kernels.mhc_post(d["x"].to(cuda), d["residual"].to(cuda), d["post_layer_mix"].to(cuda), d["comb_res_mix"].to(cuda))
    ref = O.mhc_post(d["x"], d["residual"], d["post_layer_mix"], d["comb_res_mix"])
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=BF16_RTOL, atol=1e-5)
    # post is linear in x: doubling x doubles the first term exactly (powers of two commute with bf16 rounding)
    out0 = kernels.mhc_post(torch.zeros_like(d["x"]).to(cuda), d["residual"].to(cuda), d["post_layer_mix"].to(cuda),
                            d["comb_res_mix"].to(cuda))
    ref0 = O.mhc_post(torch.zeros_like(d["x"]), d["residual"], d["post_layer_mix"], d["comb_res_mix"])
    torch.testing.assert_close(out0.cpu().float(), ref0.float(), rtol=BF16_RTOL, atol=1e-5)


def test_rejects_what_is_not_built(cuda, lib):
    d = O.make_mhc_inputs(4, 64, 4)
    with pytest.raises(ValueError):
        kernels.mhc_post(d["x"].float().to(cuda), d["residual"].to(cuda), d["post_layer_mix"].to(cuda), d["comb_res_mix"].to(cuda))
    r3 = torch.zeros(4, 3, 64, dtype=torch.bfloat16, device=cuda)       # hc_mult = 3
    fn = torch.zeros(15, 192, device=cuda)
    from tilelang_moe_b200._lib import MoeLibraryError
    with pytest.raises(MoeLibraryError):
        kernels.mhc_pre(r3, fn, torch.zeros(3, device=cuda), torch.zeros(15, device=cuda))
