"""The CPU oracle replayed against the fixtures produced by the reference's own baseline code."""
import hashlib

import numpy as np
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def test_topk_config1_all_conventions():
    g = np.load(GOLDEN / "topk_c1.npz")
    logits = torch.from_numpy(g["logits"])
    regen = torch.randn(320, 128, generator=torch.Generator().manual_seed(0))
    assert torch.equal(regen, logits), "CPU generator stream differs from the one the fixture was made with"
    for tag, mode in (("B", "B"), ("A", "A"), ("AR", "A_renorm")):
        s, i = O.topk_softmax(logits, 6, mode)
        assert i.dtype == torch.int64 and s.dtype == torch.float32
        assert np.array_equal(i.numpy(), g["idx_" + tag].astype(np.int64))
        assert torch.allclose(s, torch.from_numpy(g["scores_" + tag]), rtol=1e-6, atol=0)
    s, _ = O.topk_softmax(logits, 6, "B")
    assert torch.allclose(s.sum(-1), torch.ones(320), atol=1e-6)


def test_topk_config4_rows():
    g = np.load(GOLDEN / "topk_c4_rows8.npz")
    big = torch.randn(64, 32768, generator=torch.Generator().manual_seed(int(g["seed"])))
    sha = hashlib.sha256(big.view(torch.uint8).numpy().tobytes()).hexdigest()
    assert sha == str(g["sha256_logits"])
    s, i = O.topk_softmax(big[:8], 2048, "B")
    assert np.array_equal(i.numpy(), g["idx_stable"].astype(np.int64))
    assert torch.allclose(s, torch.from_numpy(g["scores_ref"]), rtol=1e-6, atol=0)
    # the reference's own torch.topk order differs only inside runs of equal values
    ref_i = torch.from_numpy(g["idx_ref"].astype(np.int64))
    assert torch.equal(torch.gather(big[:8], 1, ref_i), torch.gather(big[:8], 1, i))


def test_topk_ties_lowest_index_first():
    g = np.load(GOLDEN / "topk_ties.npz")
    q = torch.from_numpy(g["logits"])
    s, i = O.topk_softmax(q, 8, "B")
    assert np.array_equal(i.numpy(), g["idx_stable"].astype(np.int64))
    assert torch.allclose(s, torch.from_numpy(g["scores_ref"]), rtol=1e-6, atol=0)
    v = torch.gather(q, 1, i)
    same = v[:, 1:] == v[:, :-1]
    assert same.any()
    assert (i[:, 1:][same] > i[:, :-1][same]).all()


def test_signed_zero_and_nan_rule():
    x = torch.tensor([[0.0, -0.0, 1.0, float("nan"), -0.0, 0.0]])
    _, i = O.stable_topk(x, 6)
    assert i.tolist() == [[3, 2, 0, 1, 4, 5]]


def test_selecting_on_logits_is_a_valid_selection_on_softmax_scores():
    """The reference's convention A takes torch.topk of the fp32 softmax scores; the oracle and the kernels select on
    the logits.  Softmax is monotone, so the two can differ only where distinct logits round to equal scores, and there
    any of the tied experts is a top-k of the scores.  Checked beyond the fixtures: ordinary rows, rows quantised to
    a few levels (many exact ties) and rows whose entries differ by single units in the last place."""
    g = torch.Generator().manual_seed(11)
    base = torch.randn(2000, 128, generator=g)
    quant = (torch.randn(2000, 128, generator=g) * 2).round() / 2
    near = 3.0 + torch.randint(0, 6, (2000, 128), generator=g).float() * 2.0 ** -21     # ulp-spaced around 3
    for logits in (base, quant, near):
        for k in (1, 6, 8):
            ref_scores = torch.softmax(logits, dim=-1, dtype=torch.float32)
            want, _ = torch.topk(ref_scores, k, dim=-1)
            s, idx = O.topk_softmax(logits, k, "A")
            got = torch.gather(ref_scores, 1, idx)
            assert torch.equal(torch.sort(got, dim=-1, descending=True).values, want)
            # and the scores reported are those values, to the tolerance of the contract
            torch.testing.assert_close(torch.sort(s, dim=-1, descending=True).values, want, rtol=1e-6, atol=1e-30)


def test_histogram_fixture():
    g = np.load(GOLDEN / "histogram.npz")
    idx = torch.from_numpy(g["topk_idx"].astype(np.int64))
    c, o, perm, inv = O.route_histogram(idx, int(g["E"]))
    assert np.array_equal(c.numpy(), g["counts"])
    assert np.array_equal(o.numpy()[1:], g["offsets_inclusive"]) and o[0] == 0
    assert np.array_equal(perm.numpy(), g["perm_stable"])
    assert np.array_equal(inv.numpy(), g["inv"])
    assert c[11] == 0


def test_histogram_empty_and_single():
    c, o, perm, inv = O.route_histogram(torch.zeros(0, 2, dtype=torch.int64), 4)
    assert c.tolist() == [0, 0, 0, 0] and o.tolist() == [0] * 5 and perm.numel() == 0
    c, o, perm, inv = O.route_histogram(torch.tensor([[2, 0]]), 3)
    assert c.tolist() == [1, 0, 1] and o.tolist() == [0, 1, 1, 2] and perm.tolist() == [1, 0]


def test_grouped_gemm_fixture():
    g = np.load(GOLDEN / "grouped_gemm.npz")
    X, W = _bf16(g["X"]), _bf16(g["W"])
    idx = torch.from_numpy(g["idx"].astype(np.int64))
    y = O.grouped_gemm(X, W, idx)
    assert torch.allclose(y, torch.from_numpy(g["y_ref_f32"]), rtol=1e-6, atol=1e-7)
    yb = O.grouped_gemm(X, W, idx, out_dtype=torch.bfloat16)
    assert torch.allclose(yb.float(), _bf16(g["y_ref_bf16"]).float(), rtol=1e-2, atol=2e-2)
    y2 = O.grouped_gemm(X, W, torch.stack([idx, (idx + 1) % 4], 1))
    assert y2.shape == (96, 2, 64) and torch.equal(y2[:, 0], y)


def test_fusedmoe_fixture():
    g = np.load(GOLDEN / "fusedmoe.npz")
    names = ["router_weight", "shared_gate", "shared_up", "shared_down", "routed_gate", "routed_up", "routed_down"]
    x = _bf16(g["x"])
    w = [_bf16(g[n]) for n in names]
    y, sc, ix = O.fusedmoe(x, *w, 2, return_routing=True)
    assert torch.allclose(y, torch.from_numpy(g["y_ref_f32"]), rtol=1e-4, atol=1e-5)
    assert np.array_equal(ix.numpy(), g["topk_idx"].astype(np.int64))
    yb = O.fusedmoe(x, *w, 2, compute_dtype=torch.bfloat16)
    assert torch.allclose(yb.float(), _bf16(g["y_ref_bf16"]).float(), rtol=1e-2, atol=2e-2)
    x2, w2 = O.make_fusedmoe_inputs(1, 48, 128, 64, 6, 1, 2, seed=42)
    assert torch.equal(x2, x) and all(torch.equal(w2[n], t) for n, t in zip(names, w))


def test_zipf_logits_are_skewed():
    lg = O.zipf_logits(4096, 64, 1.1, seed=1)
    _, idx = O.topk_softmax(lg, 4, "A")
    c, *_ = O.route_histogram(idx, 64)
    c = c.sort(descending=True).values.float()
    assert c[0] > 4 * c[32]
    assert (idx.sort(1).values[:, 1:] != idx.sort(1).values[:, :-1]).all()


def test_benchmark_input_recipe_matches_the_oracle_copy():
    from tilelang_moe_b200 import inputs
    assert torch.equal(inputs.zipf_logits(300, 64, 1.1, seed=5), O.zipf_logits(300, 64, 1.1, seed=5))


def test_mhc_oracle_matches_the_reference_fixture():
    """oracle.mhc_pre / mhc_post reproduce, bit for bit, what the reference's kernels/mhc_baseline.py produced on the
    same inputs (outputs stored by oracle/pin_against_reference.py)."""
    g = np.load(GOLDEN / "mhc.npz")
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    residual, fn = bf(g["residual"]), torch.from_numpy(g["fn"])
    post, comb, li = O.mhc_pre(residual, fn, torch.from_numpy(g["hc_scale"]), torch.from_numpy(g["hc_base"]))
    assert torch.equal(post, torch.from_numpy(g["ref_post_mix"]))
    assert torch.equal(comb, torch.from_numpy(g["ref_comb_mix"]))
    assert torch.equal(li, bf(g["ref_layer_input"]))
    out = O.mhc_post(bf(g["x"]), residual, torch.from_numpy(g["post_layer_mix"]), torch.from_numpy(g["comb_res_mix"]))
    assert torch.equal(out, bf(g["ref_post_out"]))
    # the double-precision yardstick used by the GPU tests stays within fp32 rounding of the fp32 evaluation
    p64, c64, _ = O.mhc_pre(residual, fn, torch.from_numpy(g["hc_scale"]), torch.from_numpy(g["hc_base"]),
                            accumulate=torch.float64)
    assert (p64 - post).abs().max() < 1e-5 and (c64 - comb).abs().max() < 1e-5
