"""tcgen05 grouped GEMM through the C ABI against the fp32-accumulated oracle."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe_oracle as O
from tilelang_moe_b200 import kernels, ops

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-2   # bf16 outputs vs fp32-accumulated reference


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _close(y, ref):
    torch.testing.assert_close(y.float().cpu(), ref.float(), rtol=RTOL, atol=ATOL)


def test_fixture(cuda, lib):
    g = np.load(GOLDEN / "grouped_gemm.npz")
    X, W = _bf16(g["X"]), _bf16(g["W"])
    idx = torch.from_numpy(g["idx"].astype(np.int64))
    y = kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda))
    ops.check_status(cuda)
    assert y.shape == (96, 64) and y.dtype == torch.bfloat16
    _close(y, torch.from_numpy(g["y_ref_f32"]))
    _close(y, _bf16(g["y_ref_bf16"]))
    # far tighter than the contract in practice: one rounding of an fp32 accumulation
    assert (y.float().cpu() - torch.from_numpy(g["y_ref_f32"])).abs().max() < 4e-3


def test_config2_top2(cuda, lib):
    g = torch.Generator().manual_seed(0)
    X = torch.randn(4096, 1024, generator=g).bfloat16()
    W = (torch.randn(8, 256, 1024, generator=g) * 0.02).bfloat16()
    idx = torch.argsort(torch.rand(4096, 8, generator=g), dim=1)[:, :2].contiguous()
    y = kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda))
    ops.check_status(cuda)
    assert y.shape == (4096, 2, 256)
    _close(y, O.grouped_gemm(X, W, idx))
    # the reference-equivalent flattened call gives the same rows
    y1 = kernels.grouped_gemm(X.repeat_interleave(2, 0).to(cuda), W.to(cuda), idx.reshape(-1).to(cuda))
    assert torch.equal(y1.view(4096, 2, 256), y)
    # (E,H,I) layout option
    y2 = kernels.grouped_gemm(X.to(cuda), W.transpose(1, 2).contiguous().to(cuda), idx.to(cuda), w_layout="EHI")
    assert torch.equal(y2, y)


@pytest.mark.parametrize("T,H,I,E", [(1, 64, 8, 1), (130, 72, 24, 3), (257, 128, 136, 4), (1000, 200, 264, 7),
                                     (64, 4096, 128, 2), (3000, 512, 512, 16), (5, 64, 64, 32), (2048, 1024, 768, 5)])
def test_ragged_shapes(cuda, lib, T, H, I, E):
    g = torch.Generator().manual_seed(T + H + I)
    X = torch.randn(T, H, generator=g).bfloat16()
    W = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    idx = torch.randint(0, E, (T,), generator=g)
    y = kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda))
    ops.check_status(cuda)
    _close(y, O.grouped_gemm(X, W, idx))


def test_all_rows_one_expert_and_empty_experts(cuda, lib):
    g = torch.Generator().manual_seed(4)
    X = torch.randn(700, 256, generator=g).bfloat16()
    W = (torch.randn(6, 256, 256, generator=g) * 0.05).bfloat16()
    idx = torch.full((700,), 4, dtype=torch.int64)
    _close(kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda)), O.grouped_gemm(X, W, idx))
    ops.check_status(cuda)


def test_epilogues(cuda, lib):
    g = torch.Generator().manual_seed(6)
    T, k, H, I, E = 500, 2, 256, 384, 6
    x = torch.randn(T, H, generator=g).bfloat16()
    Wg = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16()
    Wu = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16()
    Wd = (torch.randn(E, H, I, generator=g) * 0.06).bfloat16()
    idx = torch.argsort(torch.rand(T, E, generator=g), dim=1)[:, :k].contiguous()
    sc = torch.rand(T, k, generator=g)
    _, offs, perm, _ = O.route_histogram(idx, E)
    xs = x[perm.long() // k]
    eid = torch.repeat_interleave(torch.arange(E), (offs[1:] - offs[:-1]).long())
    act_ref = torch.nn.functional.silu(O.grouped_gemm(xs, Wg, eid)) * O.grouped_gemm(xs, Wu, eid)
    act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, xs.to(cuda), Wg.to(cuda), offs.to(cuda), B2=Wu.to(cuda))
    _close(act, act_ref)
    w_sorted = sc.view(-1)[perm.long()]
    yk = ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, act, Wd.to(cuda), offs.to(cuda), dst_rows=perm.to(cuda),
                                 row_w=w_sorted.to(cuda))
    yk_ref = torch.empty(T * k, H)
    yk_ref[perm.long()] = O.grouped_gemm(act.cpu(), Wd, eid) * w_sorted[:, None]
    _close(yk, yk_ref)
    f32 = ops.grouped_gemm_sorted(ops.GEMM_PLAIN_F32, xs.to(cuda), Wg.to(cuda), offs.to(cuda))
    torch.testing.assert_close(f32.cpu(), O.grouped_gemm(xs, Wg, eid), rtol=1e-4, atol=1e-4)
    ops.check_status(cuda)


@pytest.mark.parametrize("tile_rows", ["128", "pair"])
@pytest.mark.parametrize("H,I", [(256, 256), (192, 512)])
def test_both_tile_shapes_on_ragged_groups(cuda, lib, tile_rows, H, I, monkeypatch):
    """The single-CTA kernel (128-row tiles) and the CTA-pair kernel (cta_group::2: 256-row tiles, and a 128-row tile
    with 64 rows per CTA for an expert's last rows) on the same ragged problem: experts with 0, 1, 63, 64, 65, 127, 128,
    129, 255, 256, 257, 300, 384, 385 and 1000 rows exercise every tail case of both kernels."""
    monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", tile_rows)
    g = torch.Generator().manual_seed(8)
    sizes = [0, 1, 127, 128, 129, 255, 256, 257, 300, 1000, 0, 513, 63, 64, 65, 384, 385]
    E = len(sizes)
    idx = torch.cat([torch.full((n,), e, dtype=torch.int64) for e, n in enumerate(sizes)])
    idx = idx[torch.randperm(idx.numel(), generator=g)]
    T = idx.numel()
    x = torch.randn(T, H, generator=g).bfloat16()
    Wg = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16()
    Wu = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16()
    Wd = (torch.randn(E, H, I, generator=g) * 0.06).bfloat16()
    _close(kernels.grouped_gemm(x.to(cuda), Wg.to(cuda), idx.to(cuda)), O.grouped_gemm(x, Wg, idx))
    _, offs, perm, _ = O.route_histogram(idx, E)
    xs = x[perm.long()]
    eid = idx[perm.long()]
    act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, xs.to(cuda), Wg.to(cuda), offs.to(cuda), B2=Wu.to(cuda))
    _close(act, torch.nn.functional.silu(O.grouped_gemm(xs, Wg, eid)) * O.grouped_gemm(xs, Wu, eid))
    w = torch.rand(T, generator=g)
    yk = ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, act, Wd.to(cuda), offs.to(cuda), dst_rows=perm.to(cuda),
                                 row_w=w.to(cuda))
    ref = torch.empty(T, H)
    ref[perm.long()] = O.grouped_gemm(act.cpu(), Wd, eid) * w[:, None]
    _close(yk, ref)
    ops.check_status(cuda)


def test_float16_inputs(cuda, lib):
    """fp16 is the reference wrappers' own dtype (kernels/grouped_gemm_tilelang.py:664): same kernels, other
    instruction-descriptor format and output conversion."""
    g = torch.Generator().manual_seed(12)
    T, H, I, E = 777, 384, 256, 5
    X = torch.randn(T, H, generator=g).half()
    W = (torch.randn(E, I, H, generator=g) * 0.05).half()
    idx = torch.randint(0, E, (T,), generator=g)
    y = kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda))
    ops.check_status(cuda)
    assert y.dtype == torch.float16
    torch.testing.assert_close(y.float().cpu(), O.grouped_gemm(X, W, idx), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("tile_rows", ["128", "pair"])
@pytest.mark.parametrize("T,k,H,I,E,dtype", [(300, 1, 64, 40, 3, torch.bfloat16), (1000, 2, 256, 384, 6, torch.bfloat16),
                                             (4096, 8, 1024, 512, 64, torch.bfloat16), (777, 4, 448, 264, 9, torch.float16),
                                             (5, 2, 128, 64, 40, torch.bfloat16), (2000, 4, 512, 256, 12, torch.bfloat16)])
def test_fused_row_gather_is_bit_identical_to_gather_then_gemm(cuda, lib, T, k, H, I, E, dtype, tile_rows, monkeypatch):
    """The kernel's own row fetch (cp.async into the swizzled operand stage) must feed the tensor cores exactly
    what the TMA path reads from a pre-gathered matrix: every output bit equal, for each epilogue, in the single-CTA
    kernel and in the CTA-pair kernel (where the second CTA's rows are announced to the leader across the cluster)."""
    monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", tile_rows)
    g = torch.Generator().manual_seed(T + k + H)
    x = torch.randn(T, H, generator=g).to(dtype).to(cuda)
    Wg = (torch.randn(E, I, H, generator=g) * 0.06).to(dtype).to(cuda)
    Wu = (torch.randn(E, I, H, generator=g) * 0.06).to(dtype).to(cuda)
    idx = torch.argsort(torch.rand(T, E, generator=g), dim=1)[:, :k].contiguous().to(cuda)
    _, offsets, perm, _ = ops.route_histogram(idx, E, want_inv=False)
    xs = ops.gather_rows(x, perm, div=k)
    n = T * k
    ref_gate = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, xs, Wg, offsets, B2=Wu)
    got_gate = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x, Wg, offsets, B2=Wu, gather=perm, gather_div=k)
    ref_plain = ops.grouped_gemm_sorted(ops.GEMM_PLAIN, xs, Wg, offsets, dst_rows=perm,
                                        out=torch.zeros(n, I, dtype=dtype, device=cuda))
    got_plain = ops.grouped_gemm_sorted(ops.GEMM_PLAIN, x, Wg, offsets, dst_rows=perm, gather=perm, gather_div=k,
                                        out=torch.zeros(n, I, dtype=dtype, device=cuda))
    ref_f32 = ops.grouped_gemm_sorted(ops.GEMM_PLAIN_F32, xs, Wg, offsets)
    got_f32 = ops.grouped_gemm_sorted(ops.GEMM_PLAIN_F32, x, Wg, offsets, gather=perm, gather_div=k)
    ops.check_status(cuda)
    assert got_gate.shape == (n, I)
    assert torch.equal(got_gate, ref_gate)
    assert torch.equal(got_plain, ref_plain)
    assert torch.equal(got_f32, ref_f32)


def test_fused_row_gather_rejects_unsupported_k(cuda, lib):
    x = torch.zeros(8, 72, dtype=torch.bfloat16, device=cuda)
    W = torch.zeros(1, 8, 72, dtype=torch.bfloat16, device=cuda)
    offs = torch.tensor([0, 8], dtype=torch.int32, device=cuda)
    perm = torch.arange(8, dtype=torch.int32, device=cuda)
    with pytest.raises(ValueError):
        ops.grouped_gemm_sorted(ops.GEMM_PLAIN, x, W, offs, gather=perm)


@pytest.mark.parametrize("tile_rows", ["128", "pair"])
def test_scale_scatter_weight_read_at_destination(cuda, lib, tile_rows, monkeypatch):
    """SCALE_SCATTER_DSTW reads the routing weight at the destination row (the [T,k] score matrix itself when
    dst = perm): same bits as SCALE_SCATTER fed with the weights gathered into sorted order."""
    monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", tile_rows)
    g = torch.Generator().manual_seed(11)
    T, k, H, I, E = 900, 4, 256, 192, 10
    act = torch.randn(T * k, I, generator=g).bfloat16().to(cuda)
    Wd = (torch.randn(E, H, I, generator=g) * 0.06).bfloat16().to(cuda)
    scores = torch.rand(T, k, generator=g).to(cuda)
    idx = torch.argsort(torch.rand(T, E, generator=g), dim=1)[:, :k].contiguous().to(cuda)
    _, offsets, perm, _ = ops.route_histogram(idx, E, want_inv=False)
    w_sorted = scores.reshape(-1)[perm.long()].contiguous()
    ref = ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, act, Wd, offsets, dst_rows=perm, row_w=w_sorted)
    got = ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER_DSTW, act, Wd, offsets, dst_rows=perm, row_w=scores.reshape(-1))
    ops.check_status(cuda)
    assert torch.equal(got, ref)


def test_pair_kernel_gives_the_bits_of_the_single_cta_kernel(cuda, lib, monkeypatch):
    """Both kernels accumulate every output element over K in the same order in fp32 and round once, so the tile
    shape must not show in the result: SiLU-gate and scale-scatter outputs bit-equal on a ragged problem."""
    g = torch.Generator().manual_seed(21)
    sizes = [700, 3, 0, 130, 64, 257, 128, 1025]
    E, H, I = len(sizes), 512, 384
    idx = torch.cat([torch.full((n,), e, dtype=torch.int64) for e, n in enumerate(sizes)])
    T = idx.numel()
    x = torch.randn(T, H, generator=g).bfloat16().to(cuda)
    Wg = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16().to(cuda)
    Wu = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16().to(cuda)
    Wd = (torch.randn(E, 256, I, generator=g) * 0.06).bfloat16().to(cuda)
    offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device=cuda)
    w = torch.rand(T, generator=g).to(cuda)
    perm = torch.randperm(T, generator=g).int().to(cuda)
    out = {}
    for mode in ("128", "pair"):
        monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", mode)
        act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x, Wg, offs, B2=Wu)
        yk = ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, act, Wd, offs, dst_rows=perm, row_w=w)
        out[mode] = (act, yk)
    ops.check_status(cuda)
    assert torch.equal(out["128"][0], out["pair"][0])
    assert torch.equal(out["128"][1], out["pair"][1])


def test_bounded_wait_runs_out_and_the_stream_stays_usable(cuda, lib):
    """The GEMM kernels wait on their barriers with a time limit.  A one-warp kernel waits through the same routine on
    a barrier nobody arrives on, with a 1 ms limit: it must return, leave {2, site, block} in the status word (which
    check_status turns into an exception), and a GEMM launched afterwards on the same stream must still be right."""
    from tilelang_moe_b200 import _lib
    ops.check_status(cuda)
    assert ops.debug_wait_probe(cuda, limit_us=1000) == 0
    assert ops.status_buffer(cuda).tolist()[:3] == [2, 99, 0]
    with pytest.raises(_lib.MoeLibraryError, match="device status"):
        ops.check_status(cuda)
    g = torch.Generator().manual_seed(5)
    X = torch.randn(300, 128, generator=g).bfloat16()
    W = (torch.randn(3, 64, 128, generator=g) * 0.05).bfloat16()
    idx = torch.randint(0, 3, (300,), generator=g)
    _close(kernels.grouped_gemm(X.to(cuda), W.to(cuda), idx.to(cuda)), O.grouped_gemm(X, W, idx))
    ops.check_status(cuda)


def test_outputs_stay_inside_their_rows(cuda, lib, monkeypatch):
    """Canary rows before and after every output buffer of the ragged up / down GEMMs and of the permutation: a store
    one row outside a buffer would go unseen in a freshly allocated tensor, here it changes a canary."""
    for mode in ("128", "pair"):
        monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", mode)
        g = torch.Generator().manual_seed(31)
        sizes = [0, 1, 127, 129, 255, 257, 384, 0, 65]
        E, H, I, pad = len(sizes), 256, 256, 64
        idx = torch.cat([torch.full((n,), e, dtype=torch.int64) for e, n in enumerate(sizes)])
        idx = idx[torch.randperm(idx.numel(), generator=g)].to(cuda)
        T = idx.numel()
        x = torch.randn(T, H, generator=g).bfloat16().to(cuda)
        Wg = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16().to(cuda)
        Wu = (torch.randn(E, I, H, generator=g) * 0.06).bfloat16().to(cuda)
        Wd = (torch.randn(E, H, I, generator=g) * 0.06).bfloat16().to(cuda)
        counts, offsets, perm, _ = ops.route_histogram(idx.int(), E, want_inv=False)
        assert sorted(perm.tolist()) == list(range(T))
        act_buf = torch.full((T + 2 * pad, I), 77.0, dtype=torch.bfloat16, device=cuda)
        yk_buf = torch.full((T + 2 * pad, H), 77.0, dtype=torch.bfloat16, device=cuda)
        act, yk = act_buf[pad:pad + T], yk_buf[pad:pad + T]
        ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x, Wg, offsets, B2=Wu, out=act, gather=perm, gather_div=1)
        ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER_DSTW, act, Wd, offsets, dst_rows=perm,
                                row_w=torch.ones(T, device=cuda), out=yk)
        ops.check_status(cuda)
        for buf in (act_buf, yk_buf):
            assert (buf[:pad] == 77.0).all() and (buf[pad + T:] == 77.0).all(), f"a store left its buffer ({mode})"
        assert not (act == 77.0).all(dim=1).any() and not (yk == 77.0).all(dim=1).any()   # every row was written


def test_two_devices_in_one_process(lib):
    """The opt-in for large dynamic shared memory is a per-device attribute of a kernel: a process that drives two GPUs
    must get it on each of them (a process-wide flag would make the first GEMM on the second device fail)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    g = torch.Generator().manual_seed(9)
    X = torch.randn(700, 256, generator=g).bfloat16()
    W = (torch.randn(4, 256, 256, generator=g) * 0.05).bfloat16()
    idx = torch.randint(0, 4, (700,), generator=g)
    ref = O.grouped_gemm(X, W, idx)
    for d in (0, 1, 0):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            y = kernels.grouped_gemm(X.to(dev), W.to(dev), idx.to(dev))
            ops.check_status(dev)
        _close(y, ref)
