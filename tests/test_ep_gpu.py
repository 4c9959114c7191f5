"""Expert parallelism on real GPUs (needs >= 2): each rank's slice of the sharded layer against the
single-process fp32 oracle.  NVLS is switched off in NCCL and the symmetric buffers are kept off NVLink multicast
objects, so that a failing rank cannot disturb its peers; workers that outlive a failure are terminated."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, placement, q, exchange="nccl"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    from oracle import moe_oracle as O
    from tilelang_moe_b200 import ep, inputs, ops
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, H, I, E, k = 512, 256, 128, 16, 4
        g = torch.Generator().manual_seed(0)
        x = torch.randn(T, H, generator=g).bfloat16()
        Wg = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
        Wu = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
        Wd = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
        logits = inputs.zipf_logits(T, E, 1.1, seed=1)
        _, idx = O.topk_softmax(logits, k, "A")
        load = O.route_histogram(idx, E)[0].tolist()
        if placement == "tiles":     # by row tiles, ranks may hold different numbers of experts
            skewed = [v * 6 if v == max(load) else v for v in load]
            e2r = ep.balanced_placement(skewed, world, cost=ep.tile_cost, max_per_rank=E // world + 3)
            plan = ep.EPPlan(E, world, e2r, E // world + 3)
            assert len({len(l) for l in plan.local_experts}) > 1
        else:
            e2r = ep.balanced_placement(load, world) if placement == "balanced" else ep.contiguous_placement(E, world)
            plan = ep.EPPlan(E, world, e2r)
        mine = plan.padded_local_experts(rank)
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        bufs = {}
        px = ep.PeerExchange(Tl, k, H, world, dev, dedup=exchange == "peer_dedup") if exchange.startswith("peer") else None
        assert px is None or px.dedup == (exchange == "peer_dedup")
        for _ in range(3):   # later passes reuse the buffers (and, for the peer exchange, overwrite them)
            args = (x[sl].to(dev), logits[sl].to(dev), k, plan, torch.tensor(plan.id_map, dtype=torch.int32, device=dev),
                    Wg[mine].to(dev), Wu[mine].to(dev), Wd[mine].to(dev), ops)
            out = ep.ep_forward_peer(*args, px, bufs=bufs) if px is not None else ep.ep_forward(*args, bufs=bufs)
        ops.check_status(dev)
        ref = O.fusedmoe(x, None, None, None, None, Wg, Wu, Wd, k, logits=logits)[sl]
        ok = torch.isclose(out.float().cpu(), ref, rtol=1e-2, atol=2e-2).all().item()
        q.put((rank, bool(ok), float((out.float().cpu() - ref).abs().max()), None))
    except Exception as e:
        q.put((rank, False, -1.0, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("placement,exchange", [("contiguous", "nccl"), ("balanced", "nccl"), ("contiguous", "peer"),
                                                ("balanced", "peer"), ("contiguous", "peer_dedup"),
                                                ("balanced", "peer_dedup"), ("tiles", "peer_dedup"), ("tiles", "peer"),
                                                ("tiles", "nccl")])
def test_ep_two_gpus_match_oracle(lib, placement, exchange):
    _run_world(2, placement, exchange)


@pytest.mark.parametrize("exchange", ["peer", "peer_dedup"])
def test_ep_four_gpus_match_oracle(lib, exchange):
    _run_world(4, "balanced", exchange)


def _run_world(world, placement, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, placement, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in range(world):
            res.append(q.get(timeout=240))
            if res[-1][3] is not None:      # a rank raised: the others may be waiting for it (their barriers time out)
                break
        for p in procs:
            p.join(timeout=60)
    finally:                                # no worker, and no kernel of one, outlives the test
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    assert len(res) == world or any(r[3] is not None for r in res), "a rank never reported"
    for rank, ok, err, exc in res:
        assert exc is None, f"rank {rank}: {exc}"
        assert ok, f"rank {rank}: max abs error {err}"


@pytest.mark.parametrize("tile_rows,H,I", [("128", 128, 64), ("pair", 256, 128)])
@pytest.mark.parametrize("G,dedup,uneven", [(4, True, False), (8, True, False), (8, False, False), (8, True, True),
                                            (4, False, True)])
def test_peer_exchange_kernels_with_emulated_ranks_on_one_gpu(cuda, lib, G, dedup, uneven, tile_rows, H, I, monkeypatch):
    """The peer-exchange kernels for G ranks run one after another on a single GPU: every "rank" has its own receive,
    index and return buffers on that device, the all-gather is a torch.stack, and no barrier is needed because the
    phases are issued in order on one stream.  Checks the whole path (unique / plan / dispatch / gathered up GEMM /
    scattering down GEMM / combine) against the oracle for 4 and 8 ranks without needing that many GPUs."""
    from oracle import moe_oracle as O
    from tilelang_moe_b200 import ep, inputs, ops
    monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", tile_rows)   # single-CTA kernel, or the CTA-pair kernel's peer epilogue
    dev = cuda
    k, Tl = 4, 96
    E, T = G * 4, G * 96
    g = torch.Generator().manual_seed(G)
    x = torch.randn(T, H, generator=g).bfloat16()
    Wg = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    Wu = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    Wd = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    logits = inputs.zipf_logits(T, E, 1.1, seed=G)
    _, idx = O.topk_softmax(logits, k, "A")
    load = O.route_histogram(idx, E)[0].tolist()
    if uneven:   # placed by row tiles with two spare slots per rank: ranks hold different numbers of experts
        cost = lambda rows: ep.tile_cost(rows, 32)
        plan = ep.EPPlan(E, G, ep.balanced_placement(load, G, cost=cost, max_per_rank=6), 6)
        assert len({len(l) for l in plan.local_experts}) > 1
    else:
        plan = ep.EPPlan(E, G, ep.balanced_placement(load, G))
    El, NS = plan.e_local, plan.n_slots          # expert slots per rank, histogram bins
    id_map = torch.tensor(plan.id_map, dtype=torch.int32, device=dev)
    cap = Tl * k * G
    recv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(G)]
    gidx = [torch.zeros(cap, dtype=torch.int32, device=dev) for _ in range(G)]
    ret = [torch.zeros(Tl * k, H, dtype=torch.bfloat16, device=dev) for _ in range(G)]
    recv_ptrs = ops._ptr_array([t.data_ptr() for t in recv])
    gidx_ptrs = ops._ptr_array([t.data_ptr() for t in gidx])
    ret_ptrs = ops._ptr_array([t.data_ptr() for t in ret])
    routed = []
    for s in range(G):                                               # route on every rank
        sl = slice(s * Tl, (s + 1) * Tl)
        scores, idx32 = ops.topk_softmax(logits[sl].to(dev), k, mode="A", index_dtype=torch.int32)
        counts, offsets, perm, inv = ops.route_histogram(idx32, NS, id_map=id_map)
        urank, ucount = ops.ep_unique(idx32, id_map, El, G) if dedup else (None, None)
        routed.append(dict(x=x[sl].to(dev), scores=scores, idx32=idx32, counts=counts, offsets=offsets, perm=perm, inv=inv,
                           urank=urank, ucount=ucount))
    cnt_all = torch.stack([torch.cat([r["counts"], r["ucount"]]) if dedup else r["counts"] for r in routed]).contiguous()
    plans = []
    for s in range(G):                                               # plan + dispatch from every rank
        r = routed[s]
        if dedup:
            offs_local, dst_base, ret_rank, ret_row, u_base = ops.ep_plan_dedup(cnt_all, G, El, s, cap)
            ops.ep_dispatch_dedup(r["x"], r["perm"], r["idx32"], id_map, r["offsets"], dst_base, r["urank"], u_base, k, El,
                                  recv_ptrs, gidx_ptrs)
        else:
            offs_local, dst_base, ret_rank, ret_row = ops.ep_plan(cnt_all, G, El, s, cap)
            ops.ep_dispatch(r["x"], r["perm"], r["idx32"], id_map, r["offsets"], dst_base, k, El, recv_ptrs)
        plans.append((offs_local, ret_rank, ret_row))
    for d in range(G):                                               # expert GEMMs on every rank
        offs_local, ret_rank, ret_row = plans[d]
        mine = plan.padded_local_experts(d)
        wg, wu, wd = Wg[mine].to(dev), Wu[mine].to(dev), Wd[mine].to(dev)
        if dedup:
            act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, recv[d], wg, offs_local, B2=wu, gather=gidx[d], gather_div=1)
        else:
            act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, recv[d], wg, offs_local, B2=wu)
        ops.grouped_gemm_peer_scatter(act, wd, offs_local, ret_rank, ret_row, ret_ptrs, H)
    ref = O.fusedmoe(x, None, None, None, None, Wg, Wu, Wd, k, logits=logits)
    for s in range(G):                                               # combine on every rank
        r = routed[s]
        out = ops.combine(ret[s], k, row_of=r["inv"], scale=r["scores"].reshape(-1), T=Tl)
        torch.testing.assert_close(out.float().cpu(), ref[s * Tl:(s + 1) * Tl], rtol=1e-2, atol=2e-2)
    ops.check_status(dev)
    if dedup:   # fewer rows travelled than routed entries, and never more than one per (token, rank)
        sent = int(cnt_all[:, NS:].sum())
        assert sent <= T * min(k, G) and sent < T * k


def test_barrier_gives_up_after_its_time_limit_and_reports_it(cuda, lib):
    """The group barrier with a peer that never arrives: two flag blocks on one GPU stand for two ranks, nothing ever
    writes "rank 1"'s slot.  The wait must run out (2 ms here), leave {2, 40 + channel, peer} in the status word and
    return - the stream stays usable - and check_status must raise.  Nothing faults or spins for ever."""
    from tilelang_moe_b200 import _lib, ops
    flags = [torch.zeros(64, dtype=torch.int32, device=cuda) for _ in range(2)]
    ptrs = ops._ptr_array([f.data_ptr() for f in flags])
    ops.check_status(cuda)
    ops.ep_barrier(ptrs, 0, 1, 7, cuda, timeout_us=2000)
    torch.cuda.synchronize(cuda)
    assert ops.status_buffer(cuda).tolist()[:3] == [2, 41, 1]
    assert flags[1][16 + 0].item() == 7 and flags[0][16 + 0].item() == 7      # the arrival itself was published
    with pytest.raises(_lib.MoeLibraryError):
        ops.check_status(cuda)
    ops.check_status(cuda)                                                      # the raise cleared the status word
    # a barrier whose peers have all arrived (slots already at the epoch) passes at once and leaves no status
    flags[0][32:34] = 3
    ops.ep_barrier(ptrs, 0, 2, 3, cuda, timeout_us=2000)
    torch.cuda.synchronize(cuda)
    ops.check_status(cuda)
    y = torch.ones(8, device=cuda) * 2                                          # later work on the stream runs normally
    assert y.sum().item() == 16


def test_share_counts_fills_every_table_and_its_wait_is_limited(cuda, lib):
    """The histogram exchange over peer memory on one GPU: two tables stand for two ranks.  "Rank 0"'s vector must land
    in row [slot][0] of both tables; with the peer's arrival already published the barrier behind it passes, and with a
    peer that never arrives the wait runs out (2 ms) and reports {2, 40 + channel, peer}."""
    from tilelang_moe_b200 import _lib, ops
    counts = torch.arange(1, 9, dtype=torch.int32, device=cuda)
    extra = torch.tensor([70, 80], dtype=torch.int32, device=cuda)
    width = 10
    tables = [torch.full((2 * 2 * width,), -1, dtype=torch.int32, device=cuda) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=cuda) for _ in range(2)]
    tptrs = ops._ptr_array([t.data_ptr() for t in tables])
    fptrs = ops._ptr_array([f.data_ptr() for f in flags])
    ops.check_status(cuda)
    flags[0][3 * 16 + 1] = 5                       # "rank 1" has already arrived at barrier 5 of channel 3
    ops.ep_share_counts(counts, extra, tptrs, 1, fptrs, 0, 3, 5, timeout_us=2000)
    torch.cuda.synchronize(cuda)
    ops.check_status(cuda)
    want = torch.cat([counts, extra])
    for t in tables:
        v = t.view(2, 2, width)
        assert torch.equal(v[1, 0], want)
        assert bool((v[0] == -1).all()) and bool((v[1, 1] == -1).all())      # nothing else was touched
    assert flags[1][3 * 16 + 0].item() == 5 and flags[0][3 * 16 + 0].item() == 5
    # without the extra vector, other slot; the peer never reaches barrier 6
    ops.ep_share_counts(counts, None, ops._ptr_array([t.data_ptr() for t in tables]), 0, fptrs, 0, 3, 6, timeout_us=2000)
    torch.cuda.synchronize(cuda)
    assert ops.status_buffer(cuda).tolist()[:3] == [2, 43, 1]
    with pytest.raises(_lib.MoeLibraryError):
        ops.check_status(cuda)
    assert torch.equal(tables[1][:8], counts)       # row [0][0] at the narrower width of this call


def test_share_counts_builds_the_whole_table_for_eight_ranks(cuda, lib):
    """Eight ranks' histogram exchange, one rank after the other on one GPU (every rank's flags pre-set to the epoch, so
    no launch waits for another): afterwards every rank's table holds every rank's vector in the slot of the step."""
    from tilelang_moe_b200 import ops
    G, n, extra_n, epoch, slot = 8, 272, 8, 3, 1
    width = n + extra_n
    g = torch.Generator().manual_seed(1)
    vecs = [torch.randint(0, 500, (width,), generator=g, dtype=torch.int32).to(cuda) for _ in range(G)]
    tables = [torch.full((2 * G * width,), -7, dtype=torch.int32, device=cuda) for _ in range(G)]
    flags = [torch.zeros(64, dtype=torch.int32, device=cuda) for _ in range(G)]
    for f in flags:
        f[3 * 16:3 * 16 + G] = epoch
    tptrs = ops._ptr_array([t.data_ptr() for t in tables])
    fptrs = ops._ptr_array([f.data_ptr() for f in flags])
    for r in range(G):
        ops.ep_share_counts(vecs[r][:n].contiguous(), vecs[r][n:].contiguous(), tptrs, slot, fptrs, r, 3, epoch, timeout_us=2000)
    torch.cuda.synchronize(cuda)
    ops.check_status(cuda)
    want = torch.stack(vecs)
    for t in tables:
        v = t.view(2, G, width)
        assert torch.equal(v[slot], want)
        assert bool((v[1 - slot] == -7).all())


def test_dispatch_ignores_entries_with_an_expert_id_out_of_range(cuda, lib):
    """One routed entry carries id -1: the histogram reports it (status 1) and leaves it out of the permutation; the
    dispatch kernels must then stop at the live entries - nothing is read through the unwritten tail of the permutation
    and no row beyond the live rows of any receive buffer changes (canary rows stay intact)."""
    from tilelang_moe_b200 import _lib, ops
    G, El, k, Tl, H = 2, 2, 2, 64, 128
    E = G * El
    g = torch.Generator().manual_seed(3)
    idx = torch.argsort(torch.rand(Tl, E, generator=g), dim=1)[:, :k].contiguous().int()
    idx[5, 1] = -1
    idx32 = idx.to(cuda)
    x = torch.randn(Tl, H, generator=g).bfloat16().to(cuda)
    id_map = torch.arange(E, dtype=torch.int32, device=cuda)
    ops.check_status(cuda)
    counts, offsets, perm, inv = ops.route_histogram(idx32, E, id_map=id_map)
    torch.cuda.synchronize(cuda)
    assert ops.status_buffer(cuda).tolist()[0] == 1
    with pytest.raises(_lib.MoeLibraryError):
        ops.check_status(cuda)
    n_live = int(offsets[E].item())
    assert n_live == Tl * k - 1
    cap = Tl * k * G
    for dedup in (False, True):
        canary = torch.full((cap, H), 123.0, dtype=torch.bfloat16, device=cuda)
        recv = [canary.clone() for _ in range(G)]
        gidx = [torch.full((cap,), -7, dtype=torch.int32, device=cuda) for _ in range(G)]
        recv_ptrs = ops._ptr_array([t.data_ptr() for t in recv])
        gidx_ptrs = ops._ptr_array([t.data_ptr() for t in gidx])
        if dedup:
            urank, ucount = ops.ep_unique(idx32, id_map, El, G)
            cnt_all = torch.stack([torch.cat([counts, ucount]), torch.zeros(E + G, dtype=torch.int32, device=cuda)]).contiguous()
            offs_local, dst_base, ret_rank, ret_row, u_base = ops.ep_plan_dedup(cnt_all, G, El, 0, cap)
            ops.ep_dispatch_dedup(x, perm, idx32, id_map, offsets, dst_base, urank, u_base, k, El, recv_ptrs, gidx_ptrs)
            sent = ucount.tolist()
        else:
            cnt_all = torch.stack([counts, torch.zeros(E, dtype=torch.int32, device=cuda)]).contiguous()
            offs_local, dst_base, ret_rank, ret_row = ops.ep_plan(cnt_all, G, El, 0, cap)
            ops.ep_dispatch(x, perm, idx32, id_map, offsets, dst_base, k, El, recv_ptrs)
            sent = [int(counts[d * El:(d + 1) * El].sum()) for d in range(G)]
        torch.cuda.synchronize(cuda)
        for d in range(G):
            assert torch.equal(recv[d][sent[d]:], canary[sent[d]:]), f"rows past the {sent[d]} live ones of rank {d} changed"
            assert not torch.equal(recv[d][:sent[d]], canary[:sent[d]])
    ops.check_status(cuda)
