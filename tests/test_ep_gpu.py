"""Expert parallelism on real GPUs (needs >= 2): each rank's slice of the sharded layer against the
single-process fp32 oracle.  NVLS is switched off so that a failing rank cannot disturb its peers."""
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
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
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
        e2r = ep.balanced_placement(load, world) if placement == "balanced" else ep.contiguous_placement(E, world)
        plan = ep.EPPlan(E, world, e2r)
        mine = plan.local_experts[rank]
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
                                                ("balanced", "peer_dedup")])
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
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, err, exc in res:
        assert exc is None, f"rank {rank}: {exc}"
        assert ok, f"rank {rank}: max abs error {err}"


@pytest.mark.parametrize("tile_rows,H,I", [("128", 128, 64), ("pair", 256, 128)])
@pytest.mark.parametrize("G,dedup", [(4, True), (8, True), (8, False)])
def test_peer_exchange_kernels_with_emulated_ranks_on_one_gpu(cuda, lib, G, dedup, tile_rows, H, I, monkeypatch):
    """The peer-exchange kernels for G ranks run one after another on a single GPU: every "rank" has its own receive,
    index and return buffers on that device, the all-gather is a torch.stack, and no barrier is needed because the
    phases are issued in order on one stream.  Checks the whole path (unique / plan / dispatch / gathered up GEMM /
    scattering down GEMM / combine) against the oracle for 4 and 8 ranks without needing that many GPUs."""
    from oracle import moe_oracle as O
    from tilelang_moe_b200 import ep, inputs, ops
    monkeypatch.setenv("MOE_B200_GEMM_TILE_ROWS", tile_rows)   # single-CTA kernel, or the CTA-pair kernel's gather / peer epilogue
    dev = cuda
    El, k, Tl = 4, 4, 96
    E, T = G * El, G * 96
    g = torch.Generator().manual_seed(G)
    x = torch.randn(T, H, generator=g).bfloat16()
    Wg = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    Wu = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    Wd = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    logits = inputs.zipf_logits(T, E, 1.1, seed=G)
    _, idx = O.topk_softmax(logits, k, "A")
    plan = ep.EPPlan(E, G, ep.balanced_placement(O.route_histogram(idx, E)[0].tolist(), G))
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
        counts, offsets, perm, inv = ops.route_histogram(idx32, E, id_map=id_map)
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
        mine = plan.local_experts[d]
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
        sent = int(cnt_all[:, E:].sum())
        assert sent <= T * min(k, G) and sent < T * k
