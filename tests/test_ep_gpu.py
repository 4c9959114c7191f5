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
