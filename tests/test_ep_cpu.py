"""Expert-parallel host protocol on two (and four) gloo ranks with CPU stand-in ops: the sharded layer
must return what the single-process oracle returns, for contiguous and load-balanced placements."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from tilelang_moe_b200 import ep, inputs


def test_balanced_placement_properties():
    load = [1000, 10, 10, 10, 900, 20, 20, 20]
    e2r = ep.balanced_placement(load, 2)
    assert sorted(e2r.count(r) for r in range(2)) == [4, 4]
    assert e2r[0] != e2r[4]                       # the two heavy experts are split up
    plan = ep.EPPlan(8, 2, e2r)
    assert sorted(plan.id_map) == list(range(8))
    assert plan.imbalance(load) < ep.EPPlan(8, 2, ep.contiguous_placement(8, 2)).imbalance([1000, 900, 10, 10, 10, 20, 20, 20])
    for r in range(2):
        for slot, e in enumerate(plan.local_experts[r]):
            assert plan.id_map[e] == r * 4 + slot
    with pytest.raises(ValueError):
        ep.EPPlan(8, 2, [0] * 8)


def test_uneven_placement_gives_the_rank_of_a_hot_expert_fewer_experts():
    load = [4000, 100, 100, 100, 100, 100, 100, 100]              # expert 0: 32 row tiles, the others 1 each
    e2r = ep.balanced_placement(load, 2, cost=ep.tile_cost, max_per_rank=7)
    plan = ep.EPPlan(8, 2, e2r, 7)
    hot = e2r[0]
    assert len(plan.local_experts[hot]) == 1 and len(plan.local_experts[1 - hot]) == 7
    assert plan.e_local == 7 and plan.n_slots == 14 and len(plan.id_map) == 14
    assert sorted(v for v in plan.id_map if v >= 0) == sorted([hot * 7] + [(1 - hot) * 7 + j for j in range(7)])
    assert plan.id_map[8:] == [-1] * 6                             # ids past the real experts map to no slot
    assert plan.padded_local_experts(hot) == [0] * 7
    with pytest.raises(ValueError):
        ep.balanced_placement(load, 2, max_per_rank=3)             # 2 x 3 slots cannot hold 8 experts
    with pytest.raises(ValueError):
        ep.EPPlan(8, 2, [0] * 8, 7)                                # more experts on a rank than it has slots
    # every rank the same count when no slack is given, as before
    assert sorted(ep.balanced_placement(load, 2).count(r) for r in range(2)) == [4, 4]


def test_zipf_placement_reduces_imbalance():
    lg = inputs.zipf_logits(4096, 256, 1.1, seed=0)
    _, idx = O.topk_softmax(lg, 8, "A")
    counts = O.route_histogram(idx, 256)[0].tolist()
    calib = inputs.zipf_logits(4096, 256, 1.1, seed=0, noise_seed=77)
    ccounts = O.route_histogram(O.topk_softmax(calib, 8, "A")[1], 256)[0].tolist()
    bal = ep.EPPlan(256, 8, ep.balanced_placement(ccounts, 8)).imbalance(counts)
    con = ep.EPPlan(256, 8, ep.contiguous_placement(256, 8)).imbalance(counts)
    assert bal < 1.15 and bal < con


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, placement, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_ops
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, H, I, E, k = 64, 32, 16, 8, 3
        g = torch.Generator().manual_seed(0)
        x = torch.randn(T, H, generator=g)
        Wg = torch.randn(E, I, H, generator=g) * 0.2
        Wu = torch.randn(E, I, H, generator=g) * 0.2
        Wd = torch.randn(E, H, I, generator=g) * 0.2
        logits = inputs.zipf_logits(T, E, 1.1, seed=1)
        _, idx = O.topk_softmax(logits, k, "A")
        load = O.route_histogram(idx, E)[0].tolist()
        if placement == "tiles":     # by row tiles (of 8 rows here), a rank may hold more experts than E / world
            cost = lambda rows: ep.tile_cost(rows, 8)
            skewed = [v * 8 if v == max(load) else v for v in load]     # a calibration batch with one very popular expert
            e2r = ep.balanced_placement(skewed, world, cost=cost, max_per_rank=E // world + 2)
            plan = ep.EPPlan(E, world, e2r, E // world + 2)
            assert len({len(l) for l in plan.local_experts}) > 1, "the case is meant to be uneven"
        else:
            e2r = ep.balanced_placement(load, world) if placement == "balanced" else ep.contiguous_placement(E, world)
            plan = ep.EPPlan(E, world, e2r)
        mine = plan.padded_local_experts(rank)
        Tl = T // world
        out = ep.ep_forward(x[rank * Tl:(rank + 1) * Tl], logits[rank * Tl:(rank + 1) * Tl], k, plan,
                            torch.tensor(plan.id_map, dtype=torch.int32), Wg[mine], Wu[mine], Wd[mine], cpu_ops)
        ref = O.fusedmoe(x, None, None, None, None, Wg, Wu, Wd, k, logits=logits)[rank * Tl:(rank + 1) * Tl]
        q.put((rank, float((out - ref).abs().max()), None))
    except Exception as e:  # surfaced in the parent
        q.put((rank, None, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,placement", [(2, "contiguous"), (2, "balanced"), (4, "balanced"), (2, "tiles")])
def test_ep_protocol_matches_single_process(world, placement):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, placement, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, err, exc in res:
        assert exc is None, f"rank {rank}: {exc}"
        assert err < 1e-4, f"rank {rank}: max abs error {err}"


def _run_ranks(target, world, *args, timeout=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, *args, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = dict(q.get(timeout=timeout) for _ in range(world))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    return res


def _small_case(rank, world):
    T, H, I, E, k = 64, 32, 16, 8, 3
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, H, generator=g)
    Wg = torch.randn(E, I, H, generator=g) * 0.2
    Wu = torch.randn(E, I, H, generator=g) * 0.2
    Wd = torch.randn(E, H, I, generator=g) * 0.2
    logits = inputs.zipf_logits(T, E, 1.1, seed=1)
    plan = ep.EPPlan(E, world, ep.contiguous_placement(E, world))
    mine = plan.padded_local_experts(rank)
    Tl = T // world
    sl = slice(rank * Tl, (rank + 1) * Tl)
    return (x[sl], logits[sl], k, plan, torch.tensor(plan.id_map, dtype=torch.int32), Wg[mine], Wu[mine], Wd[mine])


def _worker_damaged_counts(rank, world, port, q):
    """Rank 1's histogram is damaged after routing: every rank must raise EPProtocolError, none may wait."""
    import sys
    import types
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_ops
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    try:
        ops = types.SimpleNamespace(**{n: getattr(cpu_ops, n) for n in dir(cpu_ops) if not n.startswith("_")})
        if rank == 1:
            def damaged(*a, **kw):
                counts, offsets, perm, inv = cpu_ops.route_histogram(*a, **kw)
                counts = counts.clone()
                counts[2] += 5
                return counts, offsets, perm, inv
            ops.route_histogram = damaged
        try:
            ep.ep_forward(*_small_case(rank, world), ops)
            q.put((rank, "returned"))
        except ep.EPProtocolError as e:
            q.put((rank, "protocol error: " + str(e)))
        except Exception as e:
            q.put((rank, "other: " + repr(e)))
    finally:
        dist.destroy_process_group()


def test_a_damaged_counts_table_makes_every_rank_raise():
    res = _run_ranks(_worker_damaged_counts, 2)
    for rank in range(2):
        assert res[rank].startswith("protocol error"), res
        assert "rank 1 reports 101 routed rows, 96 expected" in res[rank], res


def _put_and_flush(q, item):
    q.put(item)
    q.close()
    q.join_thread()      # os._exit would drop what the queue's feeder thread has not written yet


def _worker_rank_leaves(rank, world, port, q):
    """Both ranks run one step; rank 1 then leaves (between steps, nothing in flight).  Rank 0's next step must end
    with an error within the process group's time limit instead of waiting for good."""
    import sys
    import time
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_ops
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    case = _small_case(rank, world)
    ep.ep_forward(*case, cpu_ops)                    # step 1: everyone is there
    if rank == 1:
        _put_and_flush(q, (rank, "left"))
        os._exit(0)                                  # gone without a word
    t0 = time.time()
    try:
        ep.ep_forward(*case, cpu_ops)                # step 2: the peer never joins
        _put_and_flush(q, (rank, "returned"))
    except Exception as e:
        _put_and_flush(q, (rank, f"raised after {time.time() - t0:.1f} s: {type(e).__name__}"))
    os._exit(0)                                      # the group cannot be torn down in order any more


def test_a_rank_that_leaves_between_steps_ends_the_next_collective_with_an_error():
    res = _run_ranks(_worker_rank_leaves, 2, timeout=90)
    assert res[1] == "left"
    assert res[0].startswith("raised after"), res
    assert float(res[0].split()[2]) < 60.0, res


def test_check_counts_table_accepts_and_rejects():
    ok = torch.tensor([[3, 0, 5], [1, 7, 0]], dtype=torch.int32)
    ep.check_counts_table(ok, 8)
    with pytest.raises(ep.EPProtocolError, match="rank 1 reports 9 routed rows"):
        ep.check_counts_table(torch.tensor([[3, 0, 5], [1, 8, 0]]), 8)
    with pytest.raises(ep.EPProtocolError, match="reports -1 rows for expert slot 1"):
        ep.check_counts_table(torch.tensor([[3, -1, 6], [1, 7, 0]]), 8)


def test_dedup_dispatch_tables_model():
    """The arithmetic of the de-duplicated dispatch (moe_ep_unique / moe_ep_plan_dedup / moe_ep_dispatch_dedup), restated
    in numpy for all ranks in one process: a token row is stored once per destination rank, and the index list the
    sources write lets every destination find, for each expert-major position, the row of the right token."""
    import numpy as np
    rng = np.random.default_rng(0)
    G, El, Tl, k = 4, 3, 37, 5
    E = G * El
    e2r = ep.balanced_placement(list(rng.integers(1, 50, E)), G)
    plan = ep.EPPlan(E, G, e2r)
    id_map = np.array(plan.id_map)
    idx = np.stack([np.stack([rng.permutation(E)[:k] for _ in range(Tl)]) for _ in range(G)])     # [G, Tl, k] global ids
    # per source: histogram in virtual-expert order, stable permutation
    cnt = np.zeros((G, E + G), dtype=np.int64)
    perm, offs, urank = [], [], []
    for s in range(G):
        v = id_map[idx[s]].reshape(-1)
        perm.append(np.argsort(v, kind="stable"))
        c = np.bincount(v, minlength=E)
        cnt[s, :E] = c
        offs.append(np.concatenate([[0], np.cumsum(c)]))
        flags = np.zeros((Tl, G), dtype=bool)
        for t in range(Tl):
            flags[t, id_map[idx[s, t]] // El] = True
        u = np.where(flags, np.cumsum(flags, axis=0) - 1, -1)                                  # moe_ep_unique
        urank.append(u)
        cnt[s, E:] = flags.sum(0)
    # destination-side tables (moe_ep_plan_dedup on every rank)
    cap = Tl * k * G
    recv = [dict() for _ in range(G)]
    gidx = [np.full(cap, -7, dtype=np.int64) for _ in range(G)]
    dbase = np.zeros(E, dtype=np.int64)
    for d in range(G):
        run = 0
        for j in range(El):
            dbase[d * El + j] = run
            run += cnt[:, d * El + j].sum()
    for s in range(G):                                                                        # source side
        dst_base = np.array([dbase[v] + cnt[:s, v].sum() for v in range(E)])
        u_base = np.array([cnt[:s, E + d].sum() for d in range(G)])
        for t in range(Tl):
            for d in range(G):
                if urank[s][t, d] >= 0:
                    row = u_base[d] + urank[s][t, d]
                    assert row not in recv[d], "two tokens share a receive row"
                    recv[d][row] = (s, t)
        for p in range(Tl * k):
            f = perm[s][p]
            v = id_map[idx[s].reshape(-1)[f]]
            d, t = v // El, f // k
            gidx[d][dst_base[v] + (p - offs[s][v])] = u_base[d] + urank[s][t, d]
    for d in range(G):                                                                        # what the up GEMM of d gathers
        assert sorted(recv[d]) == list(range(len(recv[d]))) and len(recv[d]) == cnt[:, E + d].sum() <= Tl * G
        q = 0
        for j in range(El):
            v = d * El + j
            for s in range(G):
                for i in range(cnt[s, v]):
                    t = perm[s][offs[s][v] + i] // k
                    assert recv[d][gidx[d][q]] == (s, t)
                    q += 1
        assert (gidx[d][q:] == -7).all()
