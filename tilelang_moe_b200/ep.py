"""Expert parallelism for the routed MoE layer: one process per GPU, experts sharded, tokens
data-parallel, one exchange each way.

    rank r owns T/G tokens and E/G experts (placement table expert -> rank).
    route locally -> sort rows by (destination rank, local expert) -> all-gather of the histograms (checked)
    -> dispatch all-to-all-v of bf16 rows -> regroup expert-major -> up / down GEMMs
    -> combine all-to-all-v back -> weighted k-way sum on the owner.

The reference has no distributed code (its benchmark only shrinks the expert count,
benchmarks/benchmark_grouped_gemm.py:85-109); the contract here is that the sharded
layer returns what the single-GPU layer returns.  Received rows always sit in this
GPU's own memory before a kernel touches them.

The protocol is written against a small ops namespace (``tilelang_moe_b200.ops`` in
production) so that its host logic - placement, split sizes, the two permutations and
their inverses - can be exercised on CPU ranks over gloo with stand-in ops.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

# The exchange buffers are only ever written with plain peer stores: keep torch's symmetric memory from binding them
# to an NVLink multicast object (a rank that dies while its memory is bound to one can fault its peers' GPUs).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


# --------------------------------------------------------------------------- placement
def contiguous_placement(n_experts: int, world: int) -> List[int]:
    per = n_experts // world
    return [e // per for e in range(n_experts)]


def expert_cost(rows: float, tile_rows: int = 128, stream_tiles: float = 1.6) -> float:
    """Time an expert costs its GPU, in units of one 128-row tile through both GEMMs.

    An expert is tensor-core bound at ceil(rows/128) tiles, but never cheaper than streaming its weights from
    HBM once, which on B200 at H=7168, I=2048 takes as long as about 1.6 tiles (88 MB at 6.5 TB/s against
    11.3 GFLOP per tile at 1.3 PFLOP/s).  An expert without rows costs nothing: its weights are never touched.
    Balancing rows alone leaves the rank holding one huge expert plus many tiny ones ~17 % slower than the rest."""
    if rows <= 0:
        return 0.0
    return max(stream_tiles, float(-(-int(rows) // tile_rows)))


def tile_cost(rows: float, tile_rows: int = 128) -> float:
    """Row tiles an expert occupies in the grouped GEMMs.  A tile takes about the same time whether its expert is
    large (tensor bound) or owns that one tile only (its weights stream from HBM meanwhile), so tiles are what a rank's
    GEMM time is proportional to; an expert without rows costs nothing."""
    return 0.0 if rows <= 0 else float(-(-int(rows) // tile_rows))


def balanced_placement(load: Sequence[float], world: int, cost=None, max_per_rank: Optional[int] = None) -> List[int]:
    """Greedy longest-processing-time assignment: costliest expert first, to the least loaded rank that still has a
    free slot.  ``load`` is rows per expert; ``cost`` maps rows to time (default: rows themselves).  With
    ``max_per_rank`` = E/world (the default) every rank ends up with exactly E/world experts; a larger value lets the
    rank that holds a very popular expert take fewer of the others (see EPPlan's ``e_slots``)."""
    if cost is not None:
        load = [cost(v) for v in load]
    E = len(load)
    per = E // world if max_per_rank is None else max_per_rank
    if per * world < E:
        raise ValueError(f"{world} ranks with at most {per} experts each cannot hold {E} experts")
    order = sorted(range(E), key=lambda e: (-float(load[e]), e))
    tot = [0.0] * world
    cnt = [0] * world
    out = [0] * E
    for e in order:
        r = min((r for r in range(world) if cnt[r] < per), key=lambda r: (tot[r], r))
        out[e] = r
        tot[r] += float(load[e])
        cnt[r] += 1
    return out


@dataclass
class EPPlan:
    """Static sharding of E experts over `world` ranks.

    Every rank has ``e_local`` expert slots (``e_slots`` if given, else E / world); a rank may hold fewer experts than
    slots, and the unused slots simply never receive rows.  The kernels number experts by slot, rank-major:
    ``n_slots = world * e_local`` histogram bins, ``id_map[e] = rank * e_local + slot``; entries of ``id_map`` past the
    real experts are -1, which the histogram reports as an id out of range."""
    n_experts: int
    world: int
    expert_to_rank: List[int]
    e_slots: Optional[int] = None
    local_experts: List[List[int]] = field(init=False)   # per rank: global ids in local slot order
    id_map: List[int] = field(init=False)                 # global id -> rank * e_local + slot

    def __post_init__(self):
        E, G = self.n_experts, self.world
        if self.e_slots is None and E % G:
            raise ValueError(f"{E} experts do not split evenly over {G} ranks")
        self.e_local = E // G if self.e_slots is None else int(self.e_slots)
        self.n_slots = G * self.e_local
        self.local_experts = [[] for _ in range(G)]
        self.id_map = [-1] * max(E, self.n_slots)
        for e in range(E):
            r = self.expert_to_rank[e]
            self.id_map[e] = r * self.e_local + len(self.local_experts[r])
            self.local_experts[r].append(e)
        if any(len(l) > self.e_local for l in self.local_experts):
            raise ValueError(f"placement gives a rank more experts than its {self.e_local} slots")

    def padded_local_experts(self, rank: int) -> List[int]:
        """The rank's experts followed by repeats of its first one up to e_local entries: what to stack as the
        rank's weight tensors (the padding slots never receive rows, their weights are never read)."""
        mine = self.local_experts[rank]
        if not mine:
            raise ValueError(f"rank {rank} holds no expert")
        return mine + [mine[0]] * (self.e_local - len(mine))

    def imbalance(self, counts_per_expert: Sequence[float], cost=None) -> float:
        """max over ranks / mean over ranks of routed rows (or of cost(rows)) under this placement."""
        tot = [0.0] * self.world
        for e, c in enumerate(counts_per_expert):
            tot[self.expert_to_rank[e]] += float(c) if cost is None else cost(c)
        mean = sum(tot) / self.world
        return max(tot) / mean if mean > 0 else 1.0


# --------------------------------------------------------------------------- protocol
class EPProtocolError(RuntimeError):
    """The ranks' histograms do not describe a possible exchange (a damaged or mismatched counts table)."""


def check_counts_table(table: torch.Tensor, rows_per_rank: int) -> None:
    """table int [G,E] on the host: row g = rank g's rows per expert (placement order).  Every rank routes the same
    number of rows, so each row must be non-negative and sum to rows_per_rank; anything else would size the row
    exchange wrongly on some rank.  Every rank holds the same table and therefore raises, or passes, with the others."""
    t = table.long()
    if bool((t < 0).any()):
        g, e = [int(v[0]) for v in torch.nonzero(t < 0, as_tuple=True)]
        raise EPProtocolError(f"counts table: rank {g} reports {int(t[g, e])} rows for expert slot {e}")
    sums = t.sum(1)
    bad = torch.nonzero(sums != rows_per_rank).flatten()
    if bad.numel():
        g = int(bad[0])
        raise EPProtocolError(f"counts table: rank {g} reports {int(sums[g])} routed rows, {rows_per_rank} expected")


def ep_forward(x_local: torch.Tensor, logits_local: torch.Tensor, k: int, plan: EPPlan, id_map_dev: torch.Tensor,
               Wg: torch.Tensor, Wu: torch.Tensor, Wd: torch.Tensor, ops, group=None, bufs: Optional[dict] = None,
               timers: Optional[dict] = None, stage=None) -> torch.Tensor:
    """One expert-parallel forward of the routed layer for this rank's tokens.

    x_local bf16 [T_local,H]; logits_local fp32 [T_local,E]; Wg/Wu [E_local,I,H], Wd [E_local,H,I]
    for this rank's experts in slot order.  Returns out bf16 [T_local,H].
    """
    G, El, E = plan.world, plan.e_local, plan.n_slots
    Tl, H = x_local.shape
    n = Tl * k
    st = stage if stage is not None else (lambda name: _null)
    bufs = {} if bufs is None else bufs

    with st("route"):
        scores, idx32 = ops.topk_softmax(logits_local, k, mode="A", index_dtype=torch.int32)
        counts, offsets, perm, inv = ops.route_histogram(idx32, E, id_map=id_map_dev, workspace=bufs.get("hist_ws"))
        xs = ops.gather_rows(x_local, perm, div=k, out=bufs.get("xs"))
    with st("counts_a2a"):
        # every rank sees every rank's histogram (G x E ints) and checks all of it, so that a damaged table makes all
        # ranks raise together instead of leaving some of them waiting in the row exchange
        rank = dist.get_rank(group)
        table = torch.empty(G, E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(table.view(-1), counts.contiguous(), group=group)
        table_host = table.cpu()                                       # the one device-to-host wait of the layer
        check_counts_table(table_host, n)
        mine = table_host[:, rank * El:(rank + 1) * El]                # rows sent to this rank's experts, per source
        recv_counts = table[:, rank * El:(rank + 1) * El].contiguous().view(-1)
        in_splits = table_host[rank].view(G, El).sum(1).tolist()
        out_splits = mine.sum(1).tolist()
        n_recv = int(sum(out_splits))
    with st("dispatch_a2a"):
        recv = _take(bufs, "recv", n_recv, H, x_local)
        dist.all_to_all_single(recv, xs, out_splits, in_splits, group=group)
    with st("regroup"):
        offs_local, src_row = ops.ep_regroup(recv_counts.view(G, El), max(n_recv, 1))
        xl = ops.gather_rows(recv, src_row, out=_take(bufs, "xl", n_recv, H, x_local), n_rows=n_recv)
    with st("up_gemm"):
        act = ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, xl, Wg, offs_local, B2=Wu,
                                      out=_take(bufs, "act", n_recv, Wg.shape[1], x_local))
    with st("down_gemm"):
        yb = ops.grouped_gemm_sorted(ops.GEMM_PLAIN, act, Wd, offs_local, dst_rows=src_row,
                                     out=_take(bufs, "yb", n_recv, H, x_local))
    with st("combine_a2a"):
        yret = _take(bufs, "yret", n, H, x_local)
        dist.all_to_all_single(yret, yb, in_splits, out_splits, group=group)
    with st("combine"):
        out = ops.combine(yret, k, row_of=inv, scale=scores.reshape(-1), T=Tl, out=bufs.get("out"))
    if timers is not None:
        timers["_n_recv"] = n_recv
    return out


class PeerExchange:
    """Symmetric receive / return buffers of one expert-parallel group and the peers' addresses of them.

    recv [cap_rows, H]: rows other ranks dispatch to this rank's experts, expert-major.
    ret  [T_local*k, H]: expert outputs for this rank's routed entries, in its sorted order.
    cap_rows defaults to the global T*k (every routed row on one rank), so no overflow path exists.
    """

    def __init__(self, t_local: int, k: int, H: int, world: int, device: torch.device, group=None,
                 cap_rows: Optional[int] = None, overlap: bool = True, dedup: bool = False):
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops
        group = dist.group.WORLD if group is None else group
        self.cap = t_local * k * world if cap_rows is None else cap_rows
        self.recv = symm_mem.empty(self.cap, H, dtype=torch.bfloat16, device=device)
        self.ret = symm_mem.empty(t_local * k, H, dtype=torch.bfloat16, device=device)
        self.h_recv = symm_mem.rendezvous(self.recv, group)
        self.h_ret = symm_mem.rendezvous(self.ret, group)
        self.recv_ptrs = ops._ptr_array(list(self.h_recv.buffer_ptrs))
        self.ret_ptrs = ops._ptr_array(list(self.h_ret.buffer_ptrs))
        # phase barriers: this library's own flag barrier over peer memory, with a time limit (a peer that has died or
        # raised makes the wait run out and leave a status code instead of spinning for ever)
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)     # [4 channels][16 slots]
        self.flags.zero_()
        self.h_flags = symm_mem.rendezvous(self.flags, group)
        self.flag_ptrs = ops._ptr_array(list(self.h_flags.buffer_ptrs))
        self.rank = dist.get_rank(group)
        self.device = device
        self.epoch = [0, 0, 0, 0]
        self.barrier_timeout_us = int(os.environ.get("MOE_B200_EP_BARRIER_TIMEOUT_US", "2000000"))
        torch.cuda.synchronize(device)
        dist.barrier(group)                                                   # every rank's flags are zero before use
        # the ranks' histograms travel over peer memory too: two tables [world, E + world] (step parity)
        self.cnt_width = 0
        self.cnt_sym = None
        self.cnt_ptrs = None
        self.step_parity = 0
        self.group = group
        self.world = world
        self.plan_bufs = {}
        self.side = torch.cuda.Stream(device=device)
        self.overlap = overlap
        # de-duplicated dispatch: a token row goes to a rank once; the sources also write, for every routed entry, which
        # received row it is, and the destination's up GEMM gathers through that list (needs H % 64 == 0)
        self.dedup = dedup and H % 64 == 0
        if self.dedup:
            self.gidx = symm_mem.empty(self.cap, dtype=torch.int32, device=device)
            self.gidx.zero_()
            self.h_gidx = symm_mem.rendezvous(self.gidx, group)
            self.gidx_ptrs = ops._ptr_array(list(self.h_gidx.buffer_ptrs))
            self.uniq_bufs = {}


def _share_counts(px: "PeerExchange", ops, counts: torch.Tensor, extra: Optional[torch.Tensor]) -> torch.Tensor:
    """All ranks' (counts, extra) vectors as an int32 [world, width] table on this device: one kernel that stores this
    rank's row into every rank's table and runs the time-limited barrier (channel 3)."""
    import torch.distributed._symmetric_memory as symm_mem
    width = counts.numel() + (0 if extra is None else extra.numel())
    if px.cnt_sym is None or px.cnt_width != width:      # first step of a shape: collective allocation
        px.cnt_sym = symm_mem.empty(2 * px.world * width, dtype=torch.int32, device=px.device)
        px.cnt_sym.zero_()
        px.h_cnt = symm_mem.rendezvous(px.cnt_sym, px.group)
        px.cnt_ptrs = ops._ptr_array(list(px.h_cnt.buffer_ptrs))
        px.cnt_width = width
        torch.cuda.synchronize(px.device)
        dist.barrier(px.group)
    px.step_parity ^= 1
    px.epoch[3] += 1
    ops.ep_share_counts(counts, extra, px.cnt_ptrs, px.step_parity, px.flag_ptrs, px.rank, 3, px.epoch[3],
                        px.barrier_timeout_us)
    return px.cnt_sym.view(2, px.world, width)[px.step_parity]


def _barrier(px: "PeerExchange", ops, channel: int) -> None:
    """Enqueue barrier number epoch[channel] + 1 of `channel` on the current stream."""
    px.epoch[channel] += 1
    ops.ep_barrier(px.flag_ptrs, px.rank, channel, px.epoch[channel], px.device, px.barrier_timeout_us)


def ep_forward_peer(x_local: torch.Tensor, logits_local: torch.Tensor, k: int, plan: EPPlan, id_map_dev: torch.Tensor,
                    Wg: torch.Tensor, Wu: torch.Tensor, Wd: torch.Tensor, ops, px: PeerExchange, group=None,
                    bufs: Optional[dict] = None, timers: Optional[dict] = None, stage=None) -> torch.Tensor:
    """Expert-parallel forward with the exchange done by this library's own kernels over peer memory:
    the dispatch is a gather kernel that stores rows straight into the destination's expert-major
    buffer, the combine exchange is the down GEMM's epilogue storing into the owner's return buffer.
    The histograms are exchanged by a kernel over peer memory as well; three time-limited barriers per layer, no
    collective-library call and no host synchronisation."""
    G, El, E = plan.world, plan.e_local, plan.n_slots
    Tl, H = x_local.shape
    rank = dist.get_rank(group)
    st = stage if stage is not None else (lambda name: _null)
    bufs = {} if bufs is None else bufs
    with st("route"):
        scores, idx32 = ops.topk_softmax(logits_local, k, mode="A", index_dtype=torch.int32)
        if px.dedup:   # numbering the tokens per destination needs the top-k ids only: it runs beside the histogram kernels
            cur = torch.cuda.current_stream(x_local.device)
            fork = torch.cuda.Event()
            fork.record(cur)
            with torch.cuda.stream(px.side):
                px.side.wait_event(fork)
                urank, ucount = ops.ep_unique(idx32, id_map_dev, El, G, out=px.uniq_bufs)
                numbered = torch.cuda.Event()
                numbered.record(px.side)
        counts, offsets, perm, inv = ops.route_histogram(idx32, E, id_map=id_map_dev, workspace=bufs.get("hist_ws"))
        if px.dedup:
            cur.wait_event(numbered)
    with st("counts_allgather"):
        if px.dedup:
            cnt_all = _share_counts(px, ops, counts, ucount)
            offs_local, dst_base, ret_rank, ret_row, u_base = ops.ep_plan_dedup(cnt_all, G, El, rank, px.cap,
                                                                                out=px.plan_bufs)
        else:
            cnt_all = _share_counts(px, ops, counts, None)
            offs_local, dst_base, ret_rank, ret_row = ops.ep_plan(cnt_all, G, El, rank, px.cap, out=px.plan_bufs)
    I = Wg.shape[1]
    act = _take(bufs, "act", px.cap, I, x_local)
    split = El // 2 if (px.overlap and El >= 2 and not px.dedup) else 0
    if px.dedup:
        with st("dispatch"):
            ops.ep_dispatch_dedup(x_local, perm, idx32, id_map_dev, offsets, dst_base, urank, u_base, k, El,
                                  px.recv_ptrs, px.gidx_ptrs)
        with st("dispatch_barrier"):
            _barrier(px, ops, 0)
        with st("up_gemm"):   # expert-major row q is received row gidx[q]
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, px.recv, Wg, offs_local, B2=Wu, out=act, gather=px.gidx,
                                    gather_div=1, expected_rows=Tl * k)
        with st("down_gemm"):
            ops.grouped_gemm_peer_scatter(act, Wd, offs_local, ret_rank, ret_row, px.ret_ptrs, H, expected_rows=Tl * k)
    elif split == 0:
        with st("dispatch"):
            ops.ep_dispatch(x_local, perm, idx32, id_map_dev, offsets, dst_base, k, El, px.recv_ptrs)
        with st("dispatch_barrier"):
            _barrier(px, ops, 0)
        with st("up_gemm"):
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, px.recv, Wg, offs_local, B2=Wu, out=act, expected_rows=Tl * k)
        with st("down_gemm"):
            ops.grouped_gemm_peer_scatter(act, Wd, offs_local, ret_rank, ret_row, px.ret_ptrs, H, expected_rows=Tl * k)
    else:
        # Two groups of local experts.  The rows of the second group travel on a side stream while the GEMMs of the
        # first group run: the receive buffer is expert-major, so each group owns a contiguous range of it and the
        # GEMM of a group is the same kernel on a sub-range of the offset table and of the weights.
        cur = torch.cuda.current_stream(x_local.device)
        with st("dispatch"):
            ops.ep_dispatch(x_local, perm, idx32, id_map_dev, offsets, dst_base, k, El, px.recv_ptrs, 0, split)
        with st("dispatch_barrier"):
            _barrier(px, ops, 0)
            fork = torch.cuda.Event()
            fork.record(cur)
        with torch.cuda.stream(px.side):
            px.side.wait_event(fork)   # after the first group has landed everywhere: the links are free again
            ops.ep_dispatch(x_local, perm, idx32, id_map_dev, offsets, dst_base, k, El, px.recv_ptrs, split, El)
            _barrier(px, ops, 2)
            second_ready = torch.cuda.Event()
            second_ready.record(px.side)
        half = Tl * k // 2
        with st("up_gemm"):
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, px.recv, Wg[:split], offs_local[:split + 1], B2=Wu[:split], out=act,
                                    expected_rows=half)
        with st("down_gemm"):
            ops.grouped_gemm_peer_scatter(act, Wd[:split], offs_local[:split + 1], ret_rank, ret_row, px.ret_ptrs, H,
                                          expected_rows=half)
        with st("second_wait"):
            cur.wait_event(second_ready)
        with st("up_gemm_2"):
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, px.recv, Wg[split:], offs_local[split:], B2=Wu[split:], out=act,
                                    expected_rows=half)
        with st("down_gemm_2"):
            ops.grouped_gemm_peer_scatter(act, Wd[split:], offs_local[split:], ret_rank, ret_row, px.ret_ptrs, H,
                                          expected_rows=half)
    with st("combine_barrier"):
        _barrier(px, ops, 1)
    with st("combine"):
        out = ops.combine(px.ret, k, row_of=inv, scale=scores.reshape(-1), T=Tl, out=bufs.get("out"))
    return out


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_null = _Null()


def _take(bufs: dict, name: str, rows: int, cols: int, like: torch.Tensor) -> torch.Tensor:
    """A [rows, cols] view of a persistent buffer (grown on demand), or a fresh tensor."""
    buf = bufs.get(name)
    if buf is None or buf.shape[0] < rows or buf.shape[1] != cols:
        buf = torch.empty(max(rows, 1), cols, dtype=like.dtype, device=like.device)
        bufs[name] = buf
    return buf[:rows]


# --------------------------------------------------------------------------- bench runner
class EPRunner:
    """Holds one rank's shard (weights of its experts, buffers) for the benchmark workload."""

    def __init__(self, cfg: dict, rank: int, world: int, device: torch.device, make_weights: Callable,
                 placement: str = "balanced", calib_seed: int = 1, exchange: str = "peer_dedup"):
        from . import _lib, ops
        from .layer import _Stage
        self.ops, self._Stage = ops, _Stage
        self.cfg, self.rank, self.world, self.dev = cfg, rank, world, device
        T, E, k = cfg["T"], cfg["E"], cfg["k"]
        if T % world:
            raise ValueError("tokens must split evenly over the ranks")
        self.Tl = T // world
        # placement from the expert loads of a calibration batch with the same popularity law
        # (a different noise draw than the timed batch): what a serving system knows in advance
        load = self._calibration_load(cfg, calib_seed)
        e_slots = None
        if placement == "balanced":
            # Exactly E / world experts per rank, rows balanced - unless that leaves one rank clearly more row tiles
            # than the others (a very popular expert plus its full share of the rest: at 8 ranks 87 tiles against 78-82).
            # Then ranks may hold up to a quarter more experts than E / world and row tiles are balanced instead, so
            # the rank of the popular expert takes fewer of the others.  Measured: 8 ranks 1.35 -> 1.14 ms per step;
            # at 4 ranks, where the equal-count placement is already even, it is the faster one (1.93 against 2.02 ms).
            e2r = balanced_placement(load, world)
            spare = E // world + max(1, E // world // 4)
            alt = balanced_placement(load, world, cost=tile_cost, max_per_rank=spare)

            def fullest(table):
                tot = [0.0] * world
                for e, r in enumerate(table):
                    tot[r] += tile_cost(load[e])
                return max(tot)
            if fullest(alt) < 0.97 * fullest(e2r):
                e2r, e_slots = alt, spare
        elif placement == "tiles":       # by row tiles with spare expert slots, whatever the equal-count placement gives
            e_slots = E // world + max(1, E // world // 4)
            e2r = balanced_placement(load, world, cost=tile_cost, max_per_rank=e_slots)
        elif placement == "rows":        # by routed rows, exactly E / world experts per rank
            e2r = balanced_placement(load, world)
        elif placement == "time":        # by modelled time, exactly E / world experts per rank
            e2r = balanced_placement(load, world, cost=expert_cost)
        else:
            e2r = contiguous_placement(E, world)
        self.plan = EPPlan(E, world, e2r, e_slots)
        if e_slots is not None:          # no more slots than the fullest rank uses
            self.plan = EPPlan(E, world, e2r, max(len(l) for l in self.plan.local_experts))
        self.id_map_dev = torch.tensor(self.plan.id_map, dtype=torch.int32, device=device)
        self.Wg, self.Wu, self.Wd = make_weights(cfg, device, experts=self.plan.padded_local_experts(rank))
        need = _lib.load().moe_route_histogram_workspace(self.Tl * k, self.plan.n_slots)
        self.bufs = {"hist_ws": torch.empty(max(need, 4), dtype=torch.uint8, device=device)}
        self.imbalance = None
        self.exchange = exchange
        import os
        # Dispatching the second half of the local experts under the first half's GEMMs pays only where the dispatch
        # is a large share of the step: measured +2.5 % at 8 GPUs, nothing at 4, -3 % at 2 (the copy slows the GEMM).
        overlap = os.environ.get("MOE_B200_EP_OVERLAP", "1" if world >= 8 else "0") != "0"
        # "peer": every routed row travels; "peer_dedup": a token row travels to a rank once and the up GEMM gathers
        dedup = exchange == "peer_dedup"
        self.px = (PeerExchange(self.Tl, k, cfg["H"], world, device, overlap=overlap and not dedup, dedup=dedup)
                   if exchange in ("peer", "peer_dedup") else None)

    def _routed_counts(self, logits_cpu: torch.Tensor) -> List[int]:
        """Rows per expert when `logits_cpu` is routed top-k (through the router and histogram kernels)."""
        _, idx32 = self.ops.topk_softmax(logits_cpu.to(self.dev), self.cfg["k"], mode="A", index_dtype=torch.int32)
        counts, _, _, _ = self.ops.route_histogram(idx32, self.cfg["E"], want_perm=False, want_inv=False)
        return counts.cpu().tolist()

    def _calibration_load(self, cfg, seed):
        from .inputs import zipf_logits
        return self._routed_counts(zipf_logits(cfg["T"], cfg["E"], 1.1, seed=0, noise_seed=seed + 1000))

    def forward(self, x_local, logits_local, timers=None):
        stage = (lambda name: self._Stage(timers, name)) if timers is not None else None
        if self.px is not None:
            return ep_forward_peer(x_local, logits_local, self.cfg["k"], self.plan, self.id_map_dev, self.Wg, self.Wu,
                                   self.Wd, self.ops, self.px, bufs=self.bufs, timers=timers, stage=stage)
        return ep_forward(x_local, logits_local, self.cfg["k"], self.plan, self.id_map_dev, self.Wg, self.Wu,
                          self.Wd, self.ops, bufs=self.bufs, timers=timers, stage=stage)

    def bench_closures(self, x_cpu, logits_cpu):
        """(step, step_e2e, launches per step, h2d bytes, d2h bytes) for this rank's share of the batch."""
        Tl, r, dev = self.Tl, self.rank, self.dev
        rc = self._routed_counts(logits_cpu)
        self.imbalance = self.plan.imbalance(rc)
        self.cost_imbalance = self.plan.imbalance(rc, cost=tile_cost)
        naive = EPPlan(self.plan.n_experts, self.world, contiguous_placement(self.plan.n_experts, self.world))
        self.contiguous_imbalance = (naive.imbalance(rc), naive.imbalance(rc, cost=tile_cost))   # experts in id order
        self.experts_per_rank = [len(l) for l in self.plan.local_experts]
        x_l = x_cpu[r * Tl:(r + 1) * Tl].contiguous()
        lg_l = logits_cpu[r * Tl:(r + 1) * Tl].contiguous()
        x, lg = x_l.to(dev), lg_l.to(dev)
        x_pin, lg_pin = x_l.pin_memory(), lg_l.pin_memory()
        out_pin = torch.empty(Tl, x_l.shape[1], dtype=torch.bfloat16).pin_memory()
        x_dev, lg_dev = torch.empty_like(x), torch.empty_like(lg)

        def step(timers=None):
            return self.forward(x, lg, timers=timers)

        bufs = self.bufs

        def compute(xd, lgd, outd):
            bufs["out"] = outd
            self.forward(xd, lgd)

        from .pipeline import HostPipeline
        pipe = HostPipeline(dev, [x_pin, lg_pin], (Tl, x_l.shape[1]), torch.bfloat16, compute, depth=3)   # uploads run two steps ahead

        def step_e2e(n=1):
            pipe.run(n)
            bufs.pop("out", None)

        # kernels of this library per step: topk, 3 x histogram, gather, regroup, gather, up, down, combine
        h2d = (x_pin.numel() * 2 + lg_pin.numel() * 4) * self.world
        d2h = out_pin.numel() * 2 * self.world
        # peer exchange: topk, 3 x histogram, [unique,] histogram exchange, plan, dispatch, barrier, up, down (+ scatter),
        # barrier, combine; NCCL variant: topk, 3 x histogram, gather, regroup, gather, up, down, combine
        return step, step_e2e, ((13 if self.px.dedup else 12) if self.px is not None else 10), h2d, d2h
