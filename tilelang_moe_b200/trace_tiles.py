"""Per-tile timeline of the 128-row grouped GEMM on the routed-layer workload of the benchmark.

    python -m tilelang_moe_b200.build --trace          # libmoe_b200_trace.so (-DMOE_GEMM_TRACE)
    python -m tilelang_moe_b200.trace_tiles [--which up|down] [--T 8192 --H 7168 --I 2048 --E 256 --k 8]

The trace build stamps every tile with %globaltimer when the MMA warp starts it, when its accumulator is
complete and when the epilogue has stored it, and every CTA with clock64 / %globaltimer at start and end
(csrc/gemm_sm100.cu, MOE_GEMM_TRACE).  Printed: the launch time by CUDA events, the effective SM clock during the
launch, the tensor-pipe time one tile needs at that clock, tile times by size class of the tile's expert, the
epilogue time and the spread of CTA end times.  Routing is Zipf(1.1) (tilelang_moe_b200.inputs.zipf_logits, seed 0),
weights and activations are random: the timeline depends on shapes and routing only.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

MAX_TILES, MAX_CTAS = 32768, 256


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", choices=["up", "down"], default="up")
    for name, dflt in (("T", 8192), ("H", 7168), ("I", 2048), ("E", 256), ("k", 8)):
        ap.add_argument("--" + name, type=int, default=dflt)
    ap.add_argument("--reps", type=int, default=7)
    args = ap.parse_args()

    from . import build as _build
    if not _build.TRACE_LIB.exists():
        print(f"{_build.TRACE_LIB} is missing: run `python -m tilelang_moe_b200.build --trace` first", file=sys.stderr)
        return 2
    os.environ["MOE_B200_LIBRARY"] = str(_build.TRACE_LIB)
    import numpy as np
    import torch
    from . import _lib, inputs, ops

    T, H, I, E, k = args.T, args.H, args.I, args.E, args.k
    dev = torch.device("cuda", 0)
    lg = inputs.zipf_logits(T, E, 1.1, seed=0).to(dev)
    _, idx = ops.topk_softmax(lg, k)
    counts, offsets, perm, _ = ops.route_histogram(idx, E, want_inv=False)
    n = T * k
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    act = torch.empty(n, I, device=dev, dtype=torch.bfloat16)
    if args.which == "up":
        Wg = torch.randn(E, I, H, device=dev, dtype=torch.bfloat16) * 0.02
        Wu = torch.randn(E, I, H, device=dev, dtype=torch.bfloat16) * 0.02
        n_tiles_n, k_blocks, acc_cols = I // 128, H // 64, 256

        def run():
            ops.grouped_gemm_sorted(ops.GEMM_SILU_GATE, x, Wg, offsets, B2=Wu, out=act, gather=perm, gather_div=k)
    else:
        act.normal_()
        Wd = torch.randn(E, H, I, device=dev, dtype=torch.bfloat16) * 0.02
        yk = torch.empty(n, H, device=dev, dtype=torch.bfloat16)
        n_tiles_n, k_blocks, acc_cols = H // 256, I // 64, 256

        def run():
            ops.grouped_gemm_sorted(ops.GEMM_PLAIN, act, Wd, offsets, dst_rows=perm, out=yk)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    ms = []
    for _ in range(args.reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); run(); b.record(); torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    ops.check_status(dev)

    tile_ns = np.zeros((3, MAX_TILES), dtype=np.uint64)
    tile_cta = np.zeros(MAX_TILES, dtype=np.int32)
    cta_clk = np.zeros((MAX_CTAS, 4), dtype=np.int64)
    lib = _lib.load()
    lib.moe_gemm_trace_read.restype = ctypes.c_int
    rc = lib.moe_gemm_trace_read(tile_ns.ctypes.data_as(ctypes.c_void_p), tile_cta.ctypes.data_as(ctypes.c_void_p),
                                 cta_clk.ctypes.data_as(ctypes.c_void_p))
    _lib.check(rc, "moe_gemm_trace_read")

    cnt = counts.cpu().numpy()
    m_tiles = (cnt + 127) // 128
    n_tiles = int(m_tiles.sum()) * n_tiles_n
    if n_tiles > MAX_TILES:
        print(f"{n_tiles} tiles exceed the trace capacity of {MAX_TILES}", file=sys.stderr)
        return 2
    ctas = int(min(n_tiles, torch.cuda.get_device_properties(dev).multi_processor_count))
    st, ready, done = (tile_ns[i, :n_tiles].astype(np.int64) for i in range(3))
    t0 = st.min()
    first = np.concatenate([[0], np.cumsum(m_tiles)]) * n_tiles_n
    rows_of_tile = cnt[np.searchsorted(first, np.arange(n_tiles), side="right") - 1]
    mhz = (cta_clk[:ctas, 2] - cta_clk[:ctas, 0]) / ((cta_clk[:ctas, 3] - cta_clk[:ctas, 1]) / 1e3)
    clock = float(np.median(mhz))
    pipe_us = k_blocks * 4 * (128 * acc_cols / 256) / clock
    ends = np.array([ready[tile_cta[:n_tiles] == c].max() - t0 for c in range(ctas)]) / 1e3
    print(f"workload: T={T} H={H} I={I} E={E} k={k}  rows={int(cnt.sum())}  row tiles={int(m_tiles.sum())}  "
          f"tiles={n_tiles}  ({args.which} GEMM)")
    print(f"launch time (CUDA events): median {sorted(ms)[len(ms) // 2]:.3f} ms, min {min(ms):.3f}")
    print(f"effective SM clock during the traced launch: {clock:.0f} MHz (min {mhz.min():.0f}, max {mhz.max():.0f})")
    print(f"tensor-pipe time of one tile at that clock: {pipe_us:.1f} us")
    dur = (ready - st) / 1e3
    for lo, hi in ((0, 32), (32, 128), (128, 256), (256, 1024), (1024, 1 << 30)):
        m = (rows_of_tile >= lo) & (rows_of_tile < hi)
        if m.any():
            print(f"  experts with {lo:5d} <= rows < {hi if hi < 1 << 30 else 'inf':>5}: {int(m.sum()):6d} tiles, "
                  f"tile time mean {dur[m].mean():6.1f}  p10 {np.percentile(dur[m], 10):6.1f}  "
                  f"p90 {np.percentile(dur[m], 90):6.1f} us")
    epi = (done - ready) / 1e3
    print(f"epilogue of one tile (first epilogue warp): median {np.median(epi):.1f} us, p90 {np.percentile(epi, 90):.1f} us")
    print(f"CTA end times: min {ends.min():.0f}  mean {ends.mean():.0f}  max {ends.max():.0f} us  "
          f"(tail {100 * (ends.max() / ends.mean() - 1):.1f} %)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
