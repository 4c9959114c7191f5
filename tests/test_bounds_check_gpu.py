"""The index-checked build of the library (-DMOE_BOUNDS_CHECK, libmoe_b200_check.so): an index that points outside
its buffer is not followed and is reported; nothing faults.  Each case runs in a child process, because the library a
process uses is chosen when it is first loaded (MOE_B200_LIBRARY)."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECK_LIB = os.path.join(ROOT, "tilelang_moe_b200", "libmoe_b200_check.so")


def _run(body: str, check: bool = True) -> str:
    if check and not os.path.exists(CHECK_LIB):
        pytest.fail(f"{CHECK_LIB} is missing: build it with `python -m tilelang_moe_b200.build --check`")
    env = dict(os.environ)
    if check:
        env["MOE_B200_LIBRARY"] = CHECK_LIB
    else:
        env.pop("MOE_B200_LIBRARY", None)
    prologue = textwrap.dedent(f"""
        import sys, torch
        sys.path.insert(0, {ROOT!r})
        from tilelang_moe_b200 import ops
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        g = torch.Generator().manual_seed(3)
    """)
    r = subprocess.run([sys.executable, "-c", prologue + textwrap.dedent(body)], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


SCATTER = """
    E, H, I, rows = 4, 128, 64, 300
    idx = torch.randint(0, E, (rows, 1), generator=g, dtype=torch.int32).to(dev)
    counts, offsets, perm, inv = ops.route_histogram(idx, E)
    A = torch.randn(rows, I, generator=g).bfloat16().to(dev)
    W = (torch.randn(E, H, I, generator=g) * 0.1).bfloat16().to(dev)
    w = torch.rand(rows, generator=g).to(dev)
    As = A[perm.long()]
    def run(dst):
        out = torch.full((rows + 8, H), 7.0, dtype=torch.bfloat16, device=dev)        # 8 canary rows behind the output
        ops.grouped_gemm_sorted(ops.GEMM_SCALE_SCATTER, As, W, offsets, dst_rows=dst, row_w=w[perm.long()], out=out[:rows],
                                max_rows=rows)
        torch.cuda.synchronize()
        return out
    good = run(perm)
    print("clean", ops.debug_bounds_status(dev))
    bad_dst = perm.clone()
    bad_dst[17] = rows + 3                         # a destination inside the canary rows
    bad = run(bad_dst)
    checked, st = ops.debug_bounds_status(dev)
    print("bad", checked, st)
    victim = int(perm[17])
    same = torch.ones(rows + 8, dtype=torch.bool, device=dev)
    same[victim] = False
    print("others_equal", bool(torch.equal(bad[same], good[same])))
    print("canaries_intact", bool((bad[rows:] == 7.0).all()), "victim_untouched", bool((bad[victim] == 7.0).all()))
    print("again", ops.debug_bounds_status(dev))
"""


def test_a_scatter_destination_outside_the_output_is_skipped_and_reported():
    out = _run(SCATTER)
    assert "clean (True, [0, 0, 0])" in out, out
    assert "bad True [4, 1, 303]" in out, out
    assert "others_equal True" in out and "canaries_intact True victim_untouched True" in out, out
    assert "again (True, [0, 0, 0])" in out, out                      # reading the record clears it


COMBINE = """
    T, k, H = 64, 4, 256
    yk = torch.randn(T * k, H, generator=g).bfloat16().to(dev)
    row_of = torch.randperm(T * k, generator=g).int().to(dev)
    scale = torch.rand(T * k, generator=g).to(dev)
    good = ops.combine(yk, k, row_of=row_of, scale=scale, T=T)
    print("clean", ops.debug_bounds_status(dev))
    bad_rows = row_of.clone()
    bad_rows[5 * k + 2] = T * k + 1000             # token 5, slot 2 points far behind the buffer
    bad = ops.combine(yk, k, row_of=bad_rows, scale=scale, T=T)
    print("bad", ops.debug_bounds_status(dev))
    keep = torch.ones(T, dtype=torch.bool, device=dev)
    keep[5] = False
    print("others_equal", bool(torch.equal(bad[keep], good[keep])))
    part = sum(yk[int(row_of[5 * k + s])].float() * float(scale[5 * k + s]) for s in range(k) if s != 2)
    print("token5_without_the_slot", bool(torch.allclose(bad[5].float(), part, rtol=2e-2, atol=2e-2)))
"""


def test_a_combine_row_outside_the_buffer_adds_nothing_and_is_reported():
    out = _run(COMBINE)
    assert "clean (True, [0, 0, 0])" in out, out
    assert "bad (True, [4, 3, 1256])" in out, out
    assert "others_equal True" in out and "token5_without_the_slot True" in out, out


GATHER = """
    E, H, I, T, k = 4, 128, 64, 100, 2
    idx = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).to(dev)
    counts, offsets, perm, inv = ops.route_histogram(idx, E)
    x = torch.randn(T, H, generator=g).bfloat16().to(dev)
    W = (torch.randn(E, I, H, generator=g) * 0.1).bfloat16().to(dev)
    good = ops.grouped_gemm_sorted(ops.GEMM_PLAIN, x, W, offsets, gather=perm, gather_div=k)
    print("clean", ops.debug_bounds_status(dev))
    bad_perm = perm.clone()
    bad_perm[9] = (T + 50) * k                     # names token 150 of 100
    bad = ops.grouped_gemm_sorted(ops.GEMM_PLAIN, x, W, offsets, gather=bad_perm, gather_div=k)
    torch.cuda.synchronize()
    print("bad", ops.debug_bounds_status(dev))
    keep = torch.ones(T * k, dtype=torch.bool, device=dev)
    keep[9] = False
    print("others_equal", bool(torch.equal(bad[keep], good[keep])))
"""


def test_a_gather_source_outside_the_input_is_not_followed_and_is_reported():
    out = _run(GATHER)
    assert "clean (True, [0, 0, 0])" in out, out
    assert "bad (True, [4, 2, 150])" in out, out
    assert "others_equal True" in out, out


def test_the_normal_build_carries_no_checks():
    out = _run("""
        print("normal", ops.debug_bounds_status(dev))
    """, check=False)
    assert "normal (False, [0, 0, 0])" in out, out
