"""The histogram entry point that needs no workspace from the caller.

Some hosts cannot give the library scratch memory and do not let it allocate any (they hand a
plug-in only its inputs and outputs).  `moe_route_histogram_static` serves them from an array
built into the library.  This test drives it through the C ABI and checks, twice in a row with
different inputs, that it returns exactly what `moe_route_histogram` returns with a workspace:
the second call runs over whatever the first left in the shared array.
"""
import ctypes

import pytest
import torch

from tilelang_moe_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(lib, ids, E, id_map, static):
    dev = ids.device
    n = ids.numel()
    counts = torch.full((E,), -7, dtype=torch.int32, device=dev)
    offsets = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
    perm = torch.full((max(n, 1),), -7, dtype=torch.int32, device=dev)
    inv = torch.full((max(n, 1),), -7, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    mp = None if id_map is None else id_map.data_ptr()
    is64 = int(ids.dtype == torch.int64)
    if static:
        rc = lib.moe_route_histogram_static(ids.data_ptr(), is64, n, E, mp, counts.data_ptr(), offsets.data_ptr(),
                                            perm.data_ptr(), inv.data_ptr(), status.data_ptr(), stream)
    else:
        need = lib.moe_route_histogram_workspace(n, E)
        ws = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
        rc = lib.moe_route_histogram(ids.data_ptr(), is64, n, E, mp, counts.data_ptr(), offsets.data_ptr(),
                                     perm.data_ptr(), inv.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(),
                                     stream)
    assert rc == 0, lib.moe_last_error()
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    return counts.cpu(), offsets.cpu(), perm.cpu(), inv.cpu()


def test_static_scratch_matches_workspace_variant_twice(cuda, lib):
    torch.cuda.set_device(cuda)
    g = torch.Generator().manual_seed(21)
    # first call: the benchmark layer's size, int32 ids, with a renumbering table
    ids1 = torch.randint(0, 256, (8192 * 8,), generator=g, dtype=torch.int32).to(cuda)
    id_map = torch.randperm(256, generator=g).to(torch.int32).to(cuda)
    # second call: smaller, int64 ids, other expert count -> reads a table region the first call filled
    ids2 = torch.randint(0, 40, (5000,), generator=g, dtype=torch.int64).to(cuda)
    for ids, E, mp in ((ids1, 256, id_map), (ids2, 40, None)):
        got = _run(lib, ids, E, mp, static=True)
        want = _run(lib, ids, E, mp, static=False)
        for a, b in zip(got, want):
            assert torch.equal(a, b)                     # integer work: bit-exact
        assert int(got[1][-1]) == ids.numel()


def test_static_scratch_rejects_oversize(cuda, lib):
    torch.cuda.set_device(cuda)
    one = torch.zeros(1, dtype=torch.int32, device=cuda)
    big_n = 1024 * 1025                                   # 1025 units x 256 experts > 262144 entries
    rc = lib.moe_route_histogram_static(one.data_ptr(), 0, big_n, 256, None, one.data_ptr(), one.data_ptr(), None,
                                        None, None, None)
    assert rc == -2
    assert b"exceeds the built-in scratch" in lib.moe_last_error()
