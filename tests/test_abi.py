"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import re

from conftest import ROOT
from tilelang_moe_b200 import _lib


def _declared():
    text = (ROOT / "include" / "moe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/moe_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes prototypes and header disagree"


def test_version_and_error_channel(lib):
    assert lib.moe_abi_version() == 1
    # argument errors are detected on the host before any CUDA call
    rc = lib.moe_topk_softmax(None, 4, 8, 8, 2, 0, None, None, None, None, None)
    assert rc == -1
    assert b"null" in lib.moe_last_error()
    rc = lib.moe_topk_softmax(ctypes.c_void_p(16), 4, 8, 8, 9, 0, ctypes.c_void_p(16), ctypes.c_void_p(16), None, None, None)
    assert rc == -1 and b"bad shape" in lib.moe_last_error()
    rc = lib.moe_grouped_gemm(0, None, None, None, None, None, None, None, 8, 16, 0, 12, 8, 1, 0, None, None)
    assert rc == -1 and b"multiples of 8" in lib.moe_last_error()
    rc = lib.moe_route_histogram(None, 1, 10, 4, None, None, None, None, None, None, 0, None, None)
    assert rc == -1
    assert lib.moe_route_histogram_workspace(2048, 8) == 16 * 8 * 4          # small inputs: units of 128 ids
    assert lib.moe_route_histogram_workspace(65536, 256) == 512 * 256 * 4    # ... up to 65536 ids while the table stays small
    assert lib.moe_route_histogram_workspace(65536, 1024) == 64 * 1024 * 4   # many experts: units of 1024 ids
    assert lib.moe_route_histogram_workspace(1 << 20, 256) == 1024 * 256 * 4 # large inputs: units of 1024 ids
    assert lib.moe_route_histogram_workspace(0, 8) == 0


def test_cpu_tensors_are_rejected():
    import pytest
    import torch
    from tilelang_moe_b200 import kernels
    with pytest.raises(ValueError):
        kernels.topk_softmax(torch.randn(4, 8), 2)


def test_every_public_name_of_the_reference_package_exists():
    """The names the reference's kernels/__init__.py exports (its __all__, :67-101): code written against any of them
    must find it here."""
    import tilelang_moe_b200.kernels as K
    reference_all = [
        "topk_radix_tilelang", "topk_softmax_separate", "topk_softmax_separate_compiled", "topk_softmax_fused",
        "topk_softmax_selection", "topk_softmax_sonic", "topk_softmax_bitonic", "topk_softmax_tilelang_separate",
        "topk_softmax_best", "topk_softmax",
        "grouped_gemm_loop", "grouped_gemm_loop_compiled", "grouped_gemm_padded", "grouped_gemm_tilelang",
        "grouped_gemm_pytorch", "grouped_gemm_best", "grouped_gemm",
        "mhc_pre_pytorch", "mhc_pre_pytorch_compiled", "mhc_post_pytorch", "mhc_post_pytorch_compiled",
        "mhc_pre_tilelang_official", "mhc_pre_tilelang_optimized", "mhc_pre_tilelang_splitk", "mhc_pre",
        "mhc_post_tilelang_official", "mhc_post",
        "fusedmoe_pytorch", "fusedmoe_pytorch_compiled", "fusedmoe_tilelang", "generate_fusedmoe_inputs",
        "FusedMoETileLang",
    ]
    missing = [n for n in reference_all if not callable(getattr(K, n, None))]
    assert not missing, missing
    assert set(reference_all) <= set(K.__all__)
