"""The C ABI: every function declared in include/moe_sm100.h is exported by libmoe_sm100.so and
bound by the ctypes layer; argument validation answers with a status code and an error text
(no compute launches: these run without a GPU)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "moe_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared_functions()
    for must in ("moe_routing_metadata", "moe_mgrouped_gemm", "moe_mgrouped_gemm_gather", "moe_mgrouped_gemm_combine",
                 "moe_mgrouped_gemm_scatter", "moe_mgrouped_gemm_dglu", "moe_kgrouped_gemm", "moe_kgrouped_gemm_gather",
                 "moe_gather_rows", "moe_combine_topk", "moe_combine_bwd", "moe_last_error", "moe_query_device",
                 "moe_router_topk", "moe_set_wait_limit_cycles", "moe_read_status"):
        assert must in names


def test_library_exports_every_declared_symbol(native):
    lib = native.load()
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in moe_sm100.h but not exported"
        assert name in native.SIGNATURES, f"{name} has no ctypes signature"
    assert set(native.SIGNATURES) == set(_declared_functions())


def test_size_helpers(native):
    assert native.padded_rows_bound(0, 8) == 8 * 127 // 128 * 128 + 128 or native.padded_rows_bound(0, 8) % 128 == 0
    for rows, experts in [(1, 1), (1024, 8), (16384, 8), (65536, 60), (262144, 256), (524288, 64)]:
        rp = native.padded_rows_bound(rows, experts)
        assert rp % 128 == 0 and rp >= rows + experts * 127 and rp < rows + experts * 127 + 128
        assert native.mtiles_bound(rows, experts) * 128 == rp
        assert native.routing_workspace_bytes(rows, experts) >= 2 * 4 * experts * ((rows + 1023) // 1024)


def test_invalid_arguments_are_reported_not_launched(native):
    lib = native.load()
    rc = lib.moe_mgrouped_gemm(None, None, None, None, None, None, None, 128, 64, 64, 1, 0, 0, 0, 0, 1, None, None, None)
    assert rc == -1 and b"null" in lib.moe_last_error()
    rc = lib.moe_routing_metadata(None, -5, 8, None, None, None, None, None, None, None, None, None, None, 0, None)
    assert rc == -1 and b"negative" in lib.moe_last_error()
    rc = lib.moe_routing_metadata(None, 0, 5000, None, None, None, None, None, None, None, None, None, None, 0, None)
    assert rc == -2 and b"maximum" in lib.moe_last_error()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p += (-p) % 16  # the library checks 16-byte alignment before anything else
    # K not a multiple of 8 (the reference's K=300, N=20 test shape): unsupported, stated clearly
    rc = lib.moe_mgrouped_gemm(p, p, p, None, p, p, p, 128, 300, 20, 2, 0, 0, 0, 0, 1, None, None, None)
    assert rc == -2 and b"multiples of 8" in lib.moe_last_error()
    rc = lib.moe_mgrouped_gemm(p, p, p, None, p, p, p, 100, 64, 64, 2, 0, 0, 0, 0, 1, None, None, None)
    assert rc == -1 and b"padded_rows" in lib.moe_last_error()
    rc = lib.moe_mgrouped_gemm(p, p, p, None, p, p, p, 128, 64, 64, 2, 0, 9, 0, 0, 1, None, None, None)
    assert rc == -1 and b"activation" in lib.moe_last_error()
    rc = lib.moe_mgrouped_gemm(p, p, p, None, p, None, p, 128, 64, 64, 2, 0, 0, 0, 1, 4, None, None, None)
    assert rc == -1 and b"chunk" in lib.moe_last_error()   # chunked launches need the tile-pair list
    rc = lib.moe_mgrouped_gemm(p, p, p, None, p, p, p, 128, 64, 64, 2, 1, 3, 0, 0, 1, None, None, None)
    assert rc == -1 and b"gated" in lib.moe_last_error()   # a gated epilogue reads w as [E, K, N] only
    rc = lib.moe_mgrouped_gemm_gather(p, 0, p, 2, p, p, None, p, p, p, 128, 64, 64, 2, 0, 0, None, None, None)
    assert rc == -1 and b"gathered" in lib.moe_last_error()   # the gathered tensor needs at least one row
    rc = lib.moe_mgrouped_gemm_scatter(p, 128, None, 1, p, p, p, p, p, p, 128, 64, 64, 2, 0, 3, 0, None, None, None)
    assert rc == -1 and b"element-wise" in lib.moe_last_error()
    rc = lib.moe_mgrouped_gemm_combine(p, p, p, None, None, 2, p, p, p, 128, 64, 64, 2, 0, 0, None, None, None)
    assert rc == -1 and b"null" in lib.moe_last_error()
    rc = lib.moe_kgrouped_gemm(p, p, p, p, 128, 64, 60, 2, 0, None, None, None)
    assert rc == -2
    rc = lib.moe_router_topk(p, p, p, None, 4, 2000, 2, 0, 0, 0, None)
    assert rc == -2 and b"E <=" in lib.moe_last_error()
    rc = lib.moe_router_topk(p, p, p, None, 4, 8, 2, 0, 0, 7, None)
    assert rc == -1 and b"dtype" in lib.moe_last_error()
    rc = lib.moe_combine_topk(p, None, p, p, 4, 0, 64, 0, None)
    assert rc == -1
    rc = lib.moe_gather_rows(p, 4, p, p, p, 128, 64, 1, 7, None)
    assert rc == -1 and b"dtype" in lib.moe_last_error()


def test_python_wrappers_refuse_cpu_tensors(native):
    import torch

    from moe_explore.expert_permute import get_token_indices
    from moe_explore.functional.scale_and_reduce import scale_and_reduce

    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        get_token_indices(torch.zeros(4, 2, dtype=torch.int64), 2, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        scale_and_reduce(torch.zeros(8, 16), torch.zeros(4, 2), 4, 2, 16)
    with pytest.raises(TypeError):
        native.dtype_code(torch.float32)


def test_missing_library_fails_loudly(native, monkeypatch):
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", "/nonexistent/libmoe_sm100.so")
    with pytest.raises(ImportError, match="no fallback"):
        native.load()
