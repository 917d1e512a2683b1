"""ctypes binding of libmoe_sm100.so (the C ABI declared in include/moe_sm100.h).

The library is built in-tree by ``build_native.py`` (next to this package) and must be
present: there is no fallback path.  Every wrapper raises ``MoeNativeError`` carrying the
library's own error text when a call returns a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int32, c_int64, c_size_t, c_void_p, c_char_p, POINTER

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# MOE_SM100_LIBRARY points at another build of the same library (e.g. one compiled with instrumentation)
LIB_PATH = os.environ.get("MOE_SM100_LIBRARY") or os.path.join(os.path.dirname(_PKG_DIR), "libmoe_sm100.so")

MOE_DTYPE_BF16 = 0
MOE_DTYPE_F16 = 1
ACT_CODES = {None: 0, "none": 0, "silu": 1, "gelu": 2, "swiglu": 3, "geglu": 4}
TILE_M = 128

# name -> (restype, argtypes); the single source for both binding and the symbol-export test
SIGNATURES = {
    "moe_last_error": (c_char_p, []),
    "moe_query_device": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "moe_check_status": (c_int, [c_void_p, c_void_p]),
    "moe_padded_rows_bound": (c_int64, [c_int64, c_int]),
    "moe_mtiles_bound": (c_int64, [c_int64, c_int]),
    "moe_routing_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "moe_routing_metadata": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 9 + [c_void_p, c_size_t, c_void_p]),
    "moe_routing_static_scratch_bytes": (c_size_t, []),
    "moe_routing_metadata_static": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 9 + [c_void_p]),
    "moe_layout_from_groups": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 6 + [c_void_p]),
    "moe_gather_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "moe_gather_rows_peer": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "moe_mgrouped_gemm_push": (c_int, [c_void_p] * 8 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moe_unpad_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "moe_combine_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "moe_combine_bwd": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
    "moe_dispatch_rows": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
    "moe_mgrouped_gemm": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moe_mgrouped_gemm_dglu": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "moe_set_gemm_grid_limit": (c_int, [c_int]),
    "moe_kgrouped_gemm": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
}


class MoeNativeError(RuntimeError):
    """A libmoe_sm100 entry point returned a non-zero status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with status {code}: {text}")
        self.code = code


_lib = None

# Instrumentation used by the benchmark: LAUNCHES counts this library's kernel launches; when
# PROFILE is a dict, the grouped-GEMM wrappers bracket their launch with CUDA events on the
# current stream and append (start, end) under a key naming the kernel variant.
LAUNCHES = 0
PROFILE = None


def _count(n: int) -> None:
    global LAUNCHES
    LAUNCHES += n


class _Timed:
    def __init__(self, key: str, rows=None):
        self.key = key if PROFILE is not None else None
        self.rows = rows

    def __enter__(self):
        if self.key is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record()

    def __exit__(self, *exc):
        if self.key is not None:
            self.end.record()
            PROFILE.setdefault(self.key, []).append((self.start, self.end, self.rows))
        return False


def timed(key: str, rows=None):
    """Context manager: CUDA-event bracket on the current stream, recorded under ``key`` while
    ``PROFILE`` is a dict; free otherwise.  ``rows`` notes how many routed rows the section handled."""
    return _Timed(key, rows)


def load() -> ctypes.CDLL:
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python moe-explore_b200/build_native.py` "
                "(this package has no fallback path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def _check(fn: str, rc: int) -> None:
    if rc != 0:
        raise MoeNativeError(fn, rc, load().moe_last_error().decode())


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype is torch.bfloat16:
        return MOE_DTYPE_BF16
    if dtype is torch.float16:
        return MOE_DTYPE_F16
    raise TypeError(f"libmoe_sm100 computes in bf16 or fp16 (fp32 accumulate); got {dtype}")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libmoe_sm100 runs on CUDA tensors only (no CPU path); got a tensor on " + str(t.device))


def padded_rows_bound(num_rows: int, num_experts: int) -> int:
    return int(load().moe_padded_rows_bound(num_rows, num_experts))


def mtiles_bound(num_rows: int, num_experts: int) -> int:
    return int(load().moe_mtiles_bound(num_rows, num_experts))


def query_device(device: int = 0):
    sm, major, minor = c_int(0), c_int(0), c_int(0)
    rc = load().moe_query_device(device, ctypes.byref(sm), ctypes.byref(major), ctypes.byref(minor))
    _check("moe_query_device", rc)
    return sm.value, major.value, minor.value


def check_status(status: torch.Tensor) -> None:
    _check("moe_check_status", load().moe_check_status(status.data_ptr(), _stream()))


def routing_metadata(expert_idx, num_experts, group_indices, perm, pad_offsets, row_src, dst_row, mtile_expert,
                     tile_pairs, num_mtiles, status, workspace):
    require_cuda(expert_idx)
    rc = load().moe_routing_metadata(_ptr(expert_idx), expert_idx.numel(), num_experts, _ptr(group_indices),
                                     _ptr(perm), _ptr(pad_offsets), _ptr(row_src), _ptr(dst_row),
                                     _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), _ptr(status),
                                     _ptr(workspace),
                                     workspace.numel() * workspace.element_size(), _stream())
    _check("moe_routing_metadata", rc)
    _count(3 if expert_idx.numel() > 0 else 1)


def routing_metadata_static(expert_idx, num_experts, group_indices, perm, pad_offsets, row_src, dst_row, mtile_expert,
                            tile_pairs, num_mtiles, status):
    """Routing metadata with the library's built-in scratch: for callers that cannot allocate
    device memory.  Calls on one device must not overlap; see include/moe_sm100.h for the limits."""
    require_cuda(expert_idx)
    rc = load().moe_routing_metadata_static(_ptr(expert_idx), expert_idx.numel(), num_experts, _ptr(group_indices),
                                            _ptr(perm), _ptr(pad_offsets), _ptr(row_src), _ptr(dst_row),
                                            _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), _ptr(status),
                                            _stream())
    _check("moe_routing_metadata_static", rc)
    _count(3 if expert_idx.numel() > 0 else 1)


def routing_workspace_bytes(num_rows: int, num_experts: int) -> int:
    return int(load().moe_routing_workspace_bytes(num_rows, num_experts))


def layout_from_groups(group_indices, num_rows, num_experts, pad_offsets, row_src, dst_row, mtile_expert, tile_pairs,
                       num_mtiles):
    require_cuda(group_indices)
    rc = load().moe_layout_from_groups(_ptr(group_indices), num_rows, num_experts, _ptr(pad_offsets), _ptr(row_src),
                                       _ptr(dst_row), _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles),
                                       _stream())
    _check("moe_layout_from_groups", rc)
    _count(2 if num_rows > 0 else 1)


def gather_rows(src, row_src, num_mtiles, dst, div):
    require_cuda(src, dst)
    with _Timed("rows:gather"):
        rc = load().moe_gather_rows(_ptr(src), src.size(0), _ptr(row_src), _ptr(num_mtiles), _ptr(dst), dst.size(0),
                                    src.size(1), div, dtype_code(src.dtype), _stream())
    _check("moe_gather_rows", rc)
    _count(1)


def gather_rows_peer(peer_bases, src_rank, src_row, scale, num_mtiles, dst, tile_pairs=None, num_experts=0,
                     chunk=(0, 1)):
    """dst[p] = scale[p] * peer_bases[src_rank[p]][src_row[p]]; peer_bases: int64 device tensor of base pointers."""
    require_cuda(peer_bases, dst)
    with _Timed("rows:gather_peer"):
        rc = load().moe_gather_rows_peer(_ptr(peer_bases), _ptr(src_rank), _ptr(src_row), _ptr(scale), _ptr(num_mtiles),
                                         _ptr(tile_pairs), num_experts, chunk[0], chunk[1], _ptr(dst), dst.size(0),
                                         dst.size(1),
                                         dtype_code(dst.dtype), _stream())
    _check("moe_gather_rows_peer", rc)
    _count(1)


def mgrouped_gemm_push(a, w, peer_bases, dest_rank, dest_row, mtile_expert, tile_pairs, num_mtiles, w_transposed,
                       status=None, rows=None, chunk=(0, 1)):
    """Grouped GEMM whose epilogue stores each row into the owning rank's buffer (peer stores)."""
    require_cuda(a, w, peer_bases)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    with _Timed("mgrouped_gemm:push_wt" if w_transposed else "mgrouped_gemm:push", rows):
        rc = load().moe_mgrouped_gemm_push(_ptr(a), _ptr(w), _ptr(peer_bases), _ptr(dest_rank), _ptr(dest_row),
                                           _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), a.size(0), K, N, E,
                                           1 if w_transposed else 0, dtype_code(a.dtype), chunk[0], chunk[1],
                                           _ptr(status), _stream())
    _check("moe_mgrouped_gemm_push", rc)
    _count(1)


def unpad_rows(src, dst_row, out):
    require_cuda(src, out)
    with _Timed("rows:unpad"):
        rc = load().moe_unpad_rows(_ptr(src), _ptr(dst_row), _ptr(out), out.size(0), out.size(1),
                                   dtype_code(src.dtype), _stream())
    _check("moe_unpad_rows", rc)
    _count(1)


def combine_topk(ys, scores, dst_row, out, topk):
    require_cuda(ys, out)
    with _Timed("rows:combine"):
        rc = load().moe_combine_topk(_ptr(ys), _ptr(scores), _ptr(dst_row), _ptr(out), out.size(0), topk, out.size(1),
                                     dtype_code(ys.dtype), _stream())
    _check("moe_combine_topk", rc)
    _count(1)


def dispatch_rows(src, dst_row, row_src, num_mtiles, dst, topk):
    """dst[dst_row[t*topk+s]] = src[t]; padding rows of dst zeroed."""
    require_cuda(src, dst)
    with _Timed("rows:gather"):
        rc = load().moe_dispatch_rows(_ptr(src), _ptr(dst_row), _ptr(row_src), _ptr(num_mtiles), _ptr(dst), src.size(0),
                                      topk, dst.size(0), src.size(1), dtype_code(src.dtype), _stream())
    _check("moe_dispatch_rows", rc)
    _count(1)


def combine_bwd(dout, scores, ys, row_src, num_mtiles, gs, dscores, topk):
    require_cuda(dout, ys, dscores)
    with _Timed("rows:combine_bwd"):
        rc = load().moe_combine_bwd(_ptr(dout), _ptr(scores), _ptr(ys), _ptr(row_src), _ptr(num_mtiles), _ptr(gs),
                                    _ptr(dscores), dout.size(0), topk, ys.size(0), dout.size(1), dtype_code(dout.dtype),
                                    _stream())
    _check("moe_combine_bwd", rc)
    _count(1)


def mgrouped_gemm(a, w, out, pre_act, mtile_expert, tile_pairs, num_mtiles, w_transposed, act, status=None, rows=None,
                  chunk=(0, 1)):
    require_cuda(a, w, out)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    key = "mgrouped_gemm:" + ("glu" if act in ("swiglu", "geglu") else ("wt" if w_transposed else "plain"))
    with _Timed(key, rows):
        rc = load().moe_mgrouped_gemm(_ptr(a), _ptr(w), _ptr(out), _ptr(pre_act), _ptr(mtile_expert),
                                      _ptr(tile_pairs), _ptr(num_mtiles), a.size(0), K, N, E, 1 if w_transposed else 0, ACT_CODES[act],
                                      dtype_code(a.dtype), chunk[0], chunk[1], _ptr(status), _stream())
    _check("moe_mgrouped_gemm", rc)
    _count(1)


def mgrouped_gemm_dglu(g, w, pre_act, d_pre, mtile_expert, tile_pairs, num_mtiles, act, status=None, rows=None,
                       chunk=(0, 1)):
    require_cuda(g, w, pre_act, d_pre)
    E, N, K = w.shape
    with _Timed("mgrouped_gemm:dglu", rows):
        rc = load().moe_mgrouped_gemm_dglu(_ptr(g), _ptr(w), _ptr(pre_act), _ptr(d_pre), _ptr(mtile_expert),
                                           _ptr(tile_pairs), _ptr(num_mtiles), g.size(0), K, N, E, ACT_CODES[act], dtype_code(g.dtype),
                                           chunk[0], chunk[1], _ptr(status), _stream())
    _check("moe_mgrouped_gemm_dglu", rc)
    _count(1)


def set_gemm_grid_limit(max_ctas: int) -> None:
    """Cap the CTAs of the grouped-GEMM launches that follow (0 removes the cap)."""
    _check("moe_set_gemm_grid_limit", load().moe_set_gemm_grid_limit(int(max_ctas)))


def kgrouped_gemm(a, b, dw, pad_offsets, status=None, rows=None, tag="dw"):
    require_cuda(a, b, dw)
    E, M, N = dw.shape
    with _Timed("kgrouped_gemm:" + tag, rows):
        rc = load().moe_kgrouped_gemm(_ptr(a), _ptr(b), _ptr(dw), _ptr(pad_offsets), a.size(0), M, N, E,
                                      dtype_code(a.dtype), _ptr(status), _stream())
    _check("moe_kgrouped_gemm", rc)
    _count(1)
