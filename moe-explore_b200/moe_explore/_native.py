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
ACT_CODES = {None: 0, "none": 0, "silu": 1, "gelu": 2, "swiglu": 3, "geglu": 4, "approx_gelu": 5}
TILE_M = 128
# codes a kernel may leave in a status word (include/moe_sm100.h, moe_check_status)
STATUS_WAVE_FALLBACK = 4
STATUS_BAD_LAYOUT = 5
STATUS_BAD_EXPERT_ID = 100


class GemmOptions(ctypes.Structure):
    """``moe_gemm_options``: per-launch choices of the grouped GEMMs (zeros = the library's choices)."""
    _fields_ = [("max_ctas", c_int32), ("wave_sync", c_int32), ("wave_workers", c_int32), ("group_m", c_int32),
                ("align_experts", c_int32), ("single_cta", c_int32), ("separate_copies", c_int32), ("lane_stores", c_int32),
                ("expert_begin", c_int32), ("expert_end", c_int32), ("pair_begin", c_int32), ("pair_end", c_int32),
                ("wave_counter", c_void_p)]


# name -> (restype, argtypes); the single source for both binding and the symbol-export test
_OPT = POINTER(GemmOptions)
SIGNATURES = {
    "moe_last_error": (c_char_p, []),
    "moe_query_device": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "moe_check_status": (c_int, [c_void_p, c_void_p]),
    "moe_read_status": (c_int, [c_void_p, POINTER(c_int32), c_int, c_void_p]),
    "moe_set_wait_limit_cycles": (c_int, [c_int64]),
    "moe_gemm_options_size": (c_size_t, []),
    "moe_padded_rows_bound": (c_int64, [c_int64, c_int]),
    "moe_mtiles_bound": (c_int64, [c_int64, c_int]),
    "moe_routing_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "moe_routing_metadata": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 9 + [c_void_p, c_size_t, c_void_p]),
    "moe_routing_static_scratch_bytes": (c_size_t, []),
    "moe_routing_metadata_static": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 9 + [c_void_p]),
    "moe_layout_from_groups": (c_int, [c_void_p, c_int64, c_int] + [c_void_p] * 7 + [c_void_p]),
    "moe_router_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "moe_store_to_host": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "moe_copy_blocks": (c_int, [POINTER(c_void_p), POINTER(c_void_p), POINTER(c_size_t), c_int, c_void_p]),
    "moe_zero_padding_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "moe_gather_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "moe_gather_rows_peer": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_int, c_int,
                                     c_int, c_int, c_void_p, c_void_p]),
    "moe_unpad_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "moe_combine_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "moe_combine_bwd": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
    "moe_dispatch_rows": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
    "moe_mgrouped_gemm": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _OPT,
                                  c_void_p, c_void_p]),
    "moe_mgrouped_gemm_gather": (c_int, [c_void_p, c_int64, c_void_p, c_int] + [c_void_p] * 6 +
                                 [c_int64, c_int, c_int, c_int, c_int, c_int, _OPT, c_void_p, c_void_p]),
    "moe_mgrouped_gemm_combine": (c_int, [c_void_p] * 5 + [c_int] + [c_void_p] * 3 +
                                  [c_int64, c_int, c_int, c_int, c_int, c_int, _OPT, c_void_p, c_void_p]),
    "moe_mgrouped_gemm_scatter": (c_int, [c_void_p, c_int64, c_void_p, c_int] + [c_void_p] * 6 +
                                  [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, _OPT, c_void_p, c_void_p]),
    "moe_mgrouped_gemm_push": (c_int, [c_void_p] * 8 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _OPT,
                                       c_void_p, c_void_p]),
    "moe_mgrouped_gemm_dglu": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _OPT,
                                       c_void_p, c_void_p]),
    "moe_kgrouped_gemm": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int, c_int, c_int, _OPT, c_void_p, c_void_p]),
    "moe_kgrouped_gemm_gather": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p] +
                                 [c_int64, c_int, c_int, c_int, c_int, _OPT, c_void_p, c_void_p]),
}


class MoeNativeError(RuntimeError):
    """A libmoe_sm100 entry point returned a non-zero status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with status {code}: {text}")
        self.code = code


_lib = None

# Optional observer of the launches (None = off, the default).  A caller that wants per-kernel timings installs an
# object with ``count(n)`` and ``section(key, rows)`` (a context manager put around one launch); the benchmark does.
TRACER = None


class _NoSection:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SECTION = _NoSection()


def _count(n: int) -> None:
    if TRACER is not None:
        TRACER.count(n)


def timed(key: str, rows=None):
    """Context manager around one launch (or a group of them): handed to ``TRACER`` when one is installed."""
    return TRACER.section(key, rows) if TRACER is not None else _NO_SECTION


_Timed = timed


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
        if lib.moe_gemm_options_size() != ctypes.sizeof(GemmOptions):
            raise ImportError(f"{LIB_PATH} was built with another layout of moe_gemm_options: rebuild it")
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
    """Synchronise and raise ``MoeNativeError`` when the status word is non-zero (the word is left as it is)."""
    _check("moe_check_status", load().moe_check_status(status.data_ptr(), _stream()))


def read_status(status: torch.Tensor, reset: bool = False) -> int:
    """The status word's value (synchronises the current stream); ``reset`` clears the word afterwards."""
    code = c_int32(0)
    _check("moe_read_status", load().moe_read_status(status.data_ptr(), ctypes.byref(code), 1 if reset else 0, _stream()))
    return int(code.value)


def set_wait_limit_cycles(cycles: int) -> None:
    """Limit of every device-side wait of the launches that follow, in SM clock cycles (<= 0: the default, 2^32)."""
    _check("moe_set_wait_limit_cycles", load().moe_set_wait_limit_cycles(int(cycles)))


def gemm_options(max_ctas: int = 0, wave_sync: int = 0, wave_workers: int = 0, group_m: int = 0, align_experts: int = 0,
                 single_cta: int = 0, separate_copies: int = 0, lane_stores: int = 0, experts=(0, 0),
                 wave_counter=None, pairs=(0, 0)) -> GemmOptions:
    """``experts`` = (begin, end): the M-grouped kernels process exactly that slice of the expert list; ``pairs`` =
    (begin, end): exactly that slice of the list of row-tile pairs (it may cut through an expert)."""
    return GemmOptions(max_ctas, wave_sync, wave_workers, group_m, align_experts, single_cta, separate_copies, lane_stores,
                       int(experts[0]), int(experts[1]), int(pairs[0]), int(pairs[1]),
                       None if wave_counter is None else wave_counter.data_ptr())


def _opt(options):
    return None if options is None else ctypes.byref(options)


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
                       num_mtiles, status=None):
    require_cuda(group_indices)
    rc = load().moe_layout_from_groups(_ptr(group_indices), num_rows, num_experts, _ptr(pad_offsets), _ptr(row_src),
                                       _ptr(dst_row), _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles),
                                       _ptr(status), _stream())
    _check("moe_layout_from_groups", rc)
    _count(2 if num_rows > 0 else 1)


def router_topk(logits, topk: int, softmax_before_topk: bool, normalize: bool, want_counts: bool = False):
    """Fused router tail (see moe_router_topk in include/moe_sm100.h) -> (scores [T,k], indices int64 [T,k],
    expert_counts int32 [E] or None)."""
    require_cuda(logits)
    assert logits.dim() == 2
    logits = logits.contiguous()
    T, E = logits.shape
    code = 2 if logits.dtype is torch.float32 else dtype_code(logits.dtype)
    scores = torch.empty(T, topk, dtype=logits.dtype, device=logits.device)
    indices = torch.empty(T, topk, dtype=torch.int64, device=logits.device)
    counts = torch.empty(E, dtype=torch.int32, device=logits.device) if want_counts else None
    with timed("router:topk"):
        rc = load().moe_router_topk(_ptr(logits), _ptr(scores), _ptr(indices), _ptr(counts), T, E, topk,
                                    1 if softmax_before_topk else 0, 1 if normalize else 0, code, _stream())
    _check("moe_router_topk", rc)
    _count(1)
    return scores, indices, counts


_PINNED = {}


def read_small(values: torch.Tensor) -> list:
    """The int64 values of a small CUDA tensor as a Python list: ONE host synchronisation, and no memcpy -- a kernel
    stores the words into a cached page-locked buffer (a memcpy would queue on a copy engine behind large host
    transfers of other streams).  CPU tensors are simply converted."""
    if not values.is_cuda:
        return values.tolist()
    assert values.dtype is torch.int64
    flat = values.reshape(-1).contiguous()
    key = (flat.device.index, flat.numel())
    host = _PINNED.get(key)
    if host is None:
        host = torch.empty(max(flat.numel(), 1), dtype=torch.int64).pin_memory()
        _PINNED[key] = host
    rc = load().moe_store_to_host(_ptr(flat), host.data_ptr(), flat.numel() * 8, _stream())
    _check("moe_store_to_host", rc)
    _count(1)
    torch.cuda.current_stream().synchronize()
    return host[: flat.numel()].tolist()


def copy_blocks(dst_addresses, src_addresses, sizes) -> None:
    """One asynchronous device-to-device memcpy per (destination address, source address, bytes) triple, on the
    current stream (copy engines; sources may be peers' buffers)."""
    n = len(sizes)
    if n == 0:
        return
    with timed("rows:copy_blocks"):
        rc = load().moe_copy_blocks((c_void_p * n)(*dst_addresses), (c_void_p * n)(*src_addresses), (c_size_t * n)(*sizes), n,
                                    _stream())
    _check("moe_copy_blocks", rc)


def zero_padding_rows(row_src, num_mtiles, dst) -> None:
    """dst[p] = 0 for the padding rows (row_src[p] < 0) of a buffer in the padded layout."""
    require_cuda(dst)
    rc = load().moe_zero_padding_rows(_ptr(row_src), _ptr(num_mtiles), _ptr(dst), dst.size(0), dst.size(1),
                                      dtype_code(dst.dtype), _stream())
    _check("moe_zero_padding_rows", rc)
    _count(1)


def gather_rows(src, row_src, num_mtiles, dst, div):
    require_cuda(src, dst)
    with timed("rows:gather"):
        rc = load().moe_gather_rows(_ptr(src), src.size(0), _ptr(row_src), _ptr(num_mtiles), _ptr(dst), dst.size(0),
                                    src.size(1), div, dtype_code(src.dtype), _stream())
    _check("moe_gather_rows", rc)
    _count(1)


def gather_rows_peer(peer_bases, src_rank, src_row, scale, num_mtiles, dst, tile_pairs=None, num_experts=0,
                     chunk=(0, 1), bulk_ctas: int = 0, status=None, experts=None, dedicated_ctas: int = 0, pairs=(0, 0)):
    """dst[p] = scale[p] * peer_bases[src_rank[p]][src_row[p]]; peer_bases: int64 device tensor of base pointers.
    ``bulk_ctas`` > 0: the copy-engine kernel on that many CTAs; 0: the load/store kernel, on all SMs or, with
    ``dedicated_ctas`` > 0, as that many 1024-thread CTAs that each take a whole SM.
    ``experts`` = (begin, end) restricts the call to the rows of that slice of the expert list (else ``chunk``);
    ``pairs`` = (begin, end) to the rows of that slice of the list of row-tile pairs."""
    require_cuda(peer_bases, dst)
    if experts is not None:
        chunk = (int(experts[0]), -int(experts[1]))   # the C entry point's encoding of an explicit range
    with timed("rows:gather_peer"):
        rc = load().moe_gather_rows_peer(_ptr(peer_bases), _ptr(src_rank), _ptr(src_row), _ptr(scale), _ptr(num_mtiles),
                                         _ptr(tile_pairs), num_experts, chunk[0], chunk[1], int(pairs[0]), int(pairs[1]),
                                         _ptr(dst), dst.size(0),
                                         dst.size(1), dtype_code(dst.dtype), int(bulk_ctas), int(dedicated_ctas),
                                         _ptr(status), _stream())
    _check("moe_gather_rows_peer", rc)
    _count(1)


def mgrouped_gemm_push(a, w, peer_bases, dest_rank, dest_row, mtile_expert, tile_pairs, num_mtiles, w_transposed,
                       status=None, rows=None, chunk=(0, 1), options=None):
    """Grouped GEMM whose epilogue stores each row into the owning rank's buffer (peer stores)."""
    require_cuda(a, w, peer_bases)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    with timed("mgrouped_gemm:push_wt" if w_transposed else "mgrouped_gemm:push", rows):
        rc = load().moe_mgrouped_gemm_push(_ptr(a), _ptr(w), _ptr(peer_bases), _ptr(dest_rank), _ptr(dest_row),
                                           _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), a.size(0), K, N, E,
                                           1 if w_transposed else 0, dtype_code(a.dtype), chunk[0], chunk[1],
                                           _opt(options), _ptr(status), _stream())
    _check("moe_mgrouped_gemm_push", rc)
    _count(1)


def unpad_rows(src, dst_row, out):
    require_cuda(src, out)
    with timed("rows:unpad"):
        rc = load().moe_unpad_rows(_ptr(src), _ptr(dst_row), _ptr(out), out.size(0), out.size(1),
                                   dtype_code(src.dtype), _stream())
    _check("moe_unpad_rows", rc)
    _count(1)


def combine_topk(ys, scores, dst_row, out, topk):
    require_cuda(ys, out)
    with timed("rows:combine"):
        rc = load().moe_combine_topk(_ptr(ys), _ptr(scores), _ptr(dst_row), _ptr(out), out.size(0), topk, out.size(1),
                                     dtype_code(ys.dtype), _stream())
    _check("moe_combine_topk", rc)
    _count(1)


def dispatch_rows(src, dst_row, row_src, num_mtiles, dst, topk):
    """dst[dst_row[t*topk+s]] = src[t]; padding rows of dst zeroed."""
    require_cuda(src, dst)
    with timed("rows:gather"):
        rc = load().moe_dispatch_rows(_ptr(src), _ptr(dst_row), _ptr(row_src), _ptr(num_mtiles), _ptr(dst), src.size(0),
                                      topk, dst.size(0), src.size(1), dtype_code(src.dtype), _stream())
    _check("moe_dispatch_rows", rc)
    _count(1)


def combine_bwd(dout, scores, ys, row_src, num_mtiles, gs, dscores, topk):
    require_cuda(dout, ys, dscores)
    with timed("rows:combine_bwd"):
        rc = load().moe_combine_bwd(_ptr(dout), _ptr(scores), _ptr(ys), _ptr(row_src), _ptr(num_mtiles), _ptr(gs),
                                    _ptr(dscores), dout.size(0), topk, ys.size(0), dout.size(1), dtype_code(dout.dtype),
                                    _stream())
    _check("moe_combine_bwd", rc)
    _count(1)


def mgrouped_gemm(a, w, out, pre_act, mtile_expert, tile_pairs, num_mtiles, w_transposed, act, status=None, rows=None,
                  chunk=(0, 1), options=None):
    require_cuda(a, w, out)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    key = "mgrouped_gemm:" + ("glu" if act in ("swiglu", "geglu") else ("wt" if w_transposed else "plain"))
    with timed(key, rows):
        rc = load().moe_mgrouped_gemm(_ptr(a), _ptr(w), _ptr(out), _ptr(pre_act), _ptr(mtile_expert),
                                      _ptr(tile_pairs), _ptr(num_mtiles), a.size(0), K, N, E, 1 if w_transposed else 0,
                                      ACT_CODES[act], dtype_code(a.dtype), chunk[0], chunk[1], _opt(options), _ptr(status),
                                      _stream())
    _check("moe_mgrouped_gemm", rc)
    _count(1)


def mgrouped_gemm_gather(src, row_src, div, w, out, pre_act, mtile_expert, tile_pairs, num_mtiles, padded_rows, act,
                         status=None, rows=None, options=None):
    """out = epilogue(src[row_src // div] @ w[expert]) with the row gather inside the operand loads; w [E, K, N]."""
    require_cuda(src, w, out)
    E, K, N = w.shape
    key = "mgrouped_gemm:" + ("glu" if act in ("swiglu", "geglu") else "plain") + "+gather"
    with timed(key, rows):
        rc = load().moe_mgrouped_gemm_gather(_ptr(src), src.size(0), _ptr(row_src), div, _ptr(w), _ptr(out), _ptr(pre_act),
                                             _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), padded_rows, K, N, E,
                                             ACT_CODES[act], dtype_code(src.dtype), _opt(options), _ptr(status), _stream())
    _check("moe_mgrouped_gemm_gather", rc)
    _count(1)


def mgrouped_gemm_combine(a, w, out, row_src, scores, topk, mtile_expert, tile_pairs, num_mtiles, w_transposed,
                          status=None, rows=None, options=None):
    """out[row_src[p] // topk] += scores[row_src[p]] * (a[p] @ w[expert]); ``out`` [T, N] must be zero on entry."""
    require_cuda(a, w, out)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    with timed("mgrouped_gemm:combine", rows):
        rc = load().moe_mgrouped_gemm_combine(_ptr(a), _ptr(w), _ptr(out), _ptr(row_src), _ptr(scores), topk,
                                              _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles), a.size(0), K, N, E,
                                              1 if w_transposed else 0, dtype_code(a.dtype), _opt(options), _ptr(status),
                                              _stream())
    _check("moe_mgrouped_gemm_combine", rc)
    _count(1)


def mgrouped_gemm_scatter(a, w, out, out_rows, mtile_expert, tile_pairs, num_mtiles, padded_rows, w_transposed=False,
                          act=None, a_row_src=None, a_div=1, status=None, rows=None, options=None):
    """out[out_rows[p]] = act(a_p @ w[expert]) (rows with out_rows[p] < 0 are skipped); a_p is row p of ``a``
    [RP, K], or, with ``a_row_src``, row a_row_src[p] // a_div of ``a`` gathered by the operand loads."""
    require_cuda(a, w, out)
    E = w.size(0)
    K = a.size(1)
    N = w.size(1) if w_transposed else w.size(2)
    with timed("mgrouped_gemm:scatter", rows):
        rc = load().moe_mgrouped_gemm_scatter(_ptr(a), a.size(0), _ptr(a_row_src), a_div, _ptr(w), _ptr(out),
                                              _ptr(out_rows), _ptr(mtile_expert), _ptr(tile_pairs), _ptr(num_mtiles),
                                              padded_rows, K, N, E, 1 if w_transposed else 0, ACT_CODES[act],
                                              dtype_code(a.dtype), _opt(options), _ptr(status), _stream())
    _check("moe_mgrouped_gemm_scatter", rc)
    _count(1)


def mgrouped_gemm_dglu(g, w, pre_act, d_pre, mtile_expert, tile_pairs, num_mtiles, act, status=None, rows=None,
                       chunk=(0, 1), options=None):
    require_cuda(g, w, pre_act, d_pre)
    E, N, K = w.shape
    with timed("mgrouped_gemm:dglu", rows):
        rc = load().moe_mgrouped_gemm_dglu(_ptr(g), _ptr(w), _ptr(pre_act), _ptr(d_pre), _ptr(mtile_expert),
                                           _ptr(tile_pairs), _ptr(num_mtiles), g.size(0), K, N, E, ACT_CODES[act],
                                           dtype_code(g.dtype), chunk[0], chunk[1], _opt(options), _ptr(status), _stream())
    _check("moe_mgrouped_gemm_dglu", rc)
    _count(1)


def kgrouped_gemm(a, b, dw, pad_offsets, status=None, rows=None, tag="dw", options=None):
    require_cuda(a, b, dw)
    E, M, N = dw.shape
    with timed("kgrouped_gemm:" + tag, rows):
        rc = load().moe_kgrouped_gemm(_ptr(a), _ptr(b), _ptr(dw), _ptr(pad_offsets), a.size(0), M, N, E,
                                      dtype_code(a.dtype), _opt(options), _ptr(status), _stream())
    _check("moe_kgrouped_gemm", rc)
    _count(1)


def kgrouped_gemm_gather(src, row_src, div, b, dw, pad_offsets, status=None, rows=None, tag="dw", options=None):
    """dw[e] = src[row_src // div over the rows of e]^T @ b[rows of e]: the rows of the first operand gathered by
    the operand loads."""
    require_cuda(src, b, dw)
    E, M, N = dw.shape
    with timed("kgrouped_gemm:" + tag + "+gather", rows):
        rc = load().moe_kgrouped_gemm_gather(_ptr(src), src.size(0), _ptr(row_src), div, _ptr(b), _ptr(dw),
                                             _ptr(pad_offsets), b.size(0), M, N, E, dtype_code(src.dtype), _opt(options),
                                             _ptr(status), _stream())
    _check("moe_kgrouped_gemm_gather", rc)
    _count(1)
