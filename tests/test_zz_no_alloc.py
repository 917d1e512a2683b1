"""moe_routing_metadata_static: routing metadata for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is not available to them -- a server whose device
memory is one arena sized at start-up, a plugin host that passes an operator its inputs and outputs
and nothing more, a loop that must not touch the allocator.  For them the library carries the
counting sort's scratch inside its own image.  This test calls that entry point through the C ABI
and requires, twice in a row on different inputs, exactly the outputs of the ordinary entry point
(integer work: bit-exact).  The second call runs on the scratch the first one left behind, so it
also shows that nothing in the scratch has to be cleared between calls.

Collected last on purpose (file name), so that a run that stops at the first failure has already
run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(num_rows, num_experts, native):
    rp = native.padded_rows_bound(num_rows, num_experts)
    i32 = dict(dtype=torch.int32, device="cuda")
    return dict(group_indices=torch.full((num_experts + 1,), -3, **i32),
                perm=torch.full((num_rows,), -3, dtype=torch.int64, device="cuda"),
                pad_offsets=torch.full((num_experts + 1,), -3, **i32), row_src=torch.full((rp,), -3, **i32),
                dst_row=torch.full((num_rows,), -3, **i32), mtile_expert=torch.full((rp // 128,), -3, **i32),
                tile_pairs=torch.full((rp // 128 + num_experts + 1,), -3, **i32), num_mtiles=torch.full((4,), -3, **i32),
                status=torch.zeros(1, **i32))


def _run_both(idx, num_experts, native):
    flat = idx.reshape(-1).contiguous().cuda()
    a = _outputs(flat.numel(), num_experts, native)
    b = _outputs(flat.numel(), num_experts, native)
    ws = torch.empty(native.routing_workspace_bytes(flat.numel(), num_experts), dtype=torch.uint8, device="cuda")
    native.routing_metadata(flat, num_experts, a["group_indices"], a["perm"], a["pad_offsets"], a["row_src"],
                            a["dst_row"], a["mtile_expert"], a["tile_pairs"], a["num_mtiles"], a["status"], ws)
    native.routing_metadata_static(flat, num_experts, b["group_indices"], b["perm"], b["pad_offsets"], b["row_src"],
                                   b["dst_row"], b["mtile_expert"], b["tile_pairs"], b["num_mtiles"], b["status"])
    torch.cuda.synchronize()
    n, pairs = a["num_mtiles"].tolist()[:2]
    assert a["num_mtiles"].tolist() == b["num_mtiles"].tolist()
    assert torch.equal(a["tile_pairs"][:pairs], b["tile_pairs"][:pairs])
    bound = a["mtile_expert"].numel()
    assert torch.equal(a["tile_pairs"][bound:], b["tile_pairs"][bound:])   # per-expert pair prefix
    for key in ("group_indices", "perm", "pad_offsets", "dst_row", "status"):
        assert torch.equal(a[key], b[key]), key
    assert torch.equal(a["row_src"][: n * 128], b["row_src"][: n * 128])
    assert torch.equal(a["mtile_expert"][:n], b["mtile_expert"][:n])
    # and the result is the stable sort
    assert torch.equal(b["perm"], torch.sort(flat, stable=True).indices)


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(native):
    g = torch.Generator().manual_seed(21)
    first = torch.topk(torch.randn(16384, 60, generator=g), 4, dim=-1, sorted=False).indices     # 65536 rows, 60 experts
    second = torch.topk(torch.randn(777, 256, generator=g), 8, dim=-1, sorted=False).indices    # smaller, other E
    _run_both(first, 60, native)
    _run_both(second, 256, native)   # reuses whatever the first call left in the scratch
    _run_both(first, 60, native)


def test_static_scratch_entry_rejects_oversized_problems(native):
    lib = native.load()
    limit = lib.moe_routing_static_scratch_bytes()
    assert limit == 1 << 20
    assert native.routing_workspace_bytes(524288, 256) <= limit
    rows, experts = 524288 + 1024, 256
    assert native.routing_workspace_bytes(rows, experts) > limit
    idx = torch.zeros(rows, dtype=torch.int64, device="cuda")
    out = _outputs(rows, experts, native)
    with pytest.raises(native.MoeNativeError, match="built-in scratch holds"):
        native.routing_metadata_static(idx, experts, out["group_indices"], out["perm"], out["pad_offsets"],
                                       out["row_src"], out["dst_row"], out["mtile_expert"], out["tile_pairs"],
                                       out["num_mtiles"], out["status"])
