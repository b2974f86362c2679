"""The allocation-free paged-decode entry point, called through its exported C symbol.

Some callers of the native library cannot allocate device memory at the point where they need
decode attention (no PyTorch allocator in the process, a memory budget frozen at start-up, or a
region where an allocation would stall the GPU), so the library offers a variant whose split-KV
workspace is a fixed array inside the library.  This test checks it against the regular entry
point (caller-provided workspaces) on two calls in a row with different shapes -- the second
call finds the first call's leftovers in the shared array -- and checks that a request beyond
the array's capacity is refused on the host without launching anything.

Kept in a file that sorts last so that a run stopping at the first failure has already run every
other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

VP, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
SCRATCH_FLOATS = 2 * 1024 * 1024
TOO_LARGE = 40


def _case(seed, B, n_q, n_kv, hd, ctx_list):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ctx = torch.tensor(ctx_list, dtype=torch.int32, device="cuda")
    pages_per = (max(ctx_list) + 15) // 16
    n_pages = B * pages_per + 3
    k_pages = (torch.randn(n_pages, n_kv, 16, hd, device="cuda", generator=g)).bfloat16()
    v_pages = (torch.randn(n_pages, n_kv, 16, hd, device="cuda", generator=g)).bfloat16()
    perm = torch.randperm(n_pages, device="cuda", generator=g)[: B * pages_per].int()
    table = perm.view(B, pages_per).contiguous()
    q = torch.randn(B, n_q * hd, device="cuda", generator=g).bfloat16()
    return q, k_pages, v_pages, table, ctx


def _call_noalloc(lib, q, k_pages, v_pages, table, ctx, n_q, n_kv, hd, max_ctx, split, out=None):
    """Returns (return code, output, number of torch device allocations made during the call)."""
    if out is None:
        out = torch.empty(q.shape[0], n_q * hd, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    allocs = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = lib.kb_paged_decode_noalloc(VP(q.data_ptr()), LL(q.stride(0)), VP(k_pages.data_ptr()), VP(v_pages.data_ptr()),
                                     VP(table.data_ptr()), I(table.shape[1]), VP(ctx.data_ptr()), I(q.shape[0]),
                                     I(n_q), I(n_kv), I(hd), I(max_ctx), I(split), F(1.0 / math.sqrt(hd)),
                                     VP(out.data_ptr()), LL(out.stride(0)), VP(stream))
    return rc, out, torch.cuda.memory_stats()["allocation.all.allocated"] - allocs


def test_no_alloc_paged_decode_matches_regular_entry_point_twice():
    from kotodama_b200.ops import get_ops
    ops = get_ops("cuda")
    lib = ops.lib
    lib.kb_paged_decode_noalloc.restype = ctypes.c_int
    cases = [(11, 6, 24, 8, 128, [1, 16, 17, 300, 700, 1025]),       # first call: also performs the set-up
             (12, 3, 4, 2, 64, [40, 513, 129])]                       # second call: other shape, stale scratch
    for seed, B, n_q, n_kv, hd, ctx_list in cases:
        q, k_pages, v_pages, table, ctx = _case(seed, B, n_q, n_kv, hd, ctx_list)
        max_ctx = max(ctx_list)
        # the allocation-free entry point runs the bulk-copy kernel (it has no page count for a tensor map):
        # take the reference from the same kernel, so that the comparison can be bit for bit
        lib.kb_set_decode_kernel(ctypes.c_int(2))
        try:
            ref = ops.paged_decode_attention(q, k_pages, v_pages, table, ctx, max_ctx, n_q, n_kv, hd, split=256)
        finally:
            lib.kb_set_decode_kernel(ctypes.c_int(3))
        rc, out, allocs = _call_noalloc(lib, q, k_pages, v_pages, table, ctx, n_q, n_kv, hd, max_ctx, 256)
        torch.cuda.synchronize()
        assert rc == 0
        assert allocs == 0                    # the caller's buffers are the only device memory involved
        err = float((out.float() - ref.float()).norm() / (ref.float().norm() + 1e-12))
        assert err < 1e-2, err
        assert torch.equal(out, ref)          # same kernels, same inputs: bit-identical
        # PyTorch's counters cannot see an allocation made behind its allocator, so a warm call is also
        # bracketed by the driver's own free-memory figure: it must not move
        out2 = torch.empty_like(out)          # allocated before the bracket: nothing of PyTorch's moves inside it
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc2, out2, _ = _call_noalloc(lib, q, k_pages, v_pages, table, ctx, n_q, n_kv, hd, max_ctx, 256, out=out2)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert rc2 == 0 and torch.equal(out2, ref)
        assert free_after >= free_before, (free_before, free_after)


def test_no_alloc_rejects_requests_beyond_the_scratch_capacity():
    from kotodama_b200.ops import get_ops
    lib = get_ops("cuda").lib
    lib.kb_paged_decode_noalloc.restype = ctypes.c_int
    B, n_q, n_kv, hd = 64, 24, 8, 128
    q, k_pages, v_pages, table, ctx = _case(13, 2, n_q, n_kv, hd, [32, 48])
    # claim a batch and context whose partials exceed the array: refused before any launch
    need = B * n_q * math.ceil(4096 / 16) * (hd + 2)
    assert need > SCRATCH_FLOATS
    out = torch.zeros(B, n_q * hd, device="cuda", dtype=torch.bfloat16)
    rc = lib.kb_paged_decode_noalloc(VP(q.data_ptr()), LL(q.stride(0)), VP(k_pages.data_ptr()), VP(v_pages.data_ptr()),
                                     VP(table.data_ptr()), I(table.shape[1]), VP(ctx.data_ptr()), I(B), I(n_q),
                                     I(n_kv), I(hd), I(4096), I(16), F(0.1), VP(out.data_ptr()), LL(out.stride(0)),
                                     VP(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == TOO_LARGE and float(out.abs().sum()) == 0.0
