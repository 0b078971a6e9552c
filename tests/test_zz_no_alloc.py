"""The allocation-free routing-plan entry point against the ordinary one.

pnv_dispatch_plan_noalloc keeps its scratch in an array inside the library, for callers that cannot ask
the driver for memory when the plan is needed (a server whose own arena already owns the GPU, a loop that
cannot afford cudaMalloc's device-wide stall).  Both entry points are called through the C ABI on the same
inputs; the results must be identical.  Two calls in a row with different routings show that whatever the
first call left in the shared scratch does not leak into the second.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan(lib, check, fn_noalloc, ids, first, E, cap):
    T, topk = ids.shape
    i32 = dict(dtype=torch.int32, device="cuda")
    outs = [torch.full((E,), -7, **i32), torch.full((T * topk,), -7, **i32), torch.full((E * cap,), -7, **i32),
            torch.full((E * cap,), -7, **i32)]
    stream = torch.cuda.current_stream().cuda_stream
    args = [ids.data_ptr(), 1, T, topk, first, E, cap] + [o.data_ptr() for o in outs]
    if fn_noalloc:
        check(lib.pnv_dispatch_plan_noalloc(*args, stream))
        keep = None
    else:
        n = int(lib.pnv_dispatch_plan_scratch_ints(T * topk, E))
        keep = torch.empty((max(n, 1),), **i32)
        check(lib.pnv_dispatch_plan(*args, keep.data_ptr(), stream))
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in outs]


def test_noalloc_plan_matches_plan_with_caller_scratch_twice():
    from paired_nvfp4_kernels import _cabi
    lib, check = _cabi.lib, _cabi.check
    assert lib.pnv_dispatch_plan_noalloc_max_scratch_ints() == 65536
    E, cap, topk = 64, 96, 8
    for call, (T, seed) in enumerate([(4096, 11), (1500, 12)]):   # 32 chunks, then 12: stale totals stay behind
        rng = np.random.default_rng(seed)
        ids = torch.from_numpy(np.argsort(-rng.standard_normal((T, 96)), axis=1)[:, :topk].astype(np.int64)).cuda()
        want = _plan(lib, check, False, ids, 16, E, cap)
        got = _plan(lib, check, True, ids, 16, E, cap)
        for name, g, w in zip(("counts", "route_dest", "src_tok", "src_route"), got, want):
            assert np.array_equal(g, w), f"call {call}: {name} differs"
        assert want[0].sum() > 0 and (want[1] == -1).any()


def test_noalloc_plan_rejects_oversized_plans():
    from paired_nvfp4_kernels import _cabi
    lib = _cabi.lib
    T, topk, E = 40000, 8, 512       # 313 chunks x 512 experts = 160256 ints > 65536
    ids = torch.zeros((T, topk), dtype=torch.int64, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    outs = [torch.zeros((E,), **i32), torch.zeros((T * topk,), **i32), torch.zeros((E * 4,), **i32),
            torch.zeros((E * 4,), **i32)]
    rc = lib.pnv_dispatch_plan_noalloc(ids.data_ptr(), 1, T, topk, 0, E, 4, *[o.data_ptr() for o in outs],
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    msg = lib.pnv_last_error().decode()
    assert "65536" in msg and "scratch" in msg


def test_noalloc_plan_at_the_limit_and_without_allocating():
    """64 segments x 1024 local experts use the built-in scratch to its last int.  With every buffer made
    beforehand and one warm-up call done (the first call on a device looks up the scratch address), neither
    the driver's free-memory figure nor torch's allocator may move across the call."""
    from paired_nvfp4_kernels import _cabi
    lib, check = _cabi.lib, _cabi.check
    T, topk, E, cap = 8192, 8, 1024, 80
    assert lib.pnv_dispatch_plan_scratch_ints(T * topk, E) == lib.pnv_dispatch_plan_noalloc_max_scratch_ints()
    rng = np.random.default_rng(5)
    ids = torch.from_numpy(rng.integers(0, E + 64, (T, topk)).astype(np.int64)).cuda()   # some ids are not local
    want = _plan(lib, check, False, ids, 0, E, cap)
    i32 = dict(dtype=torch.int32, device="cuda")
    outs = [torch.full((E,), -7, **i32), torch.full((T * topk,), -7, **i32), torch.full((E * cap,), -7, **i32),
            torch.full((E * cap,), -7, **i32)]
    stream = torch.cuda.current_stream().cuda_stream
    args = [ids.data_ptr(), 1, T, topk, 0, E, cap] + [o.data_ptr() for o in outs] + [stream]
    check(lib.pnv_dispatch_plan_noalloc(*args))          # warm-up
    torch.cuda.synchronize()
    free0, allocated0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    check(lib.pnv_dispatch_plan_noalloc(*args))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.memory_allocated() == allocated0 and torch.cuda.memory_reserved() == reserved0
    for name, g, w in zip(("counts", "route_dest", "src_tok", "src_route"), outs, want):
        g = g.cpu().numpy()
        if name.startswith("src"):
            assigned = w != -7
            assert np.array_equal(g[assigned], w[assigned]), name
        else:
            assert np.array_equal(g, w), name
