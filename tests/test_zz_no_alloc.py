"""The allocation-free search entry point against the regular one.

`glide_search_static_scratch` serves hosts that may not allocate device memory at call time
(their memory comes from a pool handed out once, and a cudaMalloc in the serving loop would
stall the whole device). It must return exactly what `glide_search` returns. The file name keeps
it last in collection order, so a run that stops at the first failure has already run every
other test; it builds its own small index, so it also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers
from glide_b200 import api
from glide_b200.params import SearchParameter

pytestmark = pytest.mark.gpu


def _search(ctx, fn, d_base, d_graph, d_cent, d_sp, d_q, sp):
    q = d_q.shape[0]
    d_ids = api._u32_tensor(ctx, (q, sp.top_k))
    d_d = ctx.empty((q, sp.top_k), torch.float32)
    pc = api._params_c(sp)
    ctx.sync_inputs()
    rc = fn(ctx.handle, d_base.data_ptr(), d_base.shape[0], d_base.shape[1], d_graph.data_ptr(), d_graph.shape[1],
            d_cent.data_ptr(), d_cent.shape[0], d_sp.data_ptr(), d_q.data_ptr(), q, C.byref(pc), 0,
            d_ids.data_ptr(), d_d.data_ptr())
    return rc, api.to_u32(d_ids), d_d.cpu().numpy()


def test_static_scratch_search_equals_regular_search_twice(gpu_ctx):
    ctx = gpu_ctx
    base, queries = helpers.small_dataset("int", 3000, 64, 300, seed=21)
    P = helpers.oracle_pipeline(base)
    dev = lambda a: api.from_u32(ctx, a) if a.dtype == np.uint32 else torch.from_numpy(a).to(ctx.torch_device)
    d_base, d_graph, d_cent, d_sp = dev(base), dev(P["graph"]), dev(P["centroids"]), dev(P["orig_sp"])
    sp = SearchParameter(top_k=10, beam=64).derive(16)
    lib = ctx.lib
    # two calls in a row on different batches: the shared scratch keeps the first call's contents
    for batch in (queries[:300], queries[40:170]):
        d_q = dev(np.ascontiguousarray(batch))
        rc_a, ids_a, d_a = _search(ctx, lib.glide_search, d_base, d_graph, d_cent, d_sp, d_q, sp)
        rc_b, ids_b, d_b = _search(ctx, lib.glide_search_static_scratch, d_base, d_graph, d_cent, d_sp, d_q, sp)
        assert rc_a == 0 and rc_b == 0, lib.glide_last_error(ctx.handle)
        assert np.array_equal(ids_a, ids_b)   # bit-exact, like every id/distance comparison in this suite
        assert np.array_equal(d_a, d_b)
    # a batch beyond the fixed capacity is refused with a message, and the context stays usable
    big = torch.zeros((65537, base.shape[1]), dtype=torch.float32, device=ctx.torch_device)
    rc, _, _ = _search(ctx, lib.glide_search_static_scratch, d_base, d_graph, d_cent, d_sp, big, sp)
    assert rc == -2 and b"65536" in lib.glide_last_error(ctx.handle)
    rc, ids, _ = _search(ctx, lib.glide_search_static_scratch, d_base, d_graph, d_cent, d_sp, dev(queries[:8].copy()), sp)
    assert rc == 0 and ids.shape == (8, 10)


def test_static_scratch_search_allocates_nothing():
    """What the entry point's name promises: on a context that has never grown its scratch arena,
    a call leaves the arena at zero bytes and the device's free memory where it was."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    base, queries = helpers.small_dataset("int", 2000, 64, 200, seed=22)
    P = helpers.oracle_pipeline(base)
    ctx = api.Context(0)     # a fresh context: no earlier call has allocated scratch on it
    try:
        dev = lambda a: api.from_u32(ctx, a) if a.dtype == np.uint32 else torch.from_numpy(a).to(ctx.torch_device)
        d_base, d_graph, d_cent, d_sp = dev(base), dev(P["graph"]), dev(P["centroids"]), dev(P["orig_sp"])
        d_q = dev(queries)
        sp = SearchParameter(top_k=10, beam=64).derive(16)
        lib = ctx.lib
        assert lib.glide_ctx_workspace_bytes(ctx.handle) == 0
        # the first call resolves the array's address and loads the kernels; measure around the second
        rc, ids_0, _ = _search(ctx, lib.glide_search_static_scratch, d_base, d_graph, d_cent, d_sp, d_q, sp)
        assert rc == 0, lib.glide_last_error(ctx.handle)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(ctx.torch_device)
        q = d_q.shape[0]
        d_ids = api._u32_tensor(ctx, (q, sp.top_k))
        d_d = ctx.empty((q, sp.top_k), torch.float32)
        pc = api._params_c(sp)
        torch.cuda.synchronize()
        free_mid, _ = torch.cuda.mem_get_info(ctx.torch_device)   # the output tensors are the caller's, taken before
        rc = lib.glide_search_static_scratch(ctx.handle, d_base.data_ptr(), d_base.shape[0], d_base.shape[1],
                                             d_graph.data_ptr(), d_graph.shape[1], d_cent.data_ptr(), d_cent.shape[0],
                                             d_sp.data_ptr(), d_q.data_ptr(), q, C.byref(pc), 0, d_ids.data_ptr(),
                                             d_d.data_ptr())
        assert rc == 0, lib.glide_last_error(ctx.handle)
        free_after, _ = torch.cuda.mem_get_info(ctx.torch_device)
        assert free_after == free_mid <= free_before
        assert lib.glide_ctx_workspace_bytes(ctx.handle) == 0
        assert np.array_equal(api.to_u32(d_ids), ids_0)
        # the regular entry point does grow the arena (that is the difference between the two)
        rc, ids_1, _ = _search(ctx, lib.glide_search, d_base, d_graph, d_cent, d_sp, d_q, sp)
        assert rc == 0 and np.array_equal(ids_1, ids_0)
        assert lib.glide_ctx_workspace_bytes(ctx.handle) > 0
    finally:
        ctx.close()
