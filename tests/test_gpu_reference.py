"""Pins the CPU oracle against the REFERENCE's own kernels, run on the GPU through the harness in
oracle/ref_harness.cu (built from the reference sources where they lie into oracle/_ref/, never
committed). The oracle runs in the reference's summation order (ORDER_REF). Skipped when the
harness binary is absent (the reference tree was not available when the oracle was built).

Safety: the reference's pruning code dereferences unfilled beam slots as data rows
(graph_kernel.cuh:92,104), so its build and refine kernels are launched only on inputs for which
the oracle reports that every beam ended full."""
import numpy as np
import pytest
import torch

import helpers
import oracle
from oracle import ref
from glide_b200 import api

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF

if not ref.available():
    pytest.skip("oracle/_ref/libglide_ref.so not built", allow_module_level=True)

CASES = {
    "uniform32": dict(kind="uniform", n=4000, dim=32, nq=200, metric=oracle.EUCLIDEAN),
    "int128": dict(kind="int", n=4000, dim=128, nq=200, metric=oracle.EUCLIDEAN),   # exact distance ties occur
    "unit96": dict(kind="unit", n=3000, dim=96, nq=150, metric=oracle.COSINE),
    "uniform30": dict(kind="uniform", n=3000, dim=30, nq=100, metric=oracle.EUCLIDEAN),
}
_cache = {}


def case(name):
    if name not in _cache:
        c = CASES[name]
        base, queries = helpers.small_dataset(c["kind"], c["n"], c["dim"], c["nq"], seed=31)
        P = helpers.oracle_pipeline(base, metric=c["metric"], order=oracle.ORDER_REF, route_order=oracle.ORDER_REF,
                                    centroid_num=3)
        _cache[name] = (base, queries, P)
    return _cache[name]


def dev(ctx, a):
    a = np.ascontiguousarray(a)
    return api.from_u32(ctx, a) if a.dtype == np.uint32 else torch.from_numpy(a).to(ctx.torch_device)


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("beam", [32, 64, 100, 200])
def test_reference_search_kernel_equals_oracle(gpu_ctx, name, beam):
    base, queries, P = case(name)
    o = oracle.SearchParams.derive(beam, 16, top_k=10)
    want_ids, want_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o, P["metric"],
                                     order=oracle.ORDER_REF, route_order=oracle.ORDER_REF)
    d_ids = api._u32_tensor(gpu_ctx, want_ids.shape)
    d_d = gpu_ctx.empty(want_d.shape, torch.float32)
    t = [dev(gpu_ctx, x) for x in (base, P["graph"], P["centroids"], P["orig_sp"], queries)]
    torch.cuda.synchronize()
    rc = ref.search(t[0].data_ptr(), base.shape[1], t[1].data_ptr(), 16, t[2].data_ptr(), P["centroids"].shape[0],
                    t[3].data_ptr(), t[4].data_ptr(), queries.shape[0], o, P["metric"], d_ids.data_ptr(), d_d.data_ptr())
    assert rc == 0
    assert np.array_equal(api.to_u32(d_ids), want_ids)
    assert np.array_equal(d_d.cpu().numpy(), want_d)


@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_define_partition_equals_oracle(gpu_ctx, name):
    base, _, P = case(name)
    n, C = base.shape[0], P["centroids"].shape[0]
    want_index, _, want_len = oracle.define_partition(base, P["centroids"], 1.1, P["metric"], oracle.ORDER_REF)
    d_len = api._u32_tensor(gpu_ctx, (C + 1,))
    d_index = api._u32_tensor(gpu_ctx, (n, 3))
    d_base, d_cent = dev(gpu_ctx, base), dev(gpu_ctx, P["centroids"])
    torch.cuda.synchronize()
    assert ref.define_partition(d_base.data_ptr(), n, base.shape[1], d_cent.data_ptr(), C, 1.1, P["metric"],
                                d_len.data_ptr(), d_index.data_ptr()) == 0
    got, got_len = api.to_u32(d_index), api.to_u32(d_len)
    assert np.array_equal(got_len, want_len)
    assert np.array_equal(got[:, 0], want_index[:, 0])                                   # nearest centroid
    assert np.array_equal(got[:, 2] != INVALID, want_index[:, 2] != INVALID)             # boundary test
    for c in range(C):  # slots come from atomics: a permutation of 0..len-1 inside every segment
        assert sorted(got[got[:, 0] == c, 1].tolist()) == list(range(int(want_len[c])))
    assert sorted(got[got[:, 2] != INVALID, 2].tolist()) == list(range(int(want_len[C])))


def _full_beams(P, base, beam_build):
    n = base.shape[0]
    _, counters = oracle.build_rows(P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                                    P["mapping"], n, 16, P["p_build"], P["alpha"], P["metric"], oracle.ORDER_REF,
                                    want_counters=True)
    sizes = np.zeros(P["reorder_data"].shape[0] - n, np.uint64)
    g = P["after_build"].copy()
    if sizes.size:
        oracle.build_boundary(P["reorder_data"], P["knn"].view(np.uint32), n, int(P["local_sp"][-1]), P["mapping"], g,
                              P["p_build"], P["alpha"], P["metric"], oracle.ORDER_REF, pool_sizes=sizes)
    return bool((counters[:, 3] == beam_build).all() and (sizes == beam_build).all())


@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_build_and_boundary_kernels_equal_oracle(gpu_ctx, name):
    base, _, P = case(name)
    if not _full_beams(P, base, P["p_build"].beam):
        pytest.skip("a beam stayed unfilled: the reference kernel would read out of bounds")
    n = base.shape[0]
    t = [dev(gpu_ctx, x) for x in (P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                                   P["mapping"])]
    for with_boundary, want in ((False, P["after_build"]), (True, P["after_boundary"])):
        g = api._u32_tensor(gpu_ctx, (n, 16)); g.fill_(-1)
        torch.cuda.synchronize()
        rc = ref.build(t[0].data_ptr(), P["reorder_data"].shape[0], base.shape[1], t[1].data_ptr(), 16, t[2].data_ptr(),
                       t[3].data_ptr(), len(P["seg_start"]), t[4].data_ptr(), t[5].data_ptr(), n, 16, P["p_build"], P["alpha"],
                       P["metric"], with_boundary, g.data_ptr())
        assert rc == 0
        assert np.array_equal(api.to_u32(g), want)


@pytest.mark.parametrize("name", ["uniform32", "int128"])
def test_reference_reverse_is_one_of_the_orders_the_oracle_allows(gpu_ctx, name):
    base, _, P = case(name)
    before, want = P["after_boundary"], P["after_reverse"]
    g = dev(gpu_ctx, before)
    torch.cuda.synchronize()
    assert ref.reverse(g.data_ptr(), before.shape[0], 16) == 0
    got = api.to_u32(g)
    kept = before != INVALID
    assert np.array_equal(got[kept], before[kept])
    same_rows = (got == want).all(axis=1).mean()
    for p in range(before.shape[0]):
        new = got[p][(before[p] == INVALID) & (got[p] != INVALID)]
        for s in new:                      # every inserted id is a true missing reverse edge
            assert p in before[s] and s not in before[p]
        assert len(new) == ((before[p] == INVALID) & (want[p] != INVALID)).sum()   # as many as the oracle inserts
    assert same_rows > 0.9   # rows differ only where more reverse edges compete than there are holes


@pytest.mark.parametrize("name", ["uniform32", "int128"])
def test_reference_refine_matches_oracle_up_to_its_in_place_race(gpu_ctx, name):
    """The reference refines rows in place while other CTAs traverse them (graph_kernel.cuh:648); the
    oracle reads the graph as it was before. To keep that race rare, holes are punched into a sparse
    subset of the rows of a finished graph: a search then seldom crosses a row that was just refined."""
    base, _, P = case(name)
    n = base.shape[0]
    rng = np.random.default_rng(3)
    start = P["graph"].copy()
    full_rows = np.nonzero((start != INVALID).all(axis=1))[0]
    chosen = rng.choice(full_rows, size=min(120, full_rows.size), replace=False)
    start[chosen, 12:] = INVALID
    start[(start == INVALID).any(axis=1) & ~np.isin(np.arange(n), chosen)] = start[full_rows[0]]  # no other holes
    sizes = np.zeros(n, np.uint64)
    want = oracle.refine(base, start, P["centroids"], P["orig_sp"], P["p_refine"], P["alpha"], P["metric"],
                         oracle.ORDER_REF, route_order=oracle.ORDER_REF, pool_sizes=sizes)
    if not (sizes == P["p_refine"].beam).all():
        pytest.skip("a beam stayed unfilled: the reference kernel would read out of bounds")
    g = dev(gpu_ctx, start)
    t = [dev(gpu_ctx, x) for x in (base, P["centroids"], P["orig_sp"])]
    torch.cuda.synchronize()
    assert ref.refine(t[0].data_ptr(), n, base.shape[1], g.data_ptr(), 16, t[1].data_ptr(), P["centroids"].shape[0],
                      t[2].data_ptr(), P["p_refine"], P["alpha"], P["metric"]) == 0
    got = api.to_u32(g)
    kept = start != INVALID
    assert np.array_equal(got[kept], start[kept])                  # existing edges are never touched
    untouched = ~np.isin(np.arange(n), chosen)
    assert np.array_equal(got[untouched], start[untouched])        # rows without holes stay as they were
    assert (got[chosen] == want[chosen]).all(axis=1).mean() > 0.9  # refined rows agree up to the race
