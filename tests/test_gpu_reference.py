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


def test_reference_kernels_at_scale_same_results_and_device_time(gpu_ctx, capsys):
    """The reference's kernels and this library's on the same stage inputs of the 1,000,000 x 128
    integer-valued mixture (10 partitions, the reference's default parameters): results and device
    time side by side. On integer-valued rows every squared distance is an exact integer in
    fp32 whatever the summation order, so the two builds must agree bit for bit; routing uses
    fractional centroids, so a few queries in a million may enter at another partition.
    GLIDE_REF_SCALE_ROWS overrides the row count; with few rows per mixture component the beams of
    the build do not fill and the test skips, because the reference's pruning would then read out
    of bounds."""
    import json
    import os
    from glide_b200 import datasets, pipeline
    rows = int(os.environ.get("GLIDE_REF_SCALE_ROWS", "1000000"))
    spec = datasets.scaled(datasets.CONFIGS["cfg1"], rows)
    base, queries = datasets.make(spec)
    ctx = gpu_ctx
    d_base, d_q = dev(ctx, base), dev(ctx, queries)
    cfg = pipeline.BuildConfig(centroid_num=10, seed=spec.seed)
    res = pipeline.build_small(ctx, d_base, cfg, keep_intermediates=True)
    seg_start, seg_len = res.h_segment_start, res.h_segment_length
    h_map = api.to_u32(res.d_map)
    local, original = api.start_point_select(seg_start, seg_len, h_map, cfg.seed)
    d_local, d_sp = api.from_u32(ctx, local), api.from_u32(ctx, original)
    d_seg_start, d_seg_len = api.from_u32(ctx, seg_start), api.from_u32(ctx, seg_len)
    p_knn, p_refine = pipeline.derive_build_search_params(cfg)
    n, dim, deg = rows, base.shape[1], cfg.graph_degree
    report = {"rows": rows, "dim": dim, "partitions": 10, "degree": deg}

    # ---- subgraph build + boundary merge ----
    ours = api._u32_tensor(ctx, (n, deg)); ours.fill_(-1)
    ctx.enable_counters(True)
    t_ours = api.subgraph_build_and_merge(ctx, res.d_reorder_data, res.d_knn, seg_start, seg_len, d_local, res.d_map, n,
                                          ours, p_knn, cfg.relaxant_factor)
    short = ctx.read_counters()[3]
    ctx.enable_counters(False)
    if short:
        pytest.skip("a beam stayed unfilled: the reference kernel would read out of bounds")
    theirs = api._u32_tensor(ctx, (n, deg)); theirs.fill_(-1)
    torch.cuda.synchronize()
    assert ref.build(res.d_reorder_data.data_ptr(), res.d_reorder_data.shape[0], dim, res.d_knn.data_ptr(), cfg.knn_degree,
                     d_seg_start.data_ptr(), d_seg_len.data_ptr(), len(seg_start), d_local.data_ptr(), res.d_map.data_ptr(),
                     n, deg, p_knn, cfg.relaxant_factor, 0, True, theirs.data_ptr()) == 0
    report["subgraph_build_and_merge"] = {"reference_s": ref.last_seconds(), "ours_s": t_ours}
    assert torch.equal(ours, theirs)

    # ---- reverse edges ----
    t_ours = api.reverse_graph(ctx, ours)
    torch.cuda.synchronize()
    assert ref.reverse(theirs.data_ptr(), n, deg) == 0
    report["reverse_graph"] = {"reference_s": ref.last_seconds(), "ours_s": t_ours}
    # the reference's insertion order comes from atomics; hole counts per row must agree
    assert torch.equal((ours == -1).sum(dim=1), (theirs == -1).sum(dim=1))

    # ---- refine (both from this library's reverse result) ----
    theirs.copy_(ours)
    before = ours.clone()
    ctx.enable_counters(True)
    t_ours = api.refine(ctx, d_base, ours, res.index.centroid_view(), d_sp, p_refine, cfg.relaxant_factor)
    short = ctx.read_counters()[3]
    ctx.enable_counters(False)
    if not short:
        torch.cuda.synchronize()
        assert ref.refine(d_base.data_ptr(), n, dim, theirs.data_ptr(), deg, res.index.centroid_view().data_ptr(), 10,
                          d_sp.data_ptr(), p_refine, cfg.relaxant_factor, 0) == 0
        report["refine"] = {"reference_s": ref.last_seconds(), "ours_s": t_ours,
                            "rows_equal": float((ours == theirs).all(dim=1).float().mean())}
        # The reference refines in place while other CTAs traverse the rows, and after the reverse
        # step nearly every row has holes, so at this size its rows depend on the schedule; what
        # must hold for both: existing edges untouched, holes filled equally often.
        kept = before != -1
        assert torch.equal(ours[kept], before[kept]) and torch.equal(theirs[kept], before[kept])
        report["refine"]["filled_ours"] = float((ours != -1).float().mean())
        report["refine"]["filled_reference"] = float((theirs != -1).float().mean())
        sp = pipeline.derive_search_params(64, deg)
        gt0 = api.to_u32(api.bruteforce_knn(ctx, d_base, d_q, 10)[0])
        for name, g in (("ours", ours), ("reference", theirs)):
            ids = api.search(ctx, d_base, g, res.index.centroid_view(), d_sp, d_q, sp)[0]
            report["refine"]["recall_beam64_on_" + name + "_graph"] = api.calculate_recall(api.to_u32(ids), gt0, 10)

    # ---- search on this library's finished index, equal beam ----
    gt = api.to_u32(api.bruteforce_knn(ctx, d_base, d_q, 10)[0])
    report["search"] = []
    for beam in (32, 64, 128):
        sp = pipeline.derive_search_params(beam, deg)
        ids, dists, t_ours = api.search(ctx, d_base, ours, res.index.centroid_view(), d_sp, d_q, sp)
        for _ in range(3):
            _, _, t_ours = api.search(ctx, d_base, ours, res.index.centroid_view(), d_sp, d_q, sp)
        r_ids = api._u32_tensor(ctx, ids.shape)
        r_d = ctx.empty(dists.shape, torch.float32)
        for _ in range(4):
            torch.cuda.synchronize()
            assert ref.search(d_base.data_ptr(), dim, ours.data_ptr(), deg, res.index.centroid_view().data_ptr(), 10,
                              d_sp.data_ptr(), d_q.data_ptr(), queries.shape[0], sp, 0, r_ids.data_ptr(), r_d.data_ptr()) == 0
        same = float((ids == r_ids).all(dim=1).float().mean())
        report["search"].append({"beam": beam, "reference_qps": queries.shape[0] / ref.last_seconds(),
                                 "ours_qps": queries.shape[0] / t_ours, "queries_equal": same,
                                 "recall_ours": api.calculate_recall(api.to_u32(ids), gt, 10),
                                 "recall_reference": api.calculate_recall(api.to_u32(r_ids), gt, 10)})
        assert same > 0.999
    with capsys.disabled():
        print("\nREFERENCE_KERNELS_AT_SCALE " + json.dumps(report))
