"""GPU parity tests: every CUDA stage, called through the C ABI, against the CPU oracle on the
same seeded inputs. Ids are compared bit for bit; distances bit for bit too, because the
oracle restates the kernels' summation order (a tolerance of 1e-5 relative is what the
reference's own order differs by and is asserted separately)."""
import numpy as np
import pytest
import torch

import helpers
import oracle
from glide_b200 import api
from glide_b200.params import Metric, NNDescentParameter, SearchParameter

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


def dev(ctx, a, dtype=None):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        return api.from_u32(ctx, a)
    return torch.from_numpy(a).to(ctx.torch_device)


def sp_from(o: oracle.SearchParams) -> SearchParameter:
    return SearchParameter(top_k=o.top_k, beam=o.beam, max_iterations=o.max_iterations,
                           min_iterations=o.min_iterations, hash_bit=o.hash_bit,
                           hash_reset_interval=o.hash_reset_interval)


CASES = {
    "uniform16": dict(kind="uniform", n=3000, dim=16, nq=200, metric=oracle.EUCLIDEAN),
    "int128": dict(kind="int", n=3000, dim=128, nq=200, metric=oracle.EUCLIDEAN),     # exact ties occur
    "unit96": dict(kind="unit", n=2500, dim=96, nq=150, metric=oracle.COSINE),
    "uniform30": dict(kind="uniform", n=1500, dim=30, nq=100, metric=oracle.EUCLIDEAN),  # dim % 4 != 0
    "scaled960": dict(kind="scaled", n=1200, dim=960, nq=60, metric=oracle.EUCLIDEAN),   # wide rows (generic row path)
    "uniform200": dict(kind="uniform", n=1500, dim=200, nq=80, metric=oracle.EUCLIDEAN),  # 50 chunks: partial second round
}
_cache = {}


def case(name):
    if name not in _cache:
        c = CASES[name]
        base, queries = helpers.small_dataset(c["kind"], c["n"], c["dim"], c["nq"])
        P = helpers.oracle_pipeline(base, metric=c["metric"])
        _cache[name] = (base, queries, P)
    return _cache[name]


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("beam", [32, 64, 100, 256, 300, 512])   # above 256: the reference's two-warp merge order
def test_search_matches_oracle(gpu_ctx, name, beam):
    base, queries, P = case(name)
    metric = P["metric"]
    o = oracle.SearchParams.derive(beam, P["graph"].shape[1], top_k=10)
    want_ids, want_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o, metric)
    d_ids, d_d, _ = api.search(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, P["graph"]), dev(gpu_ctx, P["centroids"]),
                               dev(gpu_ctx, P["orig_sp"]), dev(gpu_ctx, queries), sp_from(o), Metric(metric))
    got_ids, got_d = api.to_u32(d_ids), d_d.cpu().numpy()
    assert np.array_equal(got_ids, want_ids)
    assert np.array_equal(got_d, want_d)
    # and within 1e-5 relative of the reference's own summation order
    ref_ids, ref_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o, metric,
                                   order=oracle.ORDER_REF)
    same = (ref_ids == got_ids)
    assert same.mean() > 0.99
    assert np.allclose(got_d[same], ref_d[same], rtol=1e-5)


# Adjacency rows wider than 32 entries take the shared-memory candidate path (beam_loop) in the
# search, build and refine kernels; the cases above (degree 16) never reach it. 64 is the 960-dim
# benchmark configuration's degree (with a kNN degree of 64), 48 a ragged width (one and a half
# 32-lane rounds).
WIDE_CASES = {
    "scaled960_d64": dict(kind="scaled", n=1500, dim=960, nq=60, metric=oracle.EUCLIDEAN, degree=64),
    "unit96_d48": dict(kind="unit", n=2500, dim=96, nq=100, metric=oracle.COSINE, degree=48),
    "int128_d64": dict(kind="int", n=3000, dim=128, nq=150, metric=oracle.EUCLIDEAN, degree=64),   # exact ties occur
}


def wide_case(name):
    key = "wide:" + name
    if key not in _cache:
        c = WIDE_CASES[name]
        base, queries = helpers.small_dataset(c["kind"], c["n"], c["dim"], c["nq"])
        P = helpers.oracle_pipeline(base, metric=c["metric"], knn_degree=c["degree"], graph_degree=c["degree"],
                                    build_beam=64, refine_beam=128)
        _cache[key] = (base, queries, P)
    return _cache[key]


@pytest.mark.parametrize("name", sorted(WIDE_CASES))
@pytest.mark.parametrize("beam", [32, 64, 100, 256, 300, 512])
def test_search_on_wide_adjacency_rows_matches_oracle(gpu_ctx, name, beam):
    base, queries, P = wide_case(name)
    metric, degree = P["metric"], P["graph"].shape[1]
    o = oracle.SearchParams.derive(beam, degree, top_k=10)
    want_ids, want_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o, metric)
    d_ids, d_d, _ = api.search(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, P["graph"]), dev(gpu_ctx, P["centroids"]),
                               dev(gpu_ctx, P["orig_sp"]), dev(gpu_ctx, queries), sp_from(o), Metric(metric))
    got_ids, got_d = api.to_u32(d_ids), d_d.cpu().numpy()
    assert np.array_equal(got_ids, want_ids)
    assert np.array_equal(got_d, want_d)
    ref_ids, ref_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o, metric,
                                   order=oracle.ORDER_REF)
    same = (ref_ids == got_ids)
    assert same.mean() > 0.99
    assert np.allclose(got_d[same], ref_d[same], rtol=1e-5)


def _widened_graph(graph, degree, seed=3):
    """The case's graph with random further neighbours up to `degree` entries per row (for the search
    any graph will do; rows stay free of duplicates and self loops)."""
    n, d0 = graph.shape
    rng = np.random.default_rng(seed)
    out = np.full((n, degree), INVALID, np.uint32)
    out[:, :d0] = graph
    for r in range(n):
        have = set(graph[r][graph[r] != INVALID].tolist()) | {r}
        extra = [int(x) for x in rng.permutation(n)[:degree] if int(x) not in have][:degree - d0]
        out[r, d0:d0 + len(extra)] = extra
    return out


@pytest.mark.parametrize("name,degree", [("int128_d64", 160), ("unit96_d48", 130), ("int128_d64", 256)])
@pytest.mark.parametrize("beam", [64, 128, 300])
def test_search_on_rows_wider_than_128_matches_oracle(gpu_ctx, name, degree, beam):
    """Adjacency rows of more than 128 entries: the reference sorts the candidates with two warps
    (search_kernel.cuh:38-95); with a beam above 256 it also merges with two (:148-233)."""
    base, queries, P = wide_case(name)
    metric = P["metric"]
    graph = _widened_graph(P["graph"], degree)
    o = oracle.SearchParams.derive(beam, degree, top_k=10)
    want_ids, want_d = oracle.search(base, graph, P["centroids"], P["orig_sp"], queries, o, metric)
    d_ids, d_d, _ = api.search(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, graph), dev(gpu_ctx, P["centroids"]),
                               dev(gpu_ctx, P["orig_sp"]), dev(gpu_ctx, queries), sp_from(o), Metric(metric))
    assert np.array_equal(api.to_u32(d_ids), want_ids)
    assert np.array_equal(d_d.cpu().numpy(), want_d)


@pytest.mark.parametrize("name", sorted(WIDE_CASES))
def test_build_stages_on_wide_rows_match_oracle(gpu_ctx, name):
    base, _, P = wide_case(name)
    metric, degree = Metric(P["metric"]), P["graph"].shape[1]
    n = base.shape[0]
    d_re, d_knn = dev(gpu_ctx, P["reorder_data"]), dev(gpu_ctx, P["knn"].view(np.uint32))
    d_map, d_local = dev(gpu_ctx, P["mapping"]), dev(gpu_ctx, P["local_sp"])
    g = api._u32_tensor(gpu_ctx, (n, degree)); g.fill_(-1)
    api.subgraph_build_and_merge(gpu_ctx, d_re, d_knn, P["seg_start"], P["seg_len"], d_local, d_map, n, g,
                                 sp_from(P["p_build"]), P["alpha"], metric)
    assert np.array_equal(api.to_u32(g), P["after_boundary"])
    api.reverse_graph(gpu_ctx, g)
    assert np.array_equal(api.to_u32(g), P["after_reverse"])
    api.refine(gpu_ctx, dev(gpu_ctx, base), g, dev(gpu_ctx, P["centroids"]), dev(gpu_ctx, P["orig_sp"]),
               sp_from(P["p_refine"]), P["alpha"], metric)
    assert np.array_equal(api.to_u32(g), P["graph"])


def test_search_host_entry_point(gpu_ctx):
    base, queries, P = case("int128")
    o = oracle.SearchParams.derive(64, 16, top_k=10)
    want_ids, want_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o)
    index = api.GLIDE(gpu_ctx, 16, base, P["centroids"])
    index.load(P["graph"], P["orig_sp"])
    ids, d = index.search_host(sp_from(o), queries)
    assert np.array_equal(ids, want_ids) and np.array_equal(d, want_d)
    ids2, d2, seconds = index.search(sp_from(o), dev(gpu_ctx, queries))
    assert np.array_equal(ids2, want_ids) and np.array_equal(d2, want_d) and seconds > 0


def test_search_pipe_gives_the_blocking_call_results_for_every_batch(gpu_ctx):
    """Batches of different sizes through a pipe of depth 3 (more batches than slots, so slots are
    reused while earlier batches are still in flight): each batch's results equal the oracle's."""
    from glide_b200 import large
    base, queries, P = case("int128")
    o = oracle.SearchParams.derive(64, 16, top_k=10)
    want_ids, want_d = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, o)
    index = api.GLIDE(gpu_ctx, 16, base, P["centroids"])
    index.load(P["graph"], P["orig_sp"])
    pipe = index.search_pipe(max_queries=queries.shape[0], max_top_k=10, depth=3)
    cuts = [(0, 7), (7, 60), (60, 61), (61, queries.shape[0]), (0, queries.shape[0]), (3, 40), (10, 11)]
    batches = []
    for lo, hi in cuts:
        hq = large.pinned_copy(queries[lo:hi])
        hi_ids, hi_d = large.pinned_empty((hi - lo, 10), np.uint32), large.pinned_empty((hi - lo, 10), np.float32)
        hi_ids.fill(7)
        batches.append((lo, hi, hq, hi_ids, hi_d, pipe.submit(sp_from(o), hq, hi_ids, hi_d)))
    assert [b[5] for b in batches] == [0, 1, 2, 0, 1, 2, 0]
    pipe.drain()
    for lo, hi, _, ids, d, _ in batches:
        assert np.array_equal(ids, want_ids[lo:hi]) and np.array_equal(d, want_d[lo:hi])
    with pytest.raises(api.GlideError):
        pipe.submit(sp_from(o), large.pinned_copy(np.zeros((queries.shape[0] + 1, base.shape[1]), np.float32)),
                    np.empty((queries.shape[0] + 1, 10), np.uint32), np.empty((queries.shape[0] + 1, 10), np.float32))
    pipe.close()


@pytest.mark.parametrize("name", ["uniform16", "int128", "unit96", "uniform30", "scaled960", "uniform200"])
def test_define_partition_and_reorder_match_oracle(gpu_ctx, name):
    base, _, P = case(name)
    metric = Metric(P["metric"])
    d_base = dev(gpu_ctx, base)
    d_seg, seg_start, seg_len = api.define_partition(gpu_ctx, d_base, dev(gpu_ctx, P["centroids"]), 1.1, metric)
    assert np.array_equal(api.to_u32(d_seg), P["seg_index"])
    assert np.array_equal(seg_start, P["seg_start"]) and np.array_equal(seg_len, P["seg_len"])
    d_re, d_map = api.reorder(gpu_ctx, d_base, d_seg, seg_start, int(seg_len[-1]))
    assert np.array_equal(api.to_u32(d_map), P["mapping"])
    assert np.array_equal(d_re.cpu().numpy(), P["reorder_data"])


def test_define_partition_without_boundary_and_single_centroid(gpu_ctx):
    base, _, P = case("uniform16")
    d_base = dev(gpu_ctx, base)
    d_seg, seg_start, seg_len = api.define_partition(gpu_ctx, d_base, dev(gpu_ctx, P["centroids"]), -1.0)
    want = oracle.define_partition(base, P["centroids"], -1.0)
    assert np.array_equal(api.to_u32(d_seg), want[0]) and seg_len[-1] == 0
    one = base.mean(axis=0, keepdims=True)
    d_seg, seg_start, seg_len = api.define_partition(gpu_ctx, d_base, dev(gpu_ctx, one), 1.1)
    assert seg_len.tolist() == [base.shape[0], 0]
    assert np.array_equal(api.to_u32(d_seg)[:, 1], np.arange(base.shape[0]))


@pytest.mark.parametrize("init", [0, 1])
@pytest.mark.parametrize("name,c", [("int128", 8), ("uniform16", 5), ("unit96", 6), ("int128", 40)])
def test_kmeans_matches_oracle(gpu_ctx, name, c, init):
    base, _, P = case(name)
    sample = base[:1200]
    want_c, want_l, want_r = oracle.kmeans(sample, c, 25, metric=P["metric"], init=init)
    d_c, d_l, rounds = api.kmeans_fit(gpu_ctx, dev(gpu_ctx, sample), c, 25, Metric(P["metric"]), init)
    assert rounds == want_r
    assert np.array_equal(api.to_u32(d_l), want_l)
    assert np.array_equal(d_c.cpu().numpy(), want_c)


@pytest.mark.parametrize("n,dim,c", [(1200, 128, 40), (70000, 128, 48), (5000, 30, 33), (150, 64, 150), (100000, 128, 24),
                                     (140000, 64, 20), (95000, 96, 20), (275000, 32, 12), (40000, 200, 16)])
def test_farthest_first_in_one_launch_equals_a_launch_per_centre(gpu_ctx, monkeypatch, n, dim, c):
    """The traversal runs as one persistent kernel (rows held in shared memory as far as they fit, then
    in registers for dimensions 32, 64, 96 and 128, then left in L2: the larger shapes here overflow
    shared memory, 40,000 x 200 has no register form) or as two launches per centre; both give the
    oracle's centres. One Lloyd round follows, so labels and centres are functions of the traversal's
    centres alone."""
    rng = np.random.default_rng(n + dim)
    sample = rng.integers(0, 50, (n, dim)).astype(np.float32)
    sample[n // 2] = sample[n // 3]   # equal rows: the lower one wins a tie
    want_c, want_l, _ = oracle.kmeans(sample, c, 1, init=1)
    d_sample = dev(gpu_ctx, sample)
    d_one, l_one, _ = api.kmeans_fit(gpu_ctx, d_sample, c, 1, Metric.Euclidean, 1)
    monkeypatch.setenv("GLIDE_B200_FF_LAUNCHES", "1")
    d_two, l_two, _ = api.kmeans_fit(gpu_ctx, d_sample, c, 1, Metric.Euclidean, 1)
    assert np.array_equal(api.to_u32(l_one), want_l) and np.array_equal(d_one.cpu().numpy(), want_c)
    assert np.array_equal(api.to_u32(l_two), want_l) and np.array_equal(d_two.cpu().numpy(), want_c)


def test_get_centroids_uses_seeded_sample(gpu_ctx):
    base, _, _ = case("int128")
    ids = api.sample_ids(base.shape[0], 600, 3)
    want_c, _, _ = oracle.kmeans(base[ids], 4, 25)
    d_c, _ = api.get_centroids(gpu_ctx, dev(gpu_ctx, base), 4, 0.2, seed=3)
    assert np.array_equal(d_c.cpu().numpy(), want_c)


@pytest.mark.parametrize("name", ["uniform16", "int128", "unit96", "uniform30", "scaled960", "uniform200"])
def test_build_boundary_reverse_refine_match_oracle(gpu_ctx, name):
    base, _, P = case(name)
    metric = Metric(P["metric"])
    n = base.shape[0]
    d_re, d_knn = dev(gpu_ctx, P["reorder_data"]), dev(gpu_ctx, P["knn"].view(np.uint32))
    d_map, d_local = dev(gpu_ctx, P["mapping"]), dev(gpu_ctx, P["local_sp"])
    pb = sp_from(P["p_build"])
    g = api._u32_tensor(gpu_ctx, (n, 16)); g.fill_(-1)
    api.subgraph_build_and_merge(gpu_ctx, d_re, d_knn, P["seg_start"], P["seg_len"], d_local, d_map, n, g, pb,
                                 P["alpha"], metric, skip_boundary=True)
    assert np.array_equal(api.to_u32(g), P["after_build"])
    g.fill_(-1)
    api.subgraph_build_and_merge(gpu_ctx, d_re, d_knn, P["seg_start"], P["seg_len"], d_local, d_map, n, g, pb,
                                 P["alpha"], metric)
    assert np.array_equal(api.to_u32(g), P["after_boundary"])
    api.reverse_graph(gpu_ctx, g)
    assert np.array_equal(api.to_u32(g), P["after_reverse"])
    api.refine(gpu_ctx, dev(gpu_ctx, base), g, dev(gpu_ctx, P["centroids"]), dev(gpu_ctx, P["orig_sp"]),
               sp_from(P["p_refine"]), P["alpha"], metric)
    assert np.array_equal(api.to_u32(g), P["graph"])


@pytest.mark.parametrize("name", ["int128", "unit96", "uniform30"])
@pytest.mark.parametrize("wave_rows", [0, 700, 64])
def test_refine_in_waves_matches_oracle(gpu_ctx, name, wave_rows):
    """Waves of consecutive ids: a wave's searches read the rows the earlier waves wrote. 0 is one wave;
    700 leaves a ragged last wave; 64 makes the later waves walk a graph that is mostly refined."""
    base, _, P = case(name)
    metric = P["metric"]
    want = oracle.refine(base, P["after_reverse"], P["centroids"], P["orig_sp"], P["p_refine"], P["alpha"], metric,
                         wave_rows=wave_rows)
    g = dev(gpu_ctx, P["after_reverse"])
    api.refine(gpu_ctx, dev(gpu_ctx, base), g, dev(gpu_ctx, P["centroids"]), dev(gpu_ctx, P["orig_sp"]),
               sp_from(P["p_refine"]), P["alpha"], Metric(metric), wave_rows=wave_rows)
    assert np.array_equal(api.to_u32(g), want)
    if wave_rows and name == "int128":   # the waves matter: the result differs from the single-wave one
        assert not np.array_equal(want, P["graph"])


def test_refine_of_one_partition_matches_oracle(gpu_ctx):
    """The large path's refine (one resident partition, no centroids, seeded from the partition's start point)."""
    base, _, P = case("int128")
    lo, ln = int(P["seg_start"][0]), int(P["seg_len"][0])
    part = np.ascontiguousarray(P["reorder_data"][lo:lo + ln])
    knn = np.ascontiguousarray(P["knn"][lo:lo + ln]).view(np.uint32)
    ob, orf = oracle.SearchParams.derive(64, 16), oracle.SearchParams.derive(128, 16)
    one = np.array([0], np.uint32)
    g0 = oracle.build_rows(part, knn, one, np.array([ln], np.uint32), np.array([9], np.uint32),
                           np.arange(ln, dtype=np.uint32), ln, 24, ob, 1.05)
    oracle.reverse_graph(g0)
    want = oracle.refine(part, g0, None, 9, orf, 1.05)
    assert (want != INVALID).sum() > (g0 != INVALID).sum()
    d_g = dev(gpu_ctx, g0)
    api.refine_partition(gpu_ctx, dev(gpu_ctx, part), d_g, 9, sp_from(orf), 1.05)
    assert np.array_equal(api.to_u32(d_g), want)


def test_build_with_wider_graph_than_knn(gpu_ctx):
    # graph_degree 48 > knn_degree 16, beam 64: rows keep holes that reverse edges and refinement fill
    base, _, P = case("uniform16")
    n = base.shape[0]
    o = oracle.SearchParams.derive(64, 16)
    want = oracle.build_rows(P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                             P["mapping"], n, 48, o, 1.05)
    oracle.build_boundary(P["reorder_data"], P["knn"].view(np.uint32), n, int(P["local_sp"][-1]), P["mapping"], want,
                          o, 1.05)
    g = api._u32_tensor(gpu_ctx, (n, 48)); g.fill_(-1)
    api.subgraph_build_and_merge(gpu_ctx, dev(gpu_ctx, P["reorder_data"]), dev(gpu_ctx, P["knn"].view(np.uint32)),
                                 P["seg_start"], P["seg_len"], dev(gpu_ctx, P["local_sp"]), dev(gpu_ctx, P["mapping"]),
                                 n, g, sp_from(o), 1.05)
    assert np.array_equal(api.to_u32(g), want)
    oracle.reverse_graph(want)
    api.reverse_graph(gpu_ctx, g)
    assert np.array_equal(api.to_u32(g), want)
    o2 = oracle.SearchParams.derive(128, 16)
    want2 = oracle.refine(base, want, P["centroids"], P["orig_sp"], o2, 1.05)
    api.refine(gpu_ctx, dev(gpu_ctx, base), g, dev(gpu_ctx, P["centroids"]), dev(gpu_ctx, P["orig_sp"]), sp_from(o2), 1.05)
    assert np.array_equal(api.to_u32(g), want2)


def test_reverse_graph_on_hub_heavy_graph(gpu_ctx):
    # many rows point at a few hubs, rows mostly empty: exercises capacity and ordering
    rng = np.random.default_rng(0)
    n, deg = 5000, 32
    g = np.full((n, deg), INVALID, np.uint32)
    for p in range(n):
        k = rng.integers(1, 6)
        row = np.unique(np.concatenate([rng.integers(0, 8, 2), rng.integers(0, n, k)]))
        row = row[row != p][:deg]
        g[p, :row.size] = rng.permutation(row)
    want = oracle.reverse_graph(g.copy())
    d_g = dev(gpu_ctx, g)
    api.reverse_graph(gpu_ctx, d_g)
    assert np.array_equal(api.to_u32(d_g), want)


@pytest.mark.parametrize("name", ["int128", "uniform30"])
def test_bruteforce_knn_matches_oracle(gpu_ctx, name):
    base, queries, P = case(name)
    want_ids, want_d = oracle.bruteforce_knn(base, queries, 10, P["metric"])
    ids, d = api.bruteforce_knn(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, queries), 10, Metric(P["metric"]))
    ids, d = api.to_u32(ids), d.cpu().numpy()
    assert np.allclose(d, want_d, rtol=1e-5)
    if name == "int128":  # exact arithmetic: ids must agree, ties broken by id on both sides
        assert np.array_equal(ids, want_ids)
    else:
        assert (ids == want_ids).mean() > 0.995


def test_bruteforce_knn_large_k_and_ragged_sizes(gpu_ctx):
    rng = np.random.default_rng(2)
    base = rng.integers(0, 50, (777, 20)).astype(np.float32)
    queries = rng.integers(0, 50, (65, 20)).astype(np.float32)
    want_ids, _ = oracle.bruteforce_knn(base, queries, 100)
    ids, _ = api.bruteforce_knn(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, queries), 100)
    assert np.array_equal(api.to_u32(ids), want_ids)


def knn_recall(knn, exact, k):
    hits = 0
    for r in range(knn.shape[0]):
        hits += len(set(knn[r, :k].tolist()) & set(exact[r, :k].tolist()))
    return hits / (knn.shape[0] * k)


@pytest.mark.parametrize("name", ["uniform16", "int128", "unit96"])
def test_nn_descent_graph_recall_and_invariants(gpu_ctx, name):
    base, _, P = case(name)
    rd, seg_start, seg_len = P["reorder_data"], P["seg_start"], P["seg_len"]
    metric = Metric(P["metric"])
    d_knn, rounds, seconds = api.build_nnd(gpu_ctx, NNDescentParameter(32), dev(gpu_ctx, rd), seg_start, seg_len, metric,
                                           seed=1, exact_max_rows=0)
    knn = d_knn.cpu().numpy()
    assert knn.shape == (rd.shape[0], 32) and 1 <= rounds <= 20
    exact = helpers.exact_partition_knn(rd, seg_start, seg_len, 10, P["metric"])
    # ids are partition-local, no self loops, no duplicates
    for s, l in zip(seg_start, seg_len):
        part = knn[int(s):int(s) + int(l)]
        assert part.min() >= 0 and part.max() < int(l)
    rows = np.arange(rd.shape[0])
    local = rows - np.repeat(seg_start, seg_len)
    assert not (knn == local[:, None]).any()
    assert all(len(set(r.tolist())) == 32 for r in knn[::53])
    assert knn_recall(knn, exact, 10) >= 0.95
    # reproducible
    d_knn2, rounds2, _ = api.build_nnd(gpu_ctx, NNDescentParameter(32), dev(gpu_ctx, rd), seg_start, seg_len, metric, seed=1,
                                       exact_max_rows=0)
    assert rounds2 == rounds and torch.equal(d_knn, d_knn2)


@pytest.mark.parametrize("name,degree", [("int128", 32), ("uniform16", 16), ("unit96", 48), ("uniform30", 32)])
def test_exact_partition_knn_kernel(gpu_ctx, name, degree):
    base, _, P = case(name)
    rd, seg_start, seg_len = P["reorder_data"], P["seg_start"], P["seg_len"]
    d_knn, rounds, _ = api.build_nnd(gpu_ctx, NNDescentParameter(degree), dev(gpu_ctx, rd), seg_start, seg_len,
                                     Metric(P["metric"]))
    knn = d_knn.cpu().numpy()
    assert rounds == 0 and knn.shape == (rd.shape[0], degree)
    exact = helpers.exact_partition_knn(rd, seg_start, seg_len, degree, P["metric"])
    if name == "int128":   # exact arithmetic: identical, ties by ascending id
        assert np.array_equal(knn, exact)
    else:                  # a different summation order may swap near-ties
        assert (knn == exact).mean() > 0.995
        assert knn_recall(knn, exact, degree) > 0.999


@pytest.mark.parametrize("dim,degree,kind", [(128, 32, "int"), (64, 64, "int"), (96, 48, "unit"), (32, 16, "uniform"),
                                             (128, 20, "scaled")])
def test_tensor_core_knn_equals_exact_knn(gpu_ctx, dim, degree, kind):
    """The kNN stage's tensor-core kernel (dims that are multiples of 32 up to 128) on partitions of ragged
    sizes, from a single row to several tiles: integer-valued rows give TF32 products that are exact, so
    the rows must equal the brute-force rows with ties by ascending id; elsewhere the exact re-rank of
    twice the list width leaves nothing but near-ties to differ."""
    base, _ = helpers.small_dataset(kind, 6000, dim, 10, seed=29)
    lens = [1, 2, 40, 129, 700, 1100, 2100]     # 1100 rows: nine tiles, a group size just past a power of two
    lens.append(6000 - sum(lens))
    seg_len = np.array(lens, np.uint32)
    seg_start = np.concatenate([[0], np.cumsum(seg_len)[:-1]]).astype(np.uint32)
    metric = oracle.COSINE if kind == "unit" else oracle.EUCLIDEAN
    fallbacks = gpu_ctx.tc_knn_fallbacks
    d_knn, rounds, seconds = api.build_nnd(gpu_ctx, NNDescentParameter(degree), dev(gpu_ctx, base), seg_start, seg_len,
                                           Metric(metric))
    knn = d_knn.cpu().numpy()
    assert rounds == 0 and knn.shape == (6000, degree) and seconds > 0
    assert gpu_ctx.tc_knn_fallbacks == fallbacks       # the rows below come from the tensor-core kernel, not from its fallback
    exact = helpers.exact_partition_knn(base, seg_start, seg_len, degree, metric)
    for s, l in zip(seg_start, seg_len):
        s, l = int(s), int(l)
        got, want = knn[s:s + l], exact[s:s + l]
        assert got.min() >= 0 and got.max() < l
        real = min(degree, l - 1)              # entries beyond the partition's other rows are padding
        if real == 0:
            continue
        if kind == "int":                      # exact arithmetic: identical, ties by ascending id
            assert np.array_equal(got[:, :real], want[:, :real])
        else:
            assert (got[:, :real] == want[:, :real]).mean() > 0.99
            assert knn_recall(got, want, real) > 0.999
        assert not (got[:, :real] == np.arange(l)[:, None]).any()      # no self loops


def test_mixed_exact_and_descent_partitions(gpu_ctx):
    # partitions above the threshold run NN-descent, the others the all-pairs kernel
    base, _, P = case("int128")
    rd, seg_start, seg_len = P["reorder_data"], P["seg_start"], P["seg_len"]
    threshold = int(np.sort(seg_len)[len(seg_len) // 2])
    d_knn, rounds, _ = api.build_nnd(gpu_ctx, NNDescentParameter(32), dev(gpu_ctx, rd), seg_start, seg_len,
                                     exact_max_rows=threshold, seed=2)
    knn = d_knn.cpu().numpy()
    exact = helpers.exact_partition_knn(rd, seg_start, seg_len, 32, 0)
    assert rounds >= 1
    for s, l in zip(seg_start, seg_len):
        s, l = int(s), int(l)
        if l == 0:
            continue
        if l <= threshold:
            assert np.array_equal(knn[s:s + l], exact[s:s + l])
        else:
            assert knn_recall(knn[s:s + l], exact[s:s + l], 10) >= 0.95
            assert knn[s:s + l].max() < l


def test_large_path_stages_match_oracle(gpu_ctx):
    base, queries = helpers.small_dataset("uniform", 1500, 16, 60, seed=5)
    C = 3
    centroids, _, _ = oracle.kmeans(base[:300], C, 10)
    seg_index, seg_start, seg_len = oracle.define_partition(base, centroids, -1.0)
    rd, mapping = oracle.reorder(base, seg_index, seg_start, 0)
    want_routes = oracle.select_segments(queries, centroids, 2, 1.2)
    d_q = dev(gpu_ctx, queries)
    d_routes = api.select_segments(gpu_ctx, d_q, dev(gpu_ctx, centroids), 2, 1.2)
    assert np.array_equal(api.to_u32(d_routes), want_routes)
    o = oracle.SearchParams.derive(64, 16)
    ob = oracle.SearchParams.derive(64, 16)
    want_ids = np.full((60, 10), INVALID, np.uint32)
    want_d = np.full((60, 10), np.finfo(np.float32).max, np.float32)
    d_fi = dev(gpu_ctx, want_ids.copy())
    d_fd = dev(gpu_ctx, want_d.copy())
    for s in range(C):
        lo, ln = int(seg_start[s]), int(seg_len[s])
        part = rd[lo:lo + ln]
        knn = helpers.exact_partition_knn(part, np.array([0], np.uint32), np.array([ln], np.uint32), 16, oracle.EUCLIDEAN)
        # build_for_large / refine_for_large on the resident partition
        one = np.array([0], np.uint32)
        want_g = oracle.build_rows(part, knn.view(np.uint32), one, np.array([ln], np.uint32), np.array([5], np.uint32),
                                   np.arange(ln, dtype=np.uint32), ln, 24, ob, 1.05)
        d_part = dev(gpu_ctx, part)
        d_g = api.build_partition(gpu_ctx, d_part, dev(gpu_ctx, knn.view(np.uint32)), 5, 24, sp_from(ob), 1.05)
        assert np.array_equal(api.to_u32(d_g), want_g)
        oracle.search_on_sub(part, want_g, mapping[lo:lo + ln], 5, queries, want_routes, s, o, want_ids, want_d)
        api.search_on_sub(gpu_ctx, d_part, d_g, dev(gpu_ctx, mapping[lo:lo + ln]), 5, d_q, d_routes, s, sp_from(o),
                          d_fi, d_fd)
    assert np.array_equal(api.to_u32(d_fi), want_ids)
    assert np.array_equal(d_fd.cpu().numpy(), want_d)


def test_unsupported_shapes_are_rejected(gpu_ctx):
    base, queries, P = case("uniform16")
    index = api.GLIDE(gpu_ctx, 16, base, P["centroids"])
    index.load(P["graph"], P["orig_sp"])
    bad = SearchParameter(top_k=10, beam=544, max_iterations=10, hash_bit=11, hash_reset_interval=1)
    with pytest.raises(api.UnsupportedError):  # kernel_config.cuh:47-48 "Unsupported beam"
        index.search(bad, dev(gpu_ctx, queries))
    with pytest.raises(api.GlideError):
        index.search(SearchParameter(top_k=10, beam=48, max_iterations=10, hash_bit=8, hash_reset_interval=1),
                     dev(gpu_ctx, queries))
    with pytest.raises(api.GlideError):  # top_k > beam
        index.search(SearchParameter(top_k=40, beam=32, max_iterations=10, hash_bit=8, hash_reset_interval=1),
                     dev(gpu_ctx, queries))
    # the context stays usable after a rejected call
    ok = SearchParameter(top_k=10, beam=32).derive(16)
    ids, _, _ = index.search(ok, dev(gpu_ctx, queries))
    assert ids.shape == (queries.shape[0], 10)


def test_empty_query_batch(gpu_ctx):
    base, queries, P = case("uniform16")
    index = api.GLIDE(gpu_ctx, 16, base, P["centroids"])
    index.load(P["graph"], P["orig_sp"])
    ids, d, _ = index.search(SearchParameter(top_k=10, beam=32).derive(16), dev(gpu_ctx, queries[:0]))
    assert ids.shape == (0, 10) and d.shape == (0, 10)


def test_cfg0_pipeline_recall(gpu_ctx):
    """Tiny correctness build: 10,000 x 32 uniform, degree 32, NN-descent 8 iterations, one partition."""
    from glide_b200 import datasets, pipeline
    spec = datasets.CONFIGS["cfg0"]
    base, queries = datasets.make(spec)
    cfg = pipeline.BuildConfig(centroid_num=1, knn_degree=32, graph_degree=32, nnd_max_iterations=8, seed=0,
                               sample_factor=0.05, exact_knn_max_rows=0)
    res = pipeline.build_small(gpu_ctx, dev(gpu_ctx, base), cfg, keep_intermediates=True)
    assert res.h_segment_length.tolist() == [10000, 0]
    gt = oracle.bruteforce_knn(base, queries, 10, want_dists=False)
    # kNN graph quality
    exact = helpers.exact_partition_knn(res.d_reorder_data.cpu().numpy(), res.h_segment_start, res.h_segment_length, 10, 0)
    assert knn_recall(res.d_knn.cpu().numpy(), exact, 10) >= 0.9
    graph = api.to_u32(res.index.graph_view())
    assert (graph != INVALID).all(axis=1).mean() > 0.9
    recalls = {}
    for beam in (32, 64, 128):
        sp = pipeline.derive_search_params(beam, 32)
        ids, dists, _ = res.index.search(sp, dev(gpu_ctx, queries))
        recalls[beam] = api.calculate_recall(ids, gt, 10)
        o = oracle.SearchParams(sp.beam, sp.max_iterations, sp.min_iterations, sp.hash_bit, sp.hash_reset_interval, 10)
        want_ids, want_d = oracle.search(base, graph, res.index.centroid_view().cpu().numpy(),
                                         api.to_u32(res.index.start_point_view()), queries, o)
        assert np.array_equal(ids, want_ids) and np.array_equal(dists, want_d)
    assert recalls[64] >= 0.95 and recalls[128] >= recalls[64] - 1e-6
    # the GPU-built graph equals the oracle's graph built from the same kNN graph and start points
    P = dict(rd=res.d_reorder_data.cpu().numpy(), knn=res.d_knn.cpu().numpy().view(np.uint32), mp=api.to_u32(res.d_map))
    p_knn, p_ref = pipeline.derive_build_search_params(cfg)
    local, original = api.start_point_select(res.h_segment_start, res.h_segment_length, P["mp"], cfg.seed)
    ok = oracle.SearchParams(p_knn.beam, p_knn.max_iterations, 0, p_knn.hash_bit, p_knn.hash_reset_interval)
    orf = oracle.SearchParams(p_ref.beam, p_ref.max_iterations, 0, p_ref.hash_bit, p_ref.hash_reset_interval)
    want = oracle.build_rows(P["rd"], P["knn"], res.h_segment_start, res.h_segment_length, local, P["mp"], 10000, 32, ok, 1.05)
    oracle.reverse_graph(want)
    want = oracle.refine(base, want, res.index.centroid_view().cpu().numpy(), original, orf, 1.05)
    assert np.array_equal(graph, want)


def test_sharded_build_with_one_rank_equals_plain_build(gpu_ctx):
    from glide_b200 import pipeline
    base, _ = helpers.small_dataset("int", 4000, 32, 10, seed=9)
    cfg = pipeline.BuildConfig(centroid_num=4, knn_degree=16, graph_degree=16, build_beam=32, refine_beam=64,
                               sample_factor=0.1, boundary_factor=1.15, seed=3)
    a = pipeline.build_small(gpu_ctx, dev(gpu_ctx, base), cfg)
    b = pipeline.build_small_sharded(gpu_ctx, dev(gpu_ctx, base), cfg)
    assert a.h_segment_length[-1] > 0   # the boundary path is exercised
    assert torch.equal(a.index.graph_view(), b.index.graph_view())
    assert torch.equal(a.index.start_point_view(), b.index.start_point_view())


def _sharded_rank(rank, world, port, out_dir):
    import os
    import torch.distributed as dist
    from glide_b200 import pipeline
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = api.Context(rank)
    base, _ = helpers.small_dataset("int", 4000, 32, 10, seed=9)
    cfg = pipeline.BuildConfig(centroid_num=4, knn_degree=16, graph_degree=16, build_beam=32, refine_beam=64,
                               sample_factor=0.1, boundary_factor=1.15, seed=3, refine_wave_rows=1000)
    d = torch.from_numpy(base).to(ctx.torch_device)
    from glide_b200 import sharded
    ctx.init_comm(dist, world, rank)          # the library's own NCCL communicator; the token travels over torch.distributed
    shard = pipeline.build_small_sharded(ctx, d, cfg, sharded.GlideCollectives(ctx))
    plain = pipeline.build_small(ctx, d, cfg)
    ok = torch.equal(plain.index.graph_view(), shard.index.graph_view())
    # NN-descent partitions (exact kernel off) sharded by owner give the same kNN rows too
    cfg2 = pipeline.BuildConfig(centroid_num=4, knn_degree=16, graph_degree=16, build_beam=32, refine_beam=64,
                                sample_factor=0.1, boundary_factor=1.15, seed=3, exact_knn_max_rows=0, refine_wave_rows=1000)
    a = pipeline.build_small(ctx, d, cfg2)
    b = pipeline.build_small_sharded(ctx, d, cfg2, sharded.GlideCollectives(ctx))
    ok = ok and torch.equal(a.index.graph_view(), b.index.graph_view())
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()


def test_sharded_build_on_two_gpus_equals_plain_build(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import torch.multiprocessing as mp
    port = 29400 + os.getpid() % 500
    mp.spawn(_sharded_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "rank0.txt").read() == "ok" and open(tmp_path / "rank1.txt").read() == "ok"


def test_large_path_end_to_end(gpu_ctx):
    """preprocess_for_large -> build_knn_for_large -> GLIDE_large.build -> search, checked against
    the oracle replaying the same stages on the same graphs, and against exact kNN for recall."""
    from glide_b200 import large
    from glide_b200.params import IndexParameter
    base, queries = helpers.small_dataset("uniform", 6000, 32, 150, seed=13)
    pre = large.preprocess_for_large(gpu_ctx, base, 4, 0.1, batch_num=3, seed=2)
    assert pre["h_segment_length"].sum() == 6000 and sorted(pre["h_map"].tolist()) == list(range(6000))
    want_seg = oracle.define_partition(base, pre["h_centroids"], -1.0)[0][:, 0]
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        members = pre["h_map"][int(lo):int(lo) + int(ln)]
        assert np.all(want_seg[members] == s) and np.all(np.diff(members.astype(np.int64)) > 0)
    knn, _ = large.build_knn_for_large(gpu_ctx, NNDescentParameter(16), pre["h_reorder_data"], pre["h_segment_start"],
                                       pre["h_segment_length"])
    index = large.GLIDE_large(gpu_ctx, 24, Metric.Euclidean, pre["h_reorder_data"], pre["h_map"], pre["h_centroids"],
                              pre["h_segment_start"], pre["h_segment_length"])
    pk = SearchParameter(beam=64).derive(16)
    pr = SearchParameter(beam=128).derive(16)
    index.build(IndexParameter(24, 16, 1.05), pk, pr, knn, seed=5)
    assert (index.graph_view() != INVALID).any(axis=1).all()
    sp = SearchParameter(top_k=10, beam=64).derive(24)
    ids, dists, _ = index.search(sp, 2, 1.2, dev(gpu_ctx, queries))
    # oracle replay of the search over the GPU-built subgraphs
    o = oracle.SearchParams(sp.beam, sp.max_iterations, 0, sp.hash_bit, sp.hash_reset_interval, 10)
    routes = oracle.select_segments(queries, pre["h_centroids"], 2, 1.2)
    want_ids = np.full((150, 10), INVALID, np.uint32)
    want_d = np.full((150, 10), np.finfo(np.float32).max, np.float32)
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        lo, ln = int(lo), int(ln)
        oracle.search_on_sub(pre["h_reorder_data"][lo:lo + ln], index.graph_view()[lo:lo + ln], pre["h_map"][lo:lo + ln],
                             int(index.start_point_view()[s]), queries, routes, s, o, want_ids, want_d)
    assert np.array_equal(ids, want_ids) and np.array_equal(dists, want_d)
    gt = oracle.bruteforce_knn(base, queries, 10, want_dists=False)
    assert api.calculate_recall(ids, gt, 10) > 0.9


def test_full_size_cfg1_properties(gpu_ctx):
    """The benchmark's own workload (1,000,000 x 128, 10,000 queries) through size-independent
    properties: results sorted, ids valid and distinct, distances equal to a recomputation, recall
    against exact kNN, exact kNN equal to the host's on a sample, graph rows free of duplicates and
    self loops, search idempotent, and a sample of queries bit-equal to the oracle."""
    from glide_b200 import datasets, pipeline
    spec = datasets.CONFIGS["cfg1"]
    base, queries = datasets.make(spec)
    d_base, d_q = dev(gpu_ctx, base), dev(gpu_ctx, queries)
    cfg = pipeline.BuildConfig(centroid_num=1024, sample_factor=0.1, seed=spec.seed)
    before = gpu_ctx.tc_knn_fallbacks
    res = pipeline.build_small(gpu_ctx, d_base, cfg)
    # the kNN stage stayed on the tensor-core kernel (partitions of 9 tiles once overflowed its buffers)
    assert gpu_ctx.tc_knn_fallbacks == before
    graph = api.to_u32(res.index.graph_view())
    n = base.shape[0]
    valid = graph != INVALID
    assert (graph[valid] < n).all()
    # self loops are possible but rare: the build's seed step compares partition-local ids with the
    # point's reorder id (graph_kernel.cuh:295-298), so a point listed in its start point's kNN row
    # can meet itself at distance 0
    assert (graph == np.arange(n, dtype=np.uint32)[:, None]).any(axis=1).mean() < 0.05
    for r in graph[::997]:                                                        # no duplicate neighbours
        r = r[r != INVALID]
        assert len(set(r.tolist())) == r.size
    assert valid.mean() > 0.9
    gt_ids, _ = api.bruteforce_knn(gpu_ctx, d_base, d_q, 10)
    gt = api.to_u32(gt_ids)
    host_gt = oracle.bruteforce_knn(base, queries[:32], 10, want_dists=False)
    assert np.array_equal(gt[:32], host_gt)
    sp = pipeline.derive_search_params(40, 32)
    ids, dists, _ = res.index.search(sp, d_q)
    ids2, dists2, _ = res.index.search(sp, d_q)
    assert np.array_equal(ids, ids2) and np.array_equal(dists, dists2)              # idempotent
    assert (np.diff(dists, axis=1) >= 0).all()
    assert (ids < n).all()
    assert all(len(set(r.tolist())) == 10 for r in ids[::101])
    for q in range(0, 10000, 503):   # distances are what they claim to be (integer data: exact)
        sums = ((base[ids[q]].astype(np.int64) - queries[q].astype(np.int64)) ** 2).sum(axis=1)
        assert np.array_equal(dists[q], np.sqrt(sums.astype(np.float32)))
    assert api.calculate_recall(ids, gt, 10) >= 0.95
    o = oracle.SearchParams(sp.beam, sp.max_iterations, 0, sp.hash_bit, sp.hash_reset_interval, 10)
    want_ids, want_d = oracle.search(base, graph, res.index.centroid_view().cpu().numpy(),
                                     api.to_u32(res.index.start_point_view()), queries[:200], o)
    assert np.array_equal(ids[:200], want_ids) and np.array_equal(dists[:200], want_d)


def _stress_partition_inputs(kind, rng):
    """Inputs chosen to strain the tensor-core prefilter of the assignment: many centroids, large
    common offsets (norms far above the distances), duplicated and nearly duplicated centroids."""
    n, dim, C = 6000, 128, 300
    if kind == "mixture_1024":
        C = 1024
        cent = rng.uniform(0, 120, (C, dim)).astype(np.float32)
        base = np.clip(np.rint(cent[rng.integers(0, C, n)] + rng.normal(0, 20, (n, dim))), 0, 218).astype(np.float32)
        centroids = (cent + rng.normal(0, 2, (C, dim))).astype(np.float32)
    elif kind == "offset":          # |p|, |c| ~ 1e4 while distances ~ 10: the margin swallows everything
        base = (1000.0 + rng.normal(0, 1, (n, dim))).astype(np.float32)
        centroids = (1000.0 + rng.normal(0, 1, (C, dim))).astype(np.float32)
    elif kind == "duplicates":      # exact ties between centroids -> the network's tie order decides
        centroids = rng.normal(0, 1, (C, dim)).astype(np.float32)
        centroids[1::2] = centroids[0::2]
        base = (centroids[rng.integers(0, C, n)] + rng.normal(0, 0.3, (n, dim))).astype(np.float32)
    elif kind == "near_duplicates":  # centroids one ulp-scale step apart
        centroids = rng.normal(0, 1, (C, dim)).astype(np.float32)
        centroids[1::2] = centroids[0::2] * np.float32(1.0 + 3e-7)
        base = (centroids[rng.integers(0, C, n)] + rng.normal(0, 0.3, (n, dim))).astype(np.float32)
    elif kind == "unit96":
        dim = 96
        centroids = rng.normal(0, 1, (C, dim)).astype(np.float32)
        centroids /= np.linalg.norm(centroids, axis=1, keepdims=True)
        base = (centroids[rng.integers(0, C, n)] + rng.normal(0, 0.05, (n, dim))).astype(np.float32)
        base /= np.linalg.norm(base, axis=1, keepdims=True)
    elif kind == "int_ties":        # small integers: equal distances to different centroids are common
        C = 64
        centroids = rng.integers(0, 3, (C, dim)).astype(np.float32)
        base = rng.integers(0, 3, (n, dim)).astype(np.float32)
    return base, centroids


@pytest.mark.parametrize("kind", ["mixture_1024", "offset", "duplicates", "near_duplicates", "unit96", "int_ties"])
def test_assignment_with_tensor_core_prefilter_is_exact(gpu_ctx, kind):
    """The assignment's tensor-core prefilter only proposes candidates; the exact re-rank and the
    tie fallback must give the oracle's nearest centroid, slot and boundary flag for every point."""
    base, centroids = _stress_partition_inputs(kind, np.random.default_rng(11))
    metric = oracle.COSINE if kind == "unit96" else oracle.EUCLIDEAN
    for factor in (1.1, -1.0):
        want_index, want_start, want_len = oracle.define_partition(base, centroids, factor, metric)
        gpu_ctx.enable_counters(True)
        d_seg, seg_start, seg_len = api.define_partition(gpu_ctx, dev(gpu_ctx, base), dev(gpu_ctx, centroids), factor,
                                                         Metric(metric))
        by_fallback = gpu_ctx.read_counters()[3]
        gpu_ctx.enable_counters(False)
        assert np.array_equal(seg_len, want_len) and np.array_equal(seg_start, want_start)
        assert np.array_equal(api.to_u32(d_seg), want_index)
        if kind in ("mixture_1024", "unit96"):      # the prefilter, not the fallback, does the work on ordinary data
            assert by_fallback < 0.02 * base.shape[0]
        if kind == "duplicates":                    # every nearest centroid has a twin: all points tie
            assert by_fallback == base.shape[0]


_ASSIGN_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import oracle
from glide_b200 import api
from glide_b200.params import Metric
import test_gpu_parity as t
ctx = api.Context(0)
for kind in ("mixture_1024", "unit96", "int_ties"):
    base, centroids = t._stress_partition_inputs(kind, np.random.default_rng(5))
    metric = oracle.COSINE if kind == "unit96" else oracle.EUCLIDEAN
    want = oracle.define_partition(base, centroids, 1.1, metric)
    d_seg, seg_start, seg_len = api.define_partition(ctx, torch.from_numpy(base).cuda(), torch.from_numpy(centroids).cuda(),
                                                     1.1, Metric(metric))
    assert np.array_equal(api.to_u32(d_seg), want[0]) and np.array_equal(seg_len, want[2]), kind
print("ok")
"""


@pytest.mark.parametrize("env", ["GLIDE_B200_NO_TMA", "GLIDE_B200_EXACT_ASSIGN"])
def test_assignment_variants_behind_switches_are_exact_too(env):
    """The cp.async-staged tensor-core kernel (taken when a tensor map cannot be made or dim % 32 != 0)
    and the exact fp32 kernels (other dims, no scratch) give the same partitioning; each is selected by
    an environment switch read when the library first assigns, hence the child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _ASSIGN_CHILD.format(root=root, tests=os.path.join(root, "tests"))
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, **{env: "1"}), capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
