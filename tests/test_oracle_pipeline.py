"""CPU checks of the oracle's stage restatements through their invariants, on small seeded data."""
import numpy as np
import pytest

import helpers
import oracle

INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def pipe():
    base, queries = helpers.small_dataset("uniform", 3000, 16, 200)
    return base, queries, helpers.oracle_pipeline(base)


def test_partition_and_reorder(pipe):
    base, _, P = pipe
    n = base.shape[0]
    C = P["centroids"].shape[0]
    seg_index, seg_start, seg_len = P["seg_index"], P["seg_start"], P["seg_len"]
    assert seg_len[:C].sum() == n
    assert seg_start[C] == n  # the boundary segment follows the main rows
    # nearest centroid + boundary rule, recomputed in float64 away from the decision boundary
    d = np.sqrt(((base[:, None, :].astype(np.float64) - P["centroids"][None].astype(np.float64)) ** 2).sum(-1))
    order = np.argsort(d, axis=1)
    assert np.array_equal(order[:, 0], seg_index[:, 0])
    ratio = np.take_along_axis(d, order[:, 1:2], 1)[:, 0] / np.take_along_axis(d, order[:, 0:1], 1)[:, 0]
    clear = np.abs(ratio - 1.1) > 1e-4
    assert np.array_equal((ratio <= 1.1)[clear], (seg_index[:, 2] != INVALID)[clear])
    # slots are ranks in ascending id order
    for c in range(C):
        members = np.nonzero(seg_index[:, 0] == c)[0]
        assert np.array_equal(seg_index[members, 1], np.arange(members.size))
    bmembers = np.nonzero(seg_index[:, 2] != INVALID)[0]
    assert np.array_equal(seg_index[bmembers, 2], np.arange(bmembers.size))
    # reorder: map is a permutation on the main rows, boundary rows are copies
    mapping, rd = P["mapping"], P["reorder_data"]
    assert sorted(mapping[:n].tolist()) == list(range(n))
    assert np.array_equal(rd, base[mapping])


def test_build_rows_are_pruned_subsets_in_original_ids(pipe):
    base, _, P = pipe
    g = P["after_build"]
    n = base.shape[0]
    assert g.shape == (n, 16)
    seg_of = P["seg_index"][:, 0]
    for p in range(0, n, 97):
        row = g[p][g[p] != INVALID]
        assert row.size >= 1 and len(set(row.tolist())) == row.size
        assert np.all(seg_of[row] == seg_of[p])  # main-partition edges stay inside the partition
        # rows are front-packed
        assert np.all(g[p][:row.size] != INVALID)


def test_boundary_merge_adds_cross_partition_edges(pipe):
    base, _, P = pipe
    before, after = P["after_build"], P["after_boundary"]
    seg_of = P["seg_index"][:, 0]
    changed = np.nonzero((before != after).any(axis=1))[0]
    boundary_points = np.nonzero(P["seg_index"][:, 2] != INVALID)[0]
    assert set(changed.tolist()) <= set(boundary_points.tolist())
    cross = 0
    for p in changed:
        row = after[p][after[p] != INVALID]
        cross += int(np.sum(seg_of[row] != seg_of[p]))
        new = set(after[p].tolist()) - set(before[p].tolist())
        assert len(new) <= 16 // 2  # at most half a row is replaced (graph_kernel.cuh:224-246)
    assert cross > 0


def test_reverse_only_fills_holes_with_true_reverse_edges(pipe):
    _, _, P = pipe
    before, after = P["after_boundary"], P["after_reverse"]
    kept = before != INVALID
    assert np.array_equal(before[kept], after[kept])
    filled = np.nonzero((before == INVALID) & (after != INVALID))
    for p, slot in zip(*filled):
        src = after[p, slot]
        assert p in before[src]           # src really points at p
        assert src not in before[p]       # and p did not list it yet
    # a row with holes left received every available reverse edge
    for p in np.nonzero((after == INVALID).any(axis=1))[0][:50]:
        incoming = {s for s in np.nonzero((before == p).any(axis=1))[0] if s not in before[p]}
        assert incoming <= set(after[p].tolist())


def test_refine_fills_remaining_holes_without_touching_existing_edges(pipe):
    _, _, P = pipe
    before, after = P["after_reverse"], P["graph"]
    kept = before != INVALID
    assert np.array_equal(before[kept], after[kept])
    assert (after == INVALID).sum() <= (before == INVALID).sum()
    for p in np.nonzero((before == INVALID).any(axis=1))[0][:100]:
        new = after[p][(before[p] == INVALID) & (after[p] != INVALID)]
        assert p not in new
        assert not (set(new.tolist()) & set(before[p][before[p] != INVALID].tolist()))


def test_search_recall_and_exact_distances(pipe):
    base, queries, P = pipe
    gt = oracle.bruteforce_knn(base, queries, 10, want_dists=False)
    recalls = []
    for beam in (32, 64, 128):
        sp = oracle.SearchParams.derive(beam, 16)
        ids, dists, counters = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, sp,
                                             want_counters=True)
        recalls.append(oracle.recall(ids, gt, 10))
        assert np.all(np.diff(dists, axis=1) >= 0)
        for q in range(0, 200, 37):
            for j in range(10):
                want = oracle.distance(queries[q], base[ids[q, j]], oracle.EUCLIDEAN, oracle.ORDER_WARP)
                assert dists[q, j] == want
        assert counters[:, 1].max() <= sp.max_iterations
    assert recalls[0] >= 0.9 and recalls[-1] >= recalls[0] - 1e-6 and recalls[-1] >= 0.97


def test_search_with_full_beam_on_exact_graph_is_exact():
    # beam >= n on a connected kNN graph must return the exact neighbours
    base, queries = helpers.small_dataset("uniform", 200, 8, 20, seed=11)
    knn = helpers.exact_partition_knn(base, np.array([0], np.uint32), np.array([200], np.uint32), 32, oracle.EUCLIDEAN)
    centroids = base.mean(axis=0, keepdims=True)
    sp = oracle.SearchParams.derive(256, 32, max_iterations=400)
    ids, _ = oracle.search(base, knn.view(np.uint32), centroids, np.array([0], np.uint32), queries, sp)
    gt = oracle.bruteforce_knn(base, queries, 10, want_dists=False)
    assert oracle.recall(ids, gt, 10) == 1.0


def test_integer_data_ties_are_deterministic():
    base, queries = helpers.small_dataset("int", 2000, 16, 50)
    P1 = helpers.oracle_pipeline(base, centroid_num=3)
    P2 = helpers.oracle_pipeline(base, centroid_num=3)
    assert np.array_equal(P1["graph"], P2["graph"])
    sp = oracle.SearchParams.derive(64, 16)
    a = oracle.search(base, P1["graph"], P1["centroids"], P1["orig_sp"], queries, sp, threads=1)
    b = oracle.search(base, P1["graph"], P1["centroids"], P1["orig_sp"], queries, sp, threads=4)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_single_partition_has_empty_boundary():
    # centroid_num = 1: no boundary test (partition_kernel.cuh:58), empty boundary segment
    base, _ = helpers.small_dataset("uniform", 500, 8, 10)
    P = helpers.oracle_pipeline(base, centroid_num=1, with_refine=True)
    assert P["seg_len"].tolist() == [500, 0]
    assert np.array_equal(P["after_build"], P["after_boundary"])


def test_kmeans_reduces_inertia_and_is_deterministic():
    base, _ = helpers.small_dataset("int", 4000, 16, 10)
    c1, l1, r1 = oracle.kmeans(base, 8, 25)
    c2, l2, r2 = oracle.kmeans(base, 8, 25)
    assert np.array_equal(c1, c2) and np.array_equal(l1, l2) and r1 == r2
    def inertia(c, l):
        return float(((base - c[l]) ** 2).sum())
    l0 = np.argmin(((base[:, None] - base[None, :8]) ** 2).sum(-1), axis=1)
    assert inertia(c1, l1) < inertia(base[:8], l0)


def test_large_path_routing_and_merge():
    base, queries = helpers.small_dataset("uniform", 1500, 16, 60, seed=5)
    C = 3
    centroids, _, _ = oracle.kmeans(base[:300], C, 10)
    seg_index, seg_start, seg_len = oracle.define_partition(base, centroids, -1.0)
    assert seg_len[C] == 0
    rd, mapping = oracle.reorder(base, seg_index, seg_start, 0)
    routes = oracle.select_segments(queries, centroids, 2, 1.2)
    assert np.all(routes[:, 0] != INVALID) and np.all(routes[:, 1] != INVALID)
    sp = oracle.SearchParams.derive(64, 16)
    final_ids = np.full((60, 10), INVALID, np.uint32)
    final_d = np.full((60, 10), np.finfo(np.float32).max, np.float32)
    for s in range(C):
        lo, ln = int(seg_start[s]), int(seg_len[s])
        part = rd[lo:lo + ln]
        knn = helpers.exact_partition_knn(part, np.array([0], np.uint32), np.array([ln], np.uint32), 16, oracle.EUCLIDEAN)
        oracle.search_on_sub(part, knn.view(np.uint32), mapping[lo:lo + ln], 0, queries, routes, s, sp, final_ids, final_d)
    gt = oracle.bruteforce_knn(base, queries, 10, want_dists=False)
    assert np.all(np.diff(final_d, axis=1) >= 0)
    assert oracle.recall(final_ids, gt, 10) > 0.85


@pytest.mark.parametrize("beam,degree", [(300, 16), (512, 16), (64, 160), (300, 200)])
def test_two_warp_sort_and_merge_order_the_same_keys_as_the_single_warp_network(pipe, beam, degree):
    """The reference's two-warp candidate sort (rows wider than 128) and two-warp beam merge (beams above
    256) are other routes to the same sorted beam: on data without distance ties the search must return
    exactly what the single-warp network returns; with ties only ids of equal distances may differ."""
    base, queries, P = pipe
    n = base.shape[0]
    graph = np.full((n, degree), INVALID, np.uint32)
    graph[:, :16] = P["graph"]
    rng = np.random.default_rng(1)
    for r in range(n):
        have = set(P["graph"][r][P["graph"][r] != INVALID].tolist()) | {r}
        extra = [int(x) for x in rng.permutation(n)[:degree] if int(x) not in have][:degree - 16]
        graph[r, 16:16 + len(extra)] = extra
    sp = oracle.SearchParams.derive(beam, degree, top_k=10)
    try:
        oracle.set_two_warps(False)
        ids1, d1, c1 = oracle.search(base, graph, P["centroids"], P["orig_sp"], queries[:60], sp, want_counters=True)
    finally:
        oracle.set_two_warps(True)
    ids2, d2, c2 = oracle.search(base, graph, P["centroids"], P["orig_sp"], queries[:60], sp, want_counters=True)
    assert np.array_equal(d1, d2) and np.array_equal(ids1, ids2) and np.array_equal(c1, c2)
    gt = oracle.bruteforce_knn(base, queries[:60], 10, want_dists=False)
    assert oracle.recall(ids2, gt, 10) > 0.97
