"""Large path through the library's streaming object (`glide_large_*`): partitions of a host-resident
set pass through two device slots. Checked against the per-partition entry points (which the
other GPU tests check against the oracle), against the oracle's replay of the search, and for the
properties of the host orchestration itself: uint8 rows give what fp32 rows give, partitions kept in
device memory give what streamed ones give, only partitions some query is routed to are uploaded,
and per-rank result sets fold into the single-process result."""
import numpy as np
import pytest
import torch

import helpers
import oracle
from glide_b200 import api, large
from glide_b200.params import IndexParameter, Metric, NNDescentParameter, SearchParameter

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def built(gpu_ctx):
    base, queries = helpers.small_dataset("int", 9000, 64, 300, seed=17)   # integer valued: uint8 holds it exactly
    pre = large.preprocess_for_large(gpu_ctx, base, 6, 0.1, batch_num=4, seed=2)
    index = large.GLIDE_large(gpu_ctx, 24, Metric.Euclidean, pre["h_reorder_data"], pre["h_map"], pre["h_centroids"],
                              pre["h_segment_start"], pre["h_segment_length"])
    pk, pr = SearchParameter(beam=64).derive(16), SearchParameter(beam=128).derive(16)
    index.build(IndexParameter(24, 16, 1.05), pk, pr, seed=5, want_knn=True)
    yield dict(base=base, queries=queries, pre=pre, index=index, pk=pk, pr=pr)
    index.close()


def test_streamed_build_equals_the_per_partition_entry_points(gpu_ctx, built):
    pre, index = built["pre"], built["index"]
    knn_ref, _ = large.build_knn_for_large(gpu_ctx, NNDescentParameter(16), pre["h_reorder_data"], pre["h_segment_start"],
                                           pre["h_segment_length"])
    assert np.array_equal(index.h_knn, knn_ref)
    sp = index.start_point_view()
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        lo, ln = int(lo), int(ln)
        d_part = torch.from_numpy(pre["h_reorder_data"][lo:lo + ln]).to(gpu_ctx.torch_device)
        d_knn = api.from_u32(gpu_ctx, np.ascontiguousarray(knn_ref[lo:lo + ln]).view(np.uint32))
        d_g = api.build_partition(gpu_ctx, d_part, d_knn, int(sp[s]), 24, built["pk"], 1.05)
        api.reverse_graph(gpu_ctx, d_g)
        api.refine_partition(gpu_ctx, d_part, d_g, int(sp[s]), built["pr"], 1.05)
        assert np.array_equal(index.graph_view()[lo:lo + ln], api.to_u32(d_g))
    assert index.stats["partitions_uploaded"] == 6 and index.stats["h2d_bytes"] == 9000 * 64 * 4


def test_search_equals_the_oracle_replay_streamed_and_resident(gpu_ctx, built):
    pre, index, queries = built["pre"], built["index"], built["queries"]
    sp = SearchParameter(top_k=10, beam=64).derive(24)
    d_q = torch.from_numpy(queries).to(gpu_ctx.torch_device)
    ids, dists, _ = index.search(sp, 2, 1.2, d_q)
    o = oracle.SearchParams(sp.beam, sp.max_iterations, 0, sp.hash_bit, sp.hash_reset_interval, 10)
    routes = oracle.select_segments(queries, pre["h_centroids"], 2, 1.2)
    want_ids = np.full((300, 10), INVALID, np.uint32)
    want_d = np.full((300, 10), np.finfo(np.float32).max, np.float32)
    starts = index.start_point_view()
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        lo, ln = int(lo), int(ln)
        oracle.search_on_sub(pre["h_reorder_data"][lo:lo + ln], index.graph_view()[lo:lo + ln], pre["h_map"][lo:lo + ln],
                             int(starts[s]), queries, routes, s, o, want_ids, want_d)
    assert np.array_equal(ids, want_ids) and np.array_equal(dists, want_d)
    # (no recall threshold here: this set's 16 separate clusters are spread over 6 partitions, and a search
    # only reaches the cluster it enters at; what is checked is that the path computes what the oracle computes)
    visited = int((np.bincount(routes[routes != INVALID], minlength=6) > 0).sum())
    assert index.stats["partitions_searched"] == visited and index.stats["partitions_uploaded"] == visited
    # a single query is routed to two partitions: only those two are uploaded and searched
    one_ids, _, _ = index.search(sp, 2, 1.0, d_q[:1].contiguous())
    assert index.stats["partitions_uploaded"] == 2 and np.array_equal(one_ids[0], oracle_top(queries[:1], pre, index, o, 2, 1.0)[0])
    # keep three partitions in device memory: same results, fewer uploads; then all: none
    assert index.make_resident(10 ** 9, partitions=[0, 2, 4]) == 3
    ids2, dists2, _ = index.search(sp, 2, 1.2, d_q)
    assert np.array_equal(ids2, want_ids) and np.array_equal(dists2, want_d)
    assert index.stats["partitions_uploaded"] <= visited - 1
    assert index.make_resident(10 ** 9) == 6
    ids3, dists3, _ = index.search(sp, 2, 1.2, d_q)
    assert np.array_equal(ids3, want_ids) and np.array_equal(dists3, want_d) and index.stats["partitions_uploaded"] == 0
    # a budget too small for anything keeps nothing
    fresh = large.GLIDE_large(gpu_ctx, 24, Metric.Euclidean, pre["h_reorder_data"], pre["h_map"], pre["h_centroids"],
                              pre["h_segment_start"], pre["h_segment_length"])
    assert fresh.make_resident(1000) == 0
    fresh.close()


def oracle_top(queries, pre, index, o, min_seg, factor):
    routes = oracle.select_segments(queries, pre["h_centroids"], min_seg, factor)
    ids = np.full((queries.shape[0], 10), INVALID, np.uint32)
    d = np.full((queries.shape[0], 10), np.finfo(np.float32).max, np.float32)
    starts = index.start_point_view()
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        lo, ln = int(lo), int(ln)
        oracle.search_on_sub(pre["h_reorder_data"][lo:lo + ln], index.graph_view()[lo:lo + ln], pre["h_map"][lo:lo + ln],
                             int(starts[s]), queries, routes, s, o, ids, d)
    return ids


def test_uint8_rows_give_what_fp32_rows_give(gpu_ctx, built):
    pre, index, queries = built["pre"], built["index"], built["queries"]
    rows_u8 = large.pinned_copy(pre["h_reorder_data"].astype(np.uint8))
    assert np.array_equal(rows_u8.astype(np.float32), pre["h_reorder_data"])
    # partitioning a uint8 set gives the same partitions
    pre8 = large.preprocess_for_large(gpu_ctx, built["base"].astype(np.uint8), 6, 0.1, batch_num=4, seed=2)
    assert np.array_equal(pre8["h_map"], pre["h_map"]) and pre8["h_reorder_data"].dtype == np.uint8
    idx8 = large.GLIDE_large(gpu_ctx, 24, Metric.Euclidean, rows_u8, pre["h_map"], pre["h_centroids"],
                             pre["h_segment_start"], pre["h_segment_length"])
    idx8.build(IndexParameter(24, 16, 1.05), built["pk"], built["pr"], seed=5)
    assert np.array_equal(idx8.graph_view(), index.graph_view())
    assert idx8.stats["h2d_bytes"] == 9000 * 64          # a quarter of the fp32 upload
    sp = SearchParameter(top_k=10, beam=64).derive(24)
    d_q = torch.from_numpy(queries).to(gpu_ctx.torch_device)
    a = idx8.search(sp, 2, 1.2, d_q)
    b = index.search(sp, 2, 1.2, d_q)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    idx8.close()


def test_partition_subsets_fold_into_the_whole_search(gpu_ctx, built):
    """What a multi-GPU search does: every rank searches its own partitions, the per-rank result sets
    are gathered and folded in rank order with the reference's merge network."""
    index, queries = built["index"], built["queries"]
    sp = SearchParameter(top_k=10, beam=64).derive(24)
    d_q = torch.from_numpy(queries).to(gpu_ctx.torch_device)
    sets = [index.search_device(sp, 2, 1.2, d_q, partitions=p) for p in ([0, 1], [2, 3, 4], [5])]
    d_ids = torch.stack([s[0] for s in sets]).contiguous()
    d_d = torch.stack([s[1] for s in sets]).contiguous()
    out_ids = api._u32_tensor(gpu_ctx, (300, 10))
    out_d = gpu_ctx.empty((300, 10), torch.float32)
    gpu_ctx.sync_inputs()
    gpu_ctx.check(gpu_ctx.lib.glide_merge_results(gpu_ctx.handle, d_ids.data_ptr(), d_d.data_ptr(), 3, 300, 10,
                                                  out_ids.data_ptr(), out_d.data_ptr()))
    want_ids, want_d = oracle.merge_results(np.stack([api.to_u32(s[0]) for s in sets]), d_d.cpu().numpy())
    assert np.array_equal(api.to_u32(out_ids), want_ids) and np.array_equal(out_d.cpu().numpy(), want_d)
    whole_ids, whole_d, _ = index.search(sp, 2, 1.2, d_q)
    assert np.array_equal(out_d.cpu().numpy(), whole_d)            # the same distances ...
    same = (np.sort(api.to_u32(out_ids), axis=1) == np.sort(whole_ids, axis=1)).all(axis=1)
    assert same.mean() > 0.97                                      # ... and ids, up to ties at equal distance


@pytest.mark.parametrize("dtype", [np.float32, np.uint8])
def test_preprocess_from_a_file_equals_preprocess_of_the_loaded_array(gpu_ctx, built, tmp_path, dtype):
    """The loader reads with several threads in chunks of 700 rows (13 chunks, the last one ragged)
    while the GPU assigns the chunks already read; partitions, id map and grouped rows equal those of
    the in-memory path, and the rows land in pinned memory unchanged."""
    from glide_b200 import io
    base = built["base"].astype(dtype)
    path = tmp_path / "base.bin"
    io.save_matrix_data(str(path), base)
    assert large.matrix_file_info(gpu_ctx, str(path), dtype) == base.shape
    want = large.preprocess_for_large(gpu_ctx, base, 6, 0.1, batch_num=4, seed=2)
    got = large.preprocess_file_for_large(gpu_ctx, str(path), dtype, 6, 0.1, seed=2, chunk_rows=700, threads=3)
    for key in ("h_map", "h_segment_start", "h_segment_length", "h_centroids", "h_reorder_data"):
        assert np.array_equal(got[key], want[key]), key
    assert got["h_reorder_data"].dtype == dtype and got["load"]["bytes"] == base.nbytes
    # plain read of a row range, no assignment
    rows, nearest, stats = large.load_rows(gpu_ctx, str(path), dtype, first_row=1234, rows=2000, chunk_rows=300, threads=2)
    assert nearest is None and np.array_equal(rows, base[1234:3234]) and stats["total_seconds"] > 0
    with pytest.raises(api.GlideError):
        large.load_rows(gpu_ctx, str(path), dtype, first_row=8000, rows=2000)
    with pytest.raises(IOError):
        large.load_rows(gpu_ctx, str(tmp_path / "missing.bin"), dtype)


def test_merged_index_equals_its_composition_from_oracle_pieces(gpu_ctx, built):
    """The merged index is put together from pieces that each have an oracle: routing of the data
    points (select_segments), the routed multi-partition search for the links (search_on_sub and its
    running merge), the link rule (restated here), reverse edges, and the small path's search on the
    result. Graph and search results must equal that composition bit for bit."""
    pre, index, queries = built["pre"], built["index"], built["queries"]
    rows, cent = pre["h_reorder_data"], pre["h_centroids"]
    seg_start, seg_len = pre["h_segment_start"], pre["h_segment_length"]
    n, deg, C, links, factor = rows.shape[0], 24, 6, 6, 1.3
    assert index.make_resident(10 ** 9) == C
    d_q = torch.from_numpy(queries).to(gpu_ctx.torch_device)
    sp_multi = SearchParameter(top_k=10, beam=64).derive(deg)
    before = index.search(sp_multi, 2, 1.2, d_q)
    stats = index.build_with_merge(factor, link_count=links, link_beam=32)
    # the merge turns the arena into the resident copy of rows and id maps: the routed search still works on it
    after = index.search(sp_multi, 2, 1.2, d_q)
    assert np.array_equal(before[0], after[0]) and np.array_equal(before[1], after[1])
    assert index.stats["partitions_uploaded"] == 0
    got_graph = index.merged_graph()
    # -- the composition --
    local, starts = index.graph_view(), index.start_point_view()
    owner = np.repeat(np.arange(C, dtype=np.uint32), seg_len)
    want = local.copy()
    for s in range(C):
        lo, ln = int(seg_start[s]), int(seg_len[s])
        blk = want[lo:lo + ln]
        blk[blk != INVALID] += lo
    routes = oracle.select_segments(rows, cent, 1, factor)
    for r in range(n):                                   # the point's own partition leaves its list
        keep = [int(x) for x in routes[r] if x != INVALID and x != owner[r]]
        routes[r] = INVALID
        routes[r, :len(keep)] = keep
    p_link = SearchParameter(top_k=links, beam=32).derive(deg)
    o = oracle.SearchParams(p_link.beam, p_link.max_iterations, 0, p_link.hash_bit, p_link.hash_reset_interval, links)
    link_ids = np.full((n, links), INVALID, np.uint32)
    link_d = np.full((n, links), np.finfo(np.float32).max, np.float32)
    gid = np.arange(n, dtype=np.uint32)
    for s in range(C):
        lo, ln = int(seg_start[s]), int(seg_len[s])
        oracle.search_on_sub(rows[lo:lo + ln], local[lo:lo + ln], gid[lo:lo + ln], int(starts[s]), rows, routes, s, o, link_ids, link_d)
    with_links = 0
    for r in range(n):
        row, placed, tail, any_ = want[r], set(), deg, False
        for lid in link_ids[r]:
            if lid == INVALID:
                break
            if (row == lid).any():
                continue
            holes = np.nonzero(row == INVALID)[0]
            if holes.size:
                pos = int(holes[0])
            else:
                while tail > 0 and (tail - 1) in placed:
                    tail -= 1
                if tail == 0:
                    break
                tail -= 1
                pos = tail
            row[pos] = lid
            placed.add(pos)
            any_ = True
        with_links += any_
    assert with_links == stats["rows_with_links"] and 0.02 * n < with_links < n
    oracle.reverse_graph(want)
    assert np.array_equal(got_graph, want)
    cross = owner[want[want != INVALID]] != np.repeat(owner, (want != INVALID).sum(axis=1))
    assert cross.mean() > 0.005                          # edges across partition borders exist
    # -- one search per query over the merged graph --
    sp = SearchParameter(top_k=10, beam=64).derive(deg)
    so = oracle.SearchParams(sp.beam, sp.max_iterations, 0, sp.hash_bit, sp.hash_reset_interval, 10)
    start_global = (seg_start + starts).astype(np.uint32)
    want_ids, want_d = oracle.search(rows, want, cent, start_global, queries, so)
    valid = want_ids != INVALID
    want_ids[valid] = pre["h_map"][want_ids[valid]]
    ids, dists, seconds = index.search_merged(sp, d_q)
    assert np.array_equal(ids, want_ids) and np.array_equal(dists, want_d) and seconds > 0


def test_partitions_delivered_into_resident_buffers_search_like_uploaded_ones(gpu_ctx, built):
    """A rank that did not build a partition receives its rows (fp32), graph rows and id map from the
    owner; here the delivery is a plain copy into the buffers `resident_buffers` hands out, on an
    index whose own host copy of the graph is empty."""
    pre, index, queries = built["pre"], built["index"], built["queries"]
    sp = SearchParameter(top_k=10, beam=64).derive(24)
    d_q = torch.from_numpy(queries).to(gpu_ctx.torch_device)
    want = index.search(sp, 2, 1.2, d_q)
    other = large.GLIDE_large(gpu_ctx, 24, Metric.Euclidean, pre["h_reorder_data"], pre["h_map"], pre["h_centroids"],
                              pre["h_segment_start"], pre["h_segment_length"])
    other.set_start_points(index.start_point_view())
    for s, (lo, ln) in enumerate(zip(pre["h_segment_start"], pre["h_segment_length"])):
        lo, ln = int(lo), int(ln)
        rows, graph, idmap = other.resident_buffers(s)
        assert rows and graph and idmap
        for dst, a in ((rows, pre["h_reorder_data"][lo:lo + ln]), (graph, index.graph_view()[lo:lo + ln]), (idmap, pre["h_map"][lo:lo + ln])):
            a = np.ascontiguousarray(a)
            gpu_ctx.check(gpu_ctx.lib.glide_memcpy_h2d(gpu_ctx.handle, dst, a.ctypes.data, a.nbytes))
        assert other.resident_buffers(s) == (rows, graph, idmap)                                    # stays where it is
    torch.cuda.synchronize()
    got = other.search(sp, 2, 1.2, d_q)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert other.stats["partitions_uploaded"] == 0
    other.close()


def test_bad_arguments_are_refused(gpu_ctx, built):
    pre = built["pre"]
    import ctypes as C
    h = C.c_void_p()
    rows = pre["h_reorder_data"]
    g = large.pinned_empty((rows.shape[0], 24), np.uint32)
    rc = gpu_ctx.lib.glide_large_create(gpu_ctx.handle, rows.ctypes.data, 2, 64, pre["h_segment_start"].ctypes.data,
                                        pre["h_segment_length"].ctypes.data, 6, pre["h_map"].ctypes.data, 24, 0, g.ctypes.data,
                                        C.byref(h))
    assert rc == -2 and not h.value
    parts = np.array([9], np.uint32)
    pk = api._params_c(built["pk"])
    rc = gpu_ctx.lib.glide_large_build(built["index"].handle, parts.ctypes.data, 1, 16, C.byref(pk), None, 1.05, 0, -1.0, 0,
                                       0xFFFFFFFF, 0, None, None)
    assert rc == -1 and b"out of range" in gpu_ctx.lib.glide_last_error(gpu_ctx.handle)
