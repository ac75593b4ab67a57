"""The command line tools run as the reference's test.sh runs its binaries (test.sh:27-33): stage
files in the reference's formats, one CSV line per pipeline run; small path and large path."""
import os
import subprocess

import numpy as np
import pytest

import helpers
import oracle
from glide_b200 import api, io
from glide_b200.params import SearchParameter

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "glide_b200", "apps", "bin")


def run(*args):
    r = subprocess.run([str(a) for a in args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_small_pipeline_cli(tmp_path, gpu_ctx):
    if not os.path.exists(os.path.join(BIN, "small_search")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "glide_b200", "apps")], check=True)
    base, queries = helpers.small_dataset("uniform", 8000, 32, 200, seed=17)
    gt = oracle.bruteforce_knn(base, queries, 100, want_dists=False)
    io.save_matrix_data(tmp_path / "base.fbin", base)
    io.save_matrix_data(tmp_path / "query.fbin", queries)
    io.save_matrix_data(tmp_path / "gt", gt)
    pre, knn, graph, csv = tmp_path / "pre", tmp_path / "knn", tmp_path / "graph", tmp_path / "result.csv"
    run(os.path.join(BIN, "small_preprocess"), tmp_path / "base.fbin", pre, csv, 4, 1.04, 0.05, "Euclidean")
    run(os.path.join(BIN, "small_knn"), pre, knn, csv, 32)
    run(os.path.join(BIN, "small_build"), tmp_path / "base.fbin", pre, knn, graph, csv, "Euclidean", 32, 32, 1.05, 64, 128)
    out = run(os.path.join(BIN, "small_search"), tmp_path / "base.fbin", tmp_path / "query.fbin", tmp_path / "gt", pre,
              graph, csv, "Euclidean", 10, 50)
    assert "total_recall" in out
    # stage files in the reference's formats (small_build.cu:43-48)
    seg_start, seg_len = io.load_segment(str(pre) + ".segment")
    assert seg_start.size == 5 and seg_len[:4].sum() == 8000
    mapping = io.load_vector_data(str(pre) + ".map")
    reorder = io.load_matrix_data(str(pre) + ".reorder")
    assert mapping.size == 8000 + seg_len[4] and np.array_equal(reorder, base[mapping])
    knn_m = io.load_matrix_data(knn, np.int32)
    assert knn_m.shape == (mapping.size, 32)
    g = io.load_matrix_data(str(graph) + ".graph", np.uint32)
    sp = io.load_vector_data(str(graph) + ".sp")
    cent = io.load_matrix_data(str(pre) + ".centroid")
    assert g.shape == (8000, 32) and sp.size == 4 and cent.shape == (4, 32)
    # the CSV: header then pre,knn,degree,index,beam,search,QPS,recall (small_preprocess.cu:54-56)
    lines = open(csv).read().strip().splitlines()
    assert lines[0] == "pre_time,knn_time,degree,index_time,beam,search_time,QPS,recall"
    fields = lines[1].split(",")
    assert len(fields) == 8 and fields[2] == "32" and fields[4] == "50"
    recall = float(fields[7])
    assert recall >= 0.95
    # an index built by the tools is searchable through the library, with the same recall
    index = api.GLIDE(gpu_ctx, 32, base, cent)
    index.load(g, sp)
    ids, _ = index.search_host(SearchParameter(top_k=10, beam=50).derive(32), queries)
    assert abs(api.calculate_recall(ids, gt, 10) - recall) < 1e-6


def test_cli_usage_and_bad_file(tmp_path):
    if not os.path.exists(os.path.join(BIN, "small_search")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "glide_b200", "apps")], check=True)
    r = subprocess.run([os.path.join(BIN, "small_knn")], capture_output=True, text=True)
    assert r.returncode != 0 and "preprocess_file knn_file result_file knn_degree" in r.stdout   # small_knn.cu:19-24
    r = subprocess.run([os.path.join(BIN, "small_knn"), str(tmp_path / "nope"), str(tmp_path / "k"), str(tmp_path / "r.csv"), "32"],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "Cannot open file" in r.stderr


def test_large_pipeline_cli(tmp_path, gpu_ctx):
    """The four large-path tools (argv contracts of large_*.cu) against the Python mirror of the same
    path: same partition files, and the same search results for the index the tools built."""
    from glide_b200 import large
    from glide_b200.params import IndexParameter, Metric
    if not os.path.exists(os.path.join(BIN, "large_search")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "glide_b200", "apps")], check=True)
    base, queries = helpers.small_dataset("uniform", 9000, 32, 200, seed=23)
    gt = oracle.bruteforce_knn(base, queries, 100, want_dists=False)
    io.save_matrix_data(tmp_path / "base.fbin", base)
    io.save_matrix_data(tmp_path / "query.fbin", queries)
    io.save_matrix_data(tmp_path / "gt", gt)
    pre, knn, graph, csv = tmp_path / "pre", tmp_path / "knn", tmp_path / "graph", tmp_path / "result.csv"
    run(os.path.join(BIN, "large_preprocess"), tmp_path / "base.fbin", pre, csv, 5, 0.1, "Euclidean", 3)
    run(os.path.join(BIN, "large_knn"), pre, knn, csv, 32)
    run(os.path.join(BIN, "large_build"), pre, knn, graph, csv, "Euclidean", 32, 32, 1.05, 64, 128, 3)
    out = run(os.path.join(BIN, "large_search"), pre, tmp_path / "query.fbin", tmp_path / "gt", graph, csv, "Euclidean", 10, 64,
              2, 1.2)
    assert "total_recall" in out
    seg_start, seg_len = io.load_segment(str(pre) + ".segment")
    mapping = io.load_vector_data(str(pre) + ".map")
    reorder = io.load_matrix_data(str(pre) + ".reorder")
    cent = io.load_matrix_data(str(pre) + ".centroid")
    assert seg_start.size == 5 and seg_len.sum() == 9000 and sorted(mapping.tolist()) == list(range(9000))
    assert np.array_equal(reorder, base[mapping])
    for s, l in zip(seg_start, seg_len):                 # ascending original id inside a partition
        assert (np.diff(mapping[s:s + l].astype(np.int64)) > 0).all()
    # the Python mirror partitions the same way (same seeded sample, same k-means, same assignment)
    P = large.preprocess_for_large(gpu_ctx, base, 5, 0.1, 10, Metric.Euclidean, seed=3)
    assert np.array_equal(P["h_map"], mapping) and np.array_equal(P["h_segment_length"], seg_len)
    assert np.array_equal(P["h_centroids"], cent)
    g = io.load_matrix_data(str(graph) + ".graph", np.uint32)
    sp = io.load_vector_data(str(graph) + ".sp")
    assert g.shape == (9000, 32) and sp.size == 5
    fields = open(csv).read().strip().splitlines()[-1].split(",")
    recall = float(fields[-1])
    assert recall >= 0.95
    # the index the tools wrote, searched through the Python mirror: identical recall
    index = large.GLIDE_large(gpu_ctx, 32, Metric.Euclidean, reorder, mapping, cent, seg_start, seg_len)
    index.load(g, sp)
    import torch
    ids, _, _ = index.search(SearchParameter(top_k=10, beam=64).derive(32), 2, 1.2, torch.from_numpy(queries).to(gpu_ctx.torch_device))
    assert abs(api.calculate_recall(ids, gt, 10) - recall) < 1e-6
