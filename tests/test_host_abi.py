"""Host-side checks that need no GPU: file formats, parameter helpers of the C ABI, and
that the shared library loads and exports every symbol the header declares."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from glide_b200 import _lib, io, params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(glide_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = declared_symbols()
    assert len(declared) >= 30
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    # and the Python binding table covers the header exactly
    assert set(_lib.SIGNATURES) == declared


def test_abi_parameter_helpers_match_python_mirror():
    lib = _lib.load()
    for beam_in in (10, 32, 35, 64, 100, 200, 256, 500):
        for degree in (16, 32, 64, 96, 128):
            p = params.SearchParameter(beam=beam_in).derive(degree)
            b, m = C.c_uint32(beam_in), C.c_uint32(0)
            lib.glide_adjust_search_params(0, C.byref(m), C.byref(b))
            bits = lib.glide_calculate_hash_bitlen(b.value, degree, 0.5, 0)
            interval = lib.glide_calculate_hash_reset_interval(b.value, degree, 0.5, bits)
            assert (b.value, m.value, bits, interval) == (p.beam, p.max_iterations, p.hash_bit, p.hash_reset_interval)


def test_sample_ids_are_distinct_and_seeded():
    from glide_b200.api import sample_ids
    a = sample_ids(100000, 1000, 5)
    b = sample_ids(100000, 1000, 5)
    c = sample_ids(100000, 1000, 6)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert len(set(a.tolist())) == 1000 and a.max() < 100000


def test_start_point_select_is_seeded_and_in_range():
    from glide_b200.api import start_point_select
    seg_start = np.array([0, 40, 100, 100], np.uint32)
    seg_len = np.array([40, 60, 0, 25], np.uint32)  # an empty segment must not crash
    mapping = np.arange(125, dtype=np.uint32)[::-1].copy()
    l1, o1 = start_point_select(seg_start, seg_len, mapping, 9)
    l2, o2 = start_point_select(seg_start, seg_len, mapping, 9)
    assert np.array_equal(l1, l2) and np.array_equal(o1, o2)
    assert l1[0] < 40 and l1[1] < 60 and l1[2] == 0 and l1[3] < 25
    assert o1[0] == mapping[l1[0]] and o1[1] == mapping[40 + l1[1]]


def test_matrix_segment_vector_roundtrip(tmp_path):
    m = np.arange(12, dtype=np.float32).reshape(3, 4)
    io.save_matrix_data(tmp_path / "m.fbin", m)
    raw = open(tmp_path / "m.fbin", "rb").read()
    assert raw[:8] == np.array([3, 4], np.uint32).tobytes() and len(raw) == 8 + 48  # load.cuh:10-30
    assert np.array_equal(io.load_matrix_data(tmp_path / "m.fbin"), m)
    g = np.array([[1, 2], [3, 0xFFFFFFFF]], np.uint32)
    io.save_matrix_data(tmp_path / "g.graph", g)
    assert np.array_equal(io.load_matrix_data(tmp_path / "g.graph", np.uint32), g)
    io.save_segment(tmp_path / "s.segment", [0, 5], [5, 7])
    raw = open(tmp_path / "s.segment", "rb").read()
    assert np.frombuffer(raw, np.uint32).tolist() == [2, 0, 5, 5, 7]  # load.cuh:33-68
    s, l = io.load_segment(tmp_path / "s.segment")
    assert s.tolist() == [0, 5] and l.tolist() == [5, 7]
    io.save_vector_data(tmp_path / "v.map", [9, 8, 7])
    assert io.load_vector_data(tmp_path / "v.map").tolist() == [9, 8, 7]


def test_bad_files_raise(tmp_path):
    with pytest.raises(IOError):
        io.load_matrix_data(tmp_path / "missing.fbin")
    p = tmp_path / "short.fbin"
    with open(p, "wb") as f:
        np.array([10, 4], np.uint32).tofile(f)
        np.zeros(7, np.float32).tofile(f)
    with pytest.raises(IOError):
        io.load_matrix_data(p)
    p2 = tmp_path / "hdr.fbin"
    open(p2, "wb").write(b"\x01\x00")
    with pytest.raises(IOError):
        io.load_matrix_data(p2)
    with pytest.raises(IOError):
        io.load_segment(p2)


def test_matrix_file_info_reads_the_header_and_checks_the_length(tmp_path):
    """Host-only part of the loader: header fields, and a file shorter than its header says is an error."""
    lib = _lib.load()
    m = np.arange(12 * 8, dtype=np.float32).reshape(12, 8)
    path = tmp_path / "m.fbin"
    io.save_matrix_data(str(path), m)
    rows, dim = C.c_uint32(), C.c_uint32()
    assert lib.glide_matrix_file_info(str(path).encode(), 4, C.byref(rows), C.byref(dim)) == 0
    assert (rows.value, dim.value) == (12, 8)
    # the same bytes hold 12 x 8 uint8 rows and then some: accepted; as fp64-sized elements: refused
    assert lib.glide_matrix_file_info(str(path).encode(), 1, C.byref(rows), C.byref(dim)) == 0
    assert lib.glide_matrix_file_info(str(path).encode(), 8, C.byref(rows), C.byref(dim)) == -1
    short = tmp_path / "short.fbin"
    short.write_bytes(path.read_bytes()[:-4])
    assert lib.glide_matrix_file_info(str(short).encode(), 4, C.byref(rows), C.byref(dim)) == -5
    assert lib.glide_matrix_file_info(str(tmp_path / "none.fbin").encode(), 4, C.byref(rows), C.byref(dim)) == -5
    assert lib.glide_matrix_file_info(None, 4, C.byref(rows), C.byref(dim)) == -1


def test_metric_parse():
    assert params.Metric.parse("Euclidean") == params.Metric.Euclidean
    assert params.Metric.parse("Cosine") == params.Metric.Cosine
    with pytest.raises(ValueError):
        params.Metric.parse("L1")


def test_no_product_module_imports_the_oracle():
    pkg = os.path.join(ROOT, "glide_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, fn), errors="ignore").read()
                assert "import oracle" not in text and "from oracle" not in text and "glide_oracle" not in text, fn


def test_bench_reference_arm_prints_one_contract_line_without_a_gpu():
    """`bench.py --impl reference` on a box without a CUDA device: one JSON line on stdout with the keys the
    bench contract names (the CPU arm then runs exact brute force, there being no index to search)."""
    import json
    import subprocess
    import sys
    import torch
    if torch.cuda.is_available():
        pytest.skip("with a GPU this arm searches a GPU-built index: covered by the GPU bench itself")
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--rows", "20000",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "queries/s" and line["higher_is_better"] is True
    assert line["steps"] == 1 and line["warmup"] == 0 and line["n_gpus"] == 1 and line["value"] > 0
    assert set(line["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"}
    assert line["e2e"] == {"value": line["value"], "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]
