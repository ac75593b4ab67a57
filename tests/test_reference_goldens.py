"""Pins the CPU oracle against stored outputs of the REFERENCE's own kernels (tests/golden/
reference_kernels_*.npz, made on a B200 by tests/golden/make_reference_goldens.py through the
harness in oracle/ref_harness.cu). Runs without a GPU: the inputs are regenerated here from seeds,
the oracle runs in the reference's summation order, and ids, distances, partition assignment and
built graphs must equal the reference's bit for bit."""
import os

import numpy as np
import pytest

import golden_cases
import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
INVALID = 0xFFFFFFFF


def golden(name):
    path = os.path.join(GOLDEN, f"reference_kernels_{name}.npz")
    if not os.path.exists(path):
        pytest.skip(f"{os.path.basename(path)} not generated yet")
    return np.load(path)


@pytest.mark.parametrize("name", sorted(golden_cases.CASES))
def test_oracle_search_equals_reference_kernel_output(name):
    g = golden(name)
    base, queries, P = golden_cases.inputs(name)
    for beam in golden_cases.BEAMS:
        sp = oracle.SearchParams.derive(beam, golden_cases.DEGREE, top_k=10)
        ids, dists = oracle.search(base, P["graph"], P["centroids"], P["orig_sp"], queries, sp, P["metric"],
                                   order=oracle.ORDER_REF, route_order=oracle.ORDER_REF)
        assert np.array_equal(ids, g[f"search_ids_{beam}"])
        assert np.array_equal(dists, g[f"search_dists_{beam}"])


@pytest.mark.parametrize("name", sorted(golden_cases.CASES))
def test_oracle_partition_equals_reference_kernel_output(name):
    g = golden(name)
    base, _, P = golden_cases.inputs(name)
    index, _, lengths = oracle.define_partition(base, P["centroids"], golden_cases.BOUNDARY, P["metric"], oracle.ORDER_REF)
    assert np.array_equal(index[:, 0], g["partition_nearest"])
    assert np.array_equal(index[:, 2] != INVALID, g["partition_is_boundary"])
    assert np.array_equal(lengths, g["partition_lengths"])


@pytest.mark.parametrize("name", sorted(golden_cases.CASES))
def test_oracle_build_equals_reference_kernel_output(name):
    g = golden(name)
    if "graph_after_build" not in g:
        pytest.skip("the reference's build kernels were not run on this case (a beam stayed unfilled)")
    _, _, P = golden_cases.inputs(name)
    assert np.array_equal(P["after_build"], g["graph_after_build"])
    assert np.array_equal(P["after_boundary"], g["graph_after_boundary"])
