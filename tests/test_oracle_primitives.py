"""CPU checks of the oracle's primitives: distance orders, the warp bitonic network,
parameter derivation (against the values the reference's formulas give) and recall."""
import numpy as np
import pytest

import oracle
from glide_b200 import params as P


def test_distance_orders_agree_with_float64():
    rng = np.random.default_rng(0)
    for dim in (1, 3, 32, 96, 100, 128, 960):
        a, b = rng.random(dim, dtype=np.float32), rng.random(dim, dtype=np.float32)
        ref = float(np.sqrt(np.sum((a.astype(np.float64) - b.astype(np.float64)) ** 2)))
        for order in (oracle.ORDER_REF, oracle.ORDER_TEAM, oracle.ORDER_WARP):
            assert oracle.distance(a, b, oracle.EUCLIDEAN, order) == pytest.approx(ref, rel=1e-5)
            assert oracle.distance(a, b, oracle.COSINE, order) == pytest.approx(ref * ref, rel=1e-5)


def test_distance_is_order_independent_on_integer_data():
    # sums of squares below 2^24 are exact in fp32 whatever the order
    rng = np.random.default_rng(1)
    for _ in range(20):
        a = rng.integers(0, 219, 128).astype(np.float32)
        b = rng.integers(0, 219, 128).astype(np.float32)
        exact = float(np.sum((a.astype(np.int64) - b.astype(np.int64)) ** 2))
        assert oracle.distance(a, b, oracle.COSINE, oracle.ORDER_REF) == exact
        assert oracle.distance(a, b, oracle.COSINE, oracle.ORDER_TEAM) == exact
        assert oracle.distance(a, b, oracle.EUCLIDEAN, oracle.ORDER_TEAM) == np.sqrt(np.float32(exact))
        assert oracle.distance(a, b, oracle.COSINE, oracle.ORDER_WARP) == exact


def _textbook_bitonic(keys, vals, n_regs):
    """Plain bitonic sort over element index e = N*lane + i with a comparator that never
    exchanges equal keys: the formulation the CUDA kernels use."""
    k, v = keys.copy(), vals.copy()
    total = 32 * n_regs
    size = 2
    while size <= total:
        stride = size // 2
        while stride >= 1:
            for e in range(total):
                o = e ^ stride
                if o <= e:
                    continue
                asc = (size == total) or ((e & size) == 0)
                if k[e] != k[o] and ((k[e] < k[o]) != asc):
                    k[e], k[o] = k[o], k[e]
                    v[e], v[o] = v[o], v[e]
            stride //= 2
        size *= 2
    return k, v


@pytest.mark.parametrize("n_regs", [1, 2, 4, 8, 16])
def test_network_sorts_and_matches_textbook_form_with_ties(n_regs):
    rng = np.random.default_rng(n_regs)
    total = 32 * n_regs
    for trial in range(6):
        if trial % 2 == 0:
            keys = rng.random(total, dtype=np.float32)
        else:  # many ties
            keys = rng.integers(0, 6, total).astype(np.float32)
        vals = np.arange(total, dtype=np.uint32)
        k, v = oracle.warp_sort(keys, vals, n_regs)
        assert np.all(np.diff(k) >= 0)
        assert sorted(v.tolist()) == list(range(total))
        assert np.array_equal(keys[v], k)
        tk, tv = _textbook_bitonic(keys, vals, n_regs)
        assert np.array_equal(tk, k) and np.array_equal(tv, v)


def test_sort_with_key_value_layout():
    # element j starts in lane j%32 register j/32 and is read back at N*lane+i
    keys = np.array([3, 1, 2, 1, 0], np.float32)
    vals = np.arange(5, dtype=np.uint32)
    v, k = oracle.sort_with_key_value(32, vals, keys)
    assert k.tolist() == [0, 1, 1, 2, 3]
    assert set(v[1:3].tolist()) == {1, 3}
    v64, k64 = oracle.sort_with_key_value(64, vals, keys)
    assert k64.tolist() == [0, 1, 1, 2, 3]


# (beam_in, degree) -> (beam, max_iterations, hash_bit, reset_interval): what params.cuh:49-99
# yields, as tabulated from the reference's formulas for the benchmark configurations
DERIVED = {
    (10, 32): (32, 12, 8, 3), (20, 32): (32, 23, 8, 3), (32, 32): (32, 36, 8, 3), (35, 32): (64, 39, 8, 2),
    (50, 32): (64, 56, 8, 2), (64, 32): (64, 71, 8, 2), (100, 32): (128, 111, 9, 4), (128, 32): (128, 139, 9, 4),
    (200, 32): (224, 211, 9, 1), (256, 32): (256, 267, 10, 8),
    (10, 64): (32, 12, 8, 1), (35, 64): (64, 39, 8, 1), (64, 64): (64, 71, 8, 1), (100, 64): (128, 111, 9, 2),
    (128, 64): (128, 139, 9, 2), (200, 64): (224, 211, 10, 4), (256, 64): (256, 267, 10, 4),
}


@pytest.mark.parametrize("key", sorted(DERIVED))
def test_parameter_derivation_matches_reference_formulas(key):
    beam_in, degree = key
    want = DERIVED[key]
    o = oracle.SearchParams.derive(beam_in, degree)
    assert (o.beam, o.max_iterations, o.hash_bit, o.hash_reset_interval) == want
    p = P.SearchParameter(beam=beam_in).derive(degree)
    assert (p.beam, p.max_iterations, p.hash_bit, p.hash_reset_interval) == want


def test_adjust_search_params_keeps_explicit_values():
    assert P.adjust_search_params(0, 200, 40) == (200, 64)
    assert P.adjust_search_params(50, 0, 32) == (50, 32) or P.adjust_search_params(50, 0, 32)[0] >= 36
    # max < min -> min wins only if larger than the current max (params.cuh:88-93)
    assert P.adjust_search_params(100, 10, 32) == (100, 32)


def test_recall_definition():
    nb = np.array([[1, 2, 3], [4, 5, 6]], np.uint32)
    tr = np.array([[3, 2, 9, 1], [7, 8, 9, 4]], np.uint32)
    assert oracle.recall(nb, tr, 3) == pytest.approx((2 / 3 + 0) / 2)
    from glide_b200.api import calculate_recall
    assert calculate_recall(nb, tr, 3) == pytest.approx((2 / 3 + 0) / 2)


def test_bruteforce_matches_numpy():
    rng = np.random.default_rng(3)
    base = rng.random((500, 24), dtype=np.float32)
    q = rng.random((20, 24), dtype=np.float32)
    ids, d = oracle.bruteforce_knn(base, q, 10)
    d2 = ((q[:, None, :].astype(np.float64) - base[None].astype(np.float64)) ** 2).sum(-1)
    want = np.argsort(d2, axis=1, kind="stable")[:, :10]
    assert np.array_equal(ids, want.astype(np.uint32))
    assert np.allclose(d, np.sqrt(np.take_along_axis(d2, want, 1)), rtol=1e-5)


def test_warp_order_equals_reference_order_for_odd_dims():
    # dim % 4 != 0: the kernels fall back to scalar lane-strided sums, the reference's own order
    rng = np.random.default_rng(5)
    for dim in (1, 30, 33, 101):
        a, b = rng.random(dim, dtype=np.float32), rng.random(dim, dtype=np.float32)
        assert oracle.distance(a, b, oracle.EUCLIDEAN, oracle.ORDER_WARP) == oracle.distance(a, b, oracle.EUCLIDEAN, oracle.ORDER_REF)


def test_narrow_candidate_sort_equals_the_64_slot_network():
    """The kernels sort degree <= 32 candidates with a 32-slot network although the reference uses 64
    slots (upper half padding): the first `degree` outputs agree, ties included, as long as every
    FLT_MAX slot carries the padding id; a FLT_MAX key with a valid id breaks it (the kernels then
    use the 64-slot network)."""
    rng = np.random.default_rng(1)
    fmax = np.finfo(np.float32).max

    def trial(deg, irregular):
        nvalid = int(rng.integers(0, deg + 1))
        keys = np.full(deg, fmax, np.float32)
        vals = np.full(deg, 0xFFFFFFFF, np.uint32)
        idx = rng.permutation(deg)[:nvalid]
        keys[idx] = rng.integers(0, 5, nvalid).astype(np.float32)
        vals[idx] = rng.integers(0, 1000000, nvalid)
        if irregular and nvalid < deg:
            free = sorted(set(range(deg)) - set(idx.tolist()))
            vals[rng.choice(free)] = 777
        k64 = np.full(64, fmax, np.float32)
        v64 = np.full(64, 0xFFFFFFFF, np.uint32)
        for j in range(deg):  # element j in lane j % 32, register j // 32 (search_kernel.cuh:22-27)
            k64[(j % 32) * 2 + j // 32] = keys[j]
            v64[(j % 32) * 2 + j // 32] = vals[j]
        sk, sv = oracle.warp_sort(k64, v64, 2)
        k32 = np.full(32, fmax, np.float32)
        v32 = np.full(32, 0xFFFFFFFF, np.uint32)
        k32[:deg], v32[:deg] = keys, vals
        a, b = oracle.warp_sort(k32, v32, 1)
        return np.array_equal(sk[:deg], a[:deg]) and np.array_equal(sv[:deg], b[:deg])

    for deg in (5, 16, 24, 32):
        assert all(trial(deg, False) for _ in range(3000))
    assert not all(trial(32, True) for _ in range(200))
