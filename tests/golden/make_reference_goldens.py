"""Generates tests/golden/reference_kernels_*.npz: outputs of the REFERENCE's own kernels (through
oracle/ref_harness.cu, built into oracle/_ref/ from the reference tree) on small seeded inputs.
Needs a GPU and oracle/_ref/libglide_ref.so; run from the repository root:

    python tests/golden/make_reference_goldens.py [output_dir]     # default: tests/golden

The inputs are not stored: tests/test_reference_goldens.py regenerates them on the CPU (seeded
generators + the CPU oracle's pipeline, both deterministic) and compares the oracle, in the
reference's summation order, with the stored outputs. The reference kernels are only launched on
inputs for which the oracle reports that every beam ended full (their pruning code dereferences
unfilled slots)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import golden_cases            # noqa: E402
import oracle                  # noqa: E402
from oracle import ref         # noqa: E402
from glide_b200 import api     # noqa: E402


def dev(ctx, a):
    a = np.ascontiguousarray(a)
    return api.from_u32(ctx, a) if a.dtype == np.uint32 else torch.from_numpy(a).to(ctx.torch_device)


def main():
    assert ref.available(), "oracle/_ref/libglide_ref.so is missing (make -C oracle ref)"
    ctx = api.Context(0)
    for name in golden_cases.CASES:
        base, queries, P = golden_cases.inputs(name)
        n, dim, deg = base.shape[0], base.shape[1], golden_cases.DEGREE
        out = {}
        t = [dev(ctx, x) for x in (base, P["graph"], P["centroids"], P["orig_sp"], queries)]
        for beam in golden_cases.BEAMS:
            sp = oracle.SearchParams.derive(beam, deg, top_k=10)
            d_ids = api._u32_tensor(ctx, (queries.shape[0], 10))
            d_d = ctx.empty((queries.shape[0], 10), torch.float32)
            torch.cuda.synchronize()
            assert ref.search(t[0].data_ptr(), dim, t[1].data_ptr(), deg, t[2].data_ptr(), P["centroids"].shape[0], t[3].data_ptr(),
                              t[4].data_ptr(), queries.shape[0], sp, P["metric"], d_ids.data_ptr(), d_d.data_ptr()) == 0
            out[f"search_ids_{beam}"] = api.to_u32(d_ids)
            out[f"search_dists_{beam}"] = d_d.cpu().numpy()
        C = P["centroids"].shape[0]
        d_len = api._u32_tensor(ctx, (C + 1,))
        d_index = api._u32_tensor(ctx, (n, 3))
        torch.cuda.synchronize()
        assert ref.define_partition(t[0].data_ptr(), n, dim, t[2].data_ptr(), C, golden_cases.BOUNDARY, P["metric"],
                                    d_len.data_ptr(), d_index.data_ptr()) == 0
        idx = api.to_u32(d_index)
        out["partition_nearest"] = idx[:, 0].copy()
        out["partition_is_boundary"] = (idx[:, 2] != 0xFFFFFFFF)
        out["partition_lengths"] = api.to_u32(d_len)
        if golden_cases.beams_full(P, base):
            b = [dev(ctx, x) for x in (P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                                       P["mapping"])]
            for with_boundary, key in ((False, "graph_after_build"), (True, "graph_after_boundary")):
                g = api._u32_tensor(ctx, (n, deg))
                g.fill_(-1)
                torch.cuda.synchronize()
                assert ref.build(b[0].data_ptr(), P["reorder_data"].shape[0], dim, b[1].data_ptr(), deg, b[2].data_ptr(),
                                 b[3].data_ptr(), len(P["seg_start"]), b[4].data_ptr(), b[5].data_ptr(), n, deg, P["p_build"],
                                 P["alpha"], P["metric"], with_boundary, g.data_ptr()) == 0
                out[key] = api.to_u32(g)
        out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
        path = os.path.join(out_dir, f"reference_kernels_{name}.npz")
        np.savez_compressed(path, **out)
        print(name, {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")
    large_path(ctx, sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))


def dev_u8(ctx, a):
    return torch.from_numpy(np.ascontiguousarray(a).astype(np.uint8)).to(ctx.torch_device)


def large_path(ctx, out_dir):
    """reference_kernels_large.npz: the reference's reorder_kernel and its large-path kernels
    (instantiated for uint8 rows) on golden_cases.large_inputs()."""
    L = golden_cases.large_inputs()
    base, q, C = L["base"], L["queries"], L["C"]
    n, dim = base.shape
    INVALID = 0xFFFFFFFF
    out = {}
    # reorder_kernel (fp32 rows, the oracle's slots)
    d_rows_out = ctx.empty(L["reorder_data"].shape, torch.float32)
    d_map = api._u32_tensor(ctx, L["mapping"].shape)
    t = [dev(ctx, x) for x in (base, L["seg_index"], L["seg_start"])]
    torch.cuda.synchronize()
    assert ref.reorder(t[0].data_ptr(), d_rows_out.data_ptr(), t[1].data_ptr(), d_map.data_ptr(), t[2].data_ptr(), n, dim) == 0
    out["reorder_map"] = api.to_u32(d_map)
    out["reorder_rows_u8"] = d_rows_out.cpu().numpy().astype(np.uint8)     # the values are integers in 0..255
    # define_partition_for_large_kernel
    d_len, d_index = api._u32_tensor(ctx, (C,)), api._u32_tensor(ctx, (n,))
    d_rows, d_cent = dev_u8(ctx, base), dev(ctx, L["centroids"])
    torch.cuda.synchronize()
    assert ref.define_partition_for_large(d_rows.data_ptr(), n, dim, d_cent.data_ptr(), C, 0, d_len.data_ptr(),
                                          d_index.data_ptr()) == 0
    out["partition_nearest"], out["partition_lengths"] = api.to_u32(d_index), api.to_u32(d_len)
    # select_segment_kernel
    d_q = dev_u8(ctx, q)
    for min_seg, factor in golden_cases.LARGE_ROUTES:
        d_out = api._u32_tensor(ctx, (q.shape[0], C))
        torch.cuda.synchronize()
        assert ref.select_segments(d_q.data_ptr(), q.shape[0], dim, d_cent.data_ptr(), C, min_seg, factor, 0, d_out.data_ptr()) == 0
        out[f"routes_{min_seg}_{factor}"] = api.to_u32(d_out)
    # build_for_large_kernel, only where every beam ends full
    o = L["p_build"]
    for s, part in enumerate(L["parts"]):
        if not part["beams_full"]:
            continue
        g = api._u32_tensor(ctx, (part["ln"], golden_cases.LARGE_DEGREE)); g.fill_(-1)
        d_p, d_knn = dev_u8(ctx, part["rows"]), dev(ctx, part["knn"])
        torch.cuda.synchronize()
        assert ref.build_for_large(d_p.data_ptr(), part["ln"], dim, d_knn.data_ptr(), golden_cases.LARGE_KNN, part["sp"],
                                   golden_cases.LARGE_DEGREE, o, 1.05, 0, g.data_ptr()) == 0
        out[f"build_graph_{s}"] = api.to_u32(g)
    # search_on_sub_kernel + result_merge over all partitions (on the oracle's graphs)
    routes = oracle.select_segments(q, L["centroids"], 2, 1.2, order=oracle.ORDER_REF)
    d_routes = dev(ctx, routes)
    for beam, top_k in golden_cases.LARGE_SEARCHES:
        sp = oracle.SearchParams.derive(beam, golden_cases.LARGE_DEGREE, top_k=top_k)
        d_fi = dev(ctx, np.full((q.shape[0], top_k), INVALID, np.uint32))
        d_fd = dev(ctx, np.full((q.shape[0], top_k), np.finfo(np.float32).max, np.float32))
        for s, part in enumerate(L["parts"]):
            d_p, d_g, d_m = dev_u8(ctx, part["rows"]), dev(ctx, part["graph"]), dev(ctx, part["map"])
            torch.cuda.synchronize()
            assert ref.search_on_sub(d_p.data_ptr(), dim, d_g.data_ptr(), golden_cases.LARGE_DEGREE, d_m.data_ptr(), part["sp"],
                                     d_q.data_ptr(), q.shape[0], d_routes.data_ptr(), C, s, sp, 0, d_fi.data_ptr(),
                                     d_fd.data_ptr()) == 0
        out[f"search_ids_{beam}_{top_k}"], out[f"search_dists_{beam}_{top_k}"] = api.to_u32(d_fi), d_fd.cpu().numpy()
    path = os.path.join(out_dir, "reference_kernels_large.npz")
    np.savez_compressed(path, **out)
    print("large", {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
