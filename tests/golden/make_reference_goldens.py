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


if __name__ == "__main__":
    main()
