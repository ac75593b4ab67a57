"""World-size-2 (and 3) gloo ranks on CPU: the sharded build's orchestration (row ranges,
merging rows written by different ranks, boundary-row and range exchanges) over the CPU oracle
must give the graph the single-process oracle pipeline gives."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from glide_b200 import sharded  # noqa: E402


def test_split_range_is_a_partition():
    for n in (0, 1, 7, 100, 1001):
        for world in (1, 2, 3, 8):
            parts = [sharded.split_range(n, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


class OracleBackend:
    def __init__(self, base, P, graph_i32):
        import oracle
        self.o, self.base, self.P, self.g = oracle, base, P, graph_i32

    def _view(self):
        return self.g.numpy().view(np.uint32)

    def build_range(self, first_row, row_count):
        o, P, n = self.o, self.P, self.base.shape[0]
        g = self._view()
        end = first_row + row_count
        if first_row < n and row_count:
            o.build_rows(P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                         P["mapping"], n, g.shape[1], P["p_build"], P["alpha"], P["metric"], P["order"], graph=g,
                         first=first_row, count=min(end, n) - first_row, threads=1)
        if end > n and row_count:
            # boundary copies [max(first,n), end): run the oracle on that sub-range only
            lo = max(first_row, n)
            rd, knn, mp_ = P["reorder_data"], P["knn"].view(np.uint32), P["mapping"]
            full = g.copy()
            o.build_boundary(rd, knn, n, int(P["local_sp"][-1]), mp_, full, P["p_build"], P["alpha"], P["metric"],
                             P["order"], threads=1)
            rows = mp_[lo:end]
            g[rows] = full[rows]
        return 0.0

    def reverse(self):
        self.o.reverse_graph(self._view())
        return 0.0

    def refine_range(self, snapshot, first, count):
        o, P = self.o, self.P
        out = o.refine(self.base, snapshot.numpy().view(np.uint32), P["centroids"], P["orig_sp"], P["p_refine"],
                       P["alpha"], P["metric"], P["order"], threads=1)
        self._view()[first:first + count] = out[first:first + count]
        return 0.0


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import helpers
    base, _ = helpers.small_dataset("int", 1200, 16, 10, seed=4)
    P = helpers.oracle_pipeline(base, centroid_num=3, boundary_factor=1.15)
    n = base.shape[0]
    graph = torch.full((n, 16), -1, dtype=torch.int32)
    backend = OracleBackend(base, P, graph)
    coll = sharded.Collectives(dist, world, rank)
    sharded.build_sharded(backend, coll, n, int(P["seg_len"][-1]), graph, torch.from_numpy(P["mapping"].astype(np.int64)))
    ok = np.array_equal(graph.numpy().view(np.uint32), P["graph"])
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_build_equals_single_process(tmp_path, world):
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"
