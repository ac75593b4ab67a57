"""Seeded synthetic data sets with the shapes and value ranges of the benchmark configs.

They stand in for the public ANN benchmark sets the reference was measured on (none of
whose records are used): generation is counter-based (Philox), chunked by rows, so any
row range can be produced without materialising the whole set, and the same seed gives
the same bytes on every machine.

Order of generation: centres, then base rows in row order, then queries.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

_CHUNK = 65536


@dataclass(frozen=True)
class DatasetSpec:
    name: str
    n: int
    dim: int
    n_queries: int
    kind: str            # "uniform" | "int_mixture" | "int_lowrank_mixture" | "scaled_mixture" | "unit_mixture" | "unit_lowrank_mixture"
    centres: int
    metric: str          # "Euclidean" | "Cosine"
    graph_degree: int
    seed: int


CONFIGS = {
    # tiny correctness build: 10,000 x 32 i.i.d. uniform[0,1), 1,000 queries, degree 32
    "cfg0": DatasetSpec("cfg0", 10_000, 32, 1_000, "uniform", 0, "Euclidean", 32, 0),
    # 1M x 128: 1,024-centre mixture, centres U[0,120], sigma 20, rounded, clipped to [0,218]
    "cfg1": DatasetSpec("cfg1", 1_000_000, 128, 10_000, "int_mixture", 1024, "Euclidean", 32, 1),
    # 1M x 960: 256 centres N(0,1), sigma 0.3, each row scaled by U[0.5,1.5]
    "cfg2": DatasetSpec("cfg2", 1_000_000, 960, 1_000, "scaled_mixture", 256, "Euclidean", 64, 2),
    # 10M x 96 cosine: 4,096 centres N(0,1), sigma 0.5, rows normalised
    "cfg3": DatasetSpec("cfg3", 10_000_000, 96, 10_000, "unit_mixture", 4096, "Cosine", 32, 3),
    # A 1M x 128 integer-valued set inside the reference's own size ladders (at most 32 centroids for
    # its 32-entry routing network, kernel_config.cuh:161-171): 32 mixture components, one partition
    # each (~31,000 rows, large enough for NN-descent to run instead of the all-pairs kernel). An
    # isotropic Gaussian component of that size has intrinsic dimension 128, on which no graph search
    # reaches a useful recall (measured: 0.68 at beam 100); here a component varies inside its own
    # random 24-dimensional subspace (per-coordinate sigma 20 as in cfg1) plus isotropic noise of
    # sigma 6, which gives the low intrinsic dimension of real descriptor sets. The reference's kernels
    # and this library are compared on it at equal beam and at recall@10 >= 0.95.
    "cfg1c32": DatasetSpec("cfg1c32", 1_000_000, 128, 10_000, "int_lowrank_mixture", 32, "Euclidean", 32, 11),
    # 100M x 128: as cfg1 with 16,384 centres
    "cfg4": DatasetSpec("cfg4", 100_000_000, 128, 10_000, "int_mixture", 16384, "Euclidean", 32, 4),
    # The two large configs with as many mixture components as BASELINE.json gives them partitions (64
    # and 512) and the low intrinsic dimension of cfg1c32: a partition's kNN graph is then connected and
    # recall@10 >= 0.95 is reachable at those partition counts, which the isotropic 4,096- and
    # 16,384-component sets above cannot give (a partition there spans dozens of separate clusters).
    # cfg3c64: unit vectors; a component varies in its own 24-dimensional subspace (per-coordinate sigma
    # 0.5 before normalisation) plus isotropic noise of sigma 0.15. cfg4c512: as cfg1c32.
    "cfg3c64": DatasetSpec("cfg3c64", 10_000_000, 96, 10_000, "unit_lowrank_mixture", 64, "Cosine", 32, 13),
    "cfg4c512": DatasetSpec("cfg4c512", 100_000_000, 128, 10_000, "int_lowrank_mixture", 512, "Euclidean", 32, 14),
}


def scaled(spec: DatasetSpec, n: int, n_queries: int | None = None) -> DatasetSpec:
    """The same distribution with fewer rows (parity tests run on slices of the big configs)."""
    return DatasetSpec(spec.name + f"_n{n}", n, spec.dim, spec.n_queries if n_queries is None else n_queries,
                       spec.kind, spec.centres, spec.metric, spec.graph_degree, spec.seed)


def _rng(seed: int, stream: int, chunk: int) -> np.random.Generator:
    # key = (seed, stream), counter starts at chunk * 2^64: disjoint counter ranges per chunk
    return np.random.Generator(np.random.Philox(key=[seed, stream], counter=[0, chunk, 0, 0]))


_LATENT = 24          # low-rank mixtures: dimension of a component's own subspace
_LOWRANK_NOISE = 6.0  # int_lowrank_mixture: sigma of the isotropic noise around it (latent: 20 per coordinate)
_UNIT_LATENT_SIGMA, _UNIT_LOWRANK_NOISE = 0.5, 0.15   # unit_lowrank_mixture, before normalisation

_basis_cache: dict = {}


def centres(spec: DatasetSpec) -> np.ndarray | None:
    if spec.kind == "uniform":
        return None
    g = _rng(spec.seed, 0, 0)
    if spec.kind in ("int_mixture", "int_lowrank_mixture"):
        return g.uniform(0.0, 120.0, size=(spec.centres, spec.dim)).astype(np.float32)
    return g.standard_normal(size=(spec.centres, spec.dim), dtype=np.float32)


def _subspaces(spec: DatasetSpec) -> np.ndarray:
    """Low-rank mixtures: per component _LATENT unit directions (centres x _LATENT x dim), scaled so that
    a standard normal latent vector gives the kind's per-coordinate sigma (20, or 0.5 for unit vectors)."""
    key = (spec.seed, spec.centres, spec.dim, spec.kind)
    if key not in _basis_cache:
        g = _rng(spec.seed, 3, 0)
        a = g.standard_normal(size=(spec.centres, _LATENT, spec.dim), dtype=np.float32)
        a /= np.linalg.norm(a, axis=2, keepdims=True)
        sigma = 20.0 if spec.kind == "int_lowrank_mixture" else _UNIT_LATENT_SIGMA
        _basis_cache[key] = a * np.float32(sigma * np.sqrt(spec.dim / _LATENT))
    return _basis_cache[key]


def _round_clip(block: np.ndarray) -> None:
    """Round to integers and clip to [0, 218], in place."""
    np.rint(block, out=block)
    np.maximum(block, np.float32(0.0), out=block)
    np.minimum(block, np.float32(218.0), out=block)


def _rows(spec: DatasetSpec, cent: np.ndarray | None, stream: int, first: int, count: int) -> np.ndarray:
    out = np.empty((count, spec.dim), np.float32)
    done = 0
    while done < count:
        row = first + done
        chunk, off = divmod(row, _CHUNK)
        take = min(count - done, _CHUNK - off)
        g = _rng(spec.seed, stream, chunk)
        if spec.kind == "uniform":
            block = g.random(size=(_CHUNK, spec.dim), dtype=np.float32)[off:off + take]
        else:
            comp = g.integers(0, spec.centres, size=_CHUNK)[off:off + take]
            noise = g.standard_normal(size=(_CHUNK, spec.dim), dtype=np.float32)[off:off + take]
            if spec.kind == "int_mixture":
                block = cent[comp] + np.float32(20.0) * noise
                _round_clip(block)
            elif spec.kind == "int_lowrank_mixture":
                z = g.standard_normal(size=(_CHUNK, _LATENT), dtype=np.float32)[off:off + take]
                basis = _subspaces(spec)
                block = cent[comp] + np.float32(_LOWRANK_NOISE) * noise
                for k in np.unique(comp):
                    rows = np.nonzero(comp == k)[0]
                    block[rows] += z[rows] @ basis[k]
                _round_clip(block)
            elif spec.kind == "scaled_mixture":
                scale = g.uniform(0.5, 1.5, size=_CHUNK).astype(np.float32)[off:off + take]
                block = (cent[comp] + np.float32(0.3) * noise) * scale[:, None]
            elif spec.kind == "unit_mixture":
                block = cent[comp] + np.float32(0.5) * noise
                block /= np.linalg.norm(block, axis=1, keepdims=True).astype(np.float32)
            elif spec.kind == "unit_lowrank_mixture":
                z = g.standard_normal(size=(_CHUNK, _LATENT), dtype=np.float32)[off:off + take]
                basis = _subspaces(spec)
                block = cent[comp] + np.float32(_UNIT_LOWRANK_NOISE) * noise
                for k in np.unique(comp):
                    rows = np.nonzero(comp == k)[0]
                    block[rows] += z[rows] @ basis[k]
                block /= np.linalg.norm(block, axis=1, keepdims=True).astype(np.float32)
            else:
                raise ValueError(spec.kind)
        out[done:done + take] = block
        done += take
    return out


def base_rows(spec: DatasetSpec, first: int = 0, count: int | None = None, cent: np.ndarray | None = None) -> np.ndarray:
    count = spec.n - first if count is None else count
    if cent is None:
        cent = centres(spec)
    return _rows(spec, cent, 1, first, count)


def queries(spec: DatasetSpec, cent: np.ndarray | None = None) -> np.ndarray:
    if cent is None:
        cent = centres(spec)
    return _rows(spec, cent, 2, 0, spec.n_queries)


def make(spec: DatasetSpec) -> tuple[np.ndarray, np.ndarray]:
    cent = centres(spec)
    return base_rows(spec, cent=cent), queries(spec, cent=cent)


# ---------------------------------------------------------------------------------------------
# Device-side generation for the 10M- and 100M-row configs: the same mixtures drawn with torch's
# counter-based CUDA generator, one seeded stream per block of 1,048,576 rows, so that any block can
# be produced on any rank without the others (the numpy generator above would need minutes of host
# time per 100M rows). The values differ from the numpy stream's; the distribution is the same.
# ---------------------------------------------------------------------------------------------
DEVICE_BLOCK = 1 << 20


def device_rows(spec: DatasetSpec, first: int, count: int, device, cent=None, stream: int = 1):
    """Rows [first, first + count) as a float32 tensor on `device` (first must be a multiple of DEVICE_BLOCK
    unless the range lies inside one block)."""
    import torch
    if cent is None:
        cent = torch.from_numpy(centres(spec)).to(device)
    lowrank = spec.kind in ("int_lowrank_mixture", "unit_lowrank_mixture")
    basis = torch.from_numpy(_subspaces(spec)).to(device) if lowrank else None
    out = torch.empty((count, spec.dim), dtype=torch.float32, device=device)
    done = 0
    while done < count:
        row = first + done
        block, off = divmod(row, DEVICE_BLOCK)
        take = min(count - done, DEVICE_BLOCK - off)
        g = torch.Generator(device=device)
        g.manual_seed(((spec.seed * 7 + stream) << 32) + block)
        comp = torch.randint(0, spec.centres, (DEVICE_BLOCK,), generator=g, device=device)[off:off + take]
        noise = torch.randn((DEVICE_BLOCK, spec.dim), generator=g, device=device, dtype=torch.float32)[off:off + take]
        if lowrank:
            # the row's component's subspace applied to its latent vector, 65,536 rows at a time (the
            # gathered bases of a chunk are 0.8 GB)
            z = torch.randn((DEVICE_BLOCK, _LATENT), generator=g, device=device, dtype=torch.float32)[off:off + take]
            sigma = _LOWRANK_NOISE if spec.kind == "int_lowrank_mixture" else _UNIT_LOWRANK_NOISE
            blockv = cent[comp] + sigma * noise
            for lo in range(0, take, 65536):
                hi = min(take, lo + 65536)
                blockv[lo:hi] += torch.bmm(z[lo:hi, None, :], basis[comp[lo:hi]])[:, 0, :]
            if spec.kind == "int_lowrank_mixture":
                blockv = torch.clamp(torch.round(blockv), 0.0, 218.0)
            else:
                blockv = blockv / blockv.norm(dim=1, keepdim=True)
        elif spec.kind == "int_mixture":
            blockv = torch.clamp(torch.round(cent[comp] + 20.0 * noise), 0.0, 218.0)
        elif spec.kind == "unit_mixture":
            blockv = cent[comp] + 0.5 * noise
            blockv = blockv / blockv.norm(dim=1, keepdim=True)
        elif spec.kind == "scaled_mixture":
            scale = torch.rand((DEVICE_BLOCK,), generator=g, device=device)[off:off + take] + 0.5
            blockv = (cent[comp] + 0.3 * noise) * scale[:, None]
        else:
            raise ValueError(spec.kind)
        out[done:done + take] = blockv
        done += take
    return out


def device_queries(spec: DatasetSpec, device, cent=None):
    return device_rows(spec, 0, spec.n_queries, device, cent, stream=2)
