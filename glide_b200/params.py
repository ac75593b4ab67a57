"""Parameter structs and derivations of the GLIDE pipeline.

Mirrors the reference's ``params.cuh``: ``Metric`` (:5-8), ``PartitionParameter``
(:10-15), ``NNDescentParameter`` (:17-25), ``IndexParameter`` (:27-35),
``SearchParameter`` (:37-47) and the helpers ``calculate_hash_bitlen`` (:49-66),
``calculate_hash_reset_interval`` (:68-80), ``adjust_search_params`` (:82-99).
Same names, defaults and arithmetic, so callers written against the reference read
the same here.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass


class Metric(enum.IntEnum):
    Euclidean = 0
    Cosine = 1

    @staticmethod
    def parse(name: str) -> "Metric":
        """The CLI spelling used by the reference's mains (small_build.cu:55-59)."""
        if name == "Euclidean":
            return Metric.Euclidean
        if name == "Cosine":
            return Metric.Cosine
        raise ValueError(f"unknown metric {name!r} (expected 'Euclidean' or 'Cosine')")


@dataclass
class PartitionParameter:
    centroid_num: int = 10
    boundary_factor: float = 1.05
    sample_factor: float = 0.01
    metric: Metric = Metric.Euclidean


@dataclass
class NNDescentParameter:
    graph_degree: int = 64
    intermediate_graph_degree: int = 128
    max_iterations: int = 20
    termination_threshold: float = 0.0001

    def __init__(self, graph_degree: int, max_iterations: int = 20, termination_threshold: float = 0.0001):
        self.graph_degree = int(graph_degree)
        self.intermediate_graph_degree = int(1.5 * graph_degree)
        self.max_iterations = max_iterations
        self.termination_threshold = termination_threshold


@dataclass
class IndexParameter:
    graph_degree: int = 32
    knn_degree: int = 32
    relaxant_factor: float = 1.05
    metric: Metric = Metric.Euclidean


def _f32(x: float) -> float:
    return C.c_float(x).value


def calculate_hash_bitlen(beam: int, graph_degree: int, hashmap_max_fill_rate: float, hashmap_min_bitlen: int) -> int:
    max_visited_nodes = beam + graph_degree
    min_bitlen, max_bitlen = 8, 13
    if min_bitlen < hashmap_min_bitlen:
        min_bitlen = hashmap_min_bitlen
    hash_bitlen = min_bitlen
    fill = _f32(hashmap_max_fill_rate)
    while max_visited_nodes > _f32((1 << hash_bitlen) * fill):
        hash_bitlen += 1
    return min(hash_bitlen, max_bitlen)


def calculate_hash_reset_interval(beam: int, graph_degree: int, hashmap_max_fill_rate: float, hash_bitlen: int) -> int:
    interval = 1
    fill = _f32(hashmap_max_fill_rate)
    while True:
        max_visited_nodes = beam + graph_degree * (interval + 1)
        if max_visited_nodes > _f32((1 << hash_bitlen) * fill):
            break
        interval += 1
    return interval


def adjust_search_params(min_iterations: int, max_iterations: int, beam: int) -> tuple[int, int]:
    """Returns (max_iterations, beam) as the reference leaves them in its by-reference arguments."""
    _max = max_iterations
    if max_iterations == 0:
        _max = int(1 + min(beam * 1.1, beam + 10.0))
    if max_iterations < min_iterations:
        _max = min_iterations
    if max_iterations < _max:
        max_iterations = _max
    if beam % 32:
        beam += 32 - (beam % 32)
    return max_iterations, beam


@dataclass
class SearchParameter:
    top_k: int = 10
    beam: int = 100
    max_iterations: int = 0
    min_iterations: int = 0
    hash_bit: int = 0
    hash_max_fill_rate: float = 0.5
    hashmap_min_bitlen: int = 0
    hash_reset_interval: int = 1
    search_block_size: int = 0

    def derive(self, degree_for_hash: int) -> "SearchParameter":
        """What every reference main does after filling beam/top_k (small_search.cu:98-107,
        small_build.cu:61-82): adjust, then size the visited hash for `degree_for_hash`."""
        self.max_iterations, self.beam = adjust_search_params(self.min_iterations, self.max_iterations, self.beam)
        self.hash_bit = calculate_hash_bitlen(self.beam, degree_for_hash, self.hash_max_fill_rate,
                                              self.hashmap_min_bitlen)
        self.hash_reset_interval = calculate_hash_reset_interval(self.beam, degree_for_hash,
                                                                 self.hash_max_fill_rate, self.hash_bit)
        return self
