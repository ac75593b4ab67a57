"""glide_b200: B200-native drop-in for the hot path of the GLIDE ANN graph index
(partition -> kNN graph -> graph build/refine -> search).

``params``, ``io`` and ``datasets`` are pure host code; ``api`` drives the CUDA library
through its C ABI and needs a GPU at call time.
"""
from .params import (IndexParameter, Metric, NNDescentParameter, PartitionParameter, SearchParameter,
                     adjust_search_params, calculate_hash_bitlen, calculate_hash_reset_interval)

__all__ = ["IndexParameter", "Metric", "NNDescentParameter", "PartitionParameter", "SearchParameter",
           "adjust_search_params", "calculate_hash_bitlen", "calculate_hash_reset_interval"]
