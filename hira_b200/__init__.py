"""hira_b200: the decode-time hot path of HIRA ("Louver", hierarchical range-searching
sparse attention) as hand-written CUDA for NVIDIA B200 behind the reference's Python API.

    from hira_b200 import HiraCache, HiraConfig, CUDAIndexer, CUDASearcher, hira_attention
"""
__version__ = "0.1.0"

from .attention import HiraDecodeStep, hira_attention, hira_decode_attention, make_hira_attention, register_hira_attention
from .cache import (THRESHOLD_METHODS, CacheOutput, DeviceMode, HiraCache, HiraCacheLayer, HiraConfig,
                    sample_kth, sample_max, sample_mean_topk)
from .indexer import BaseIndexer, CUDAIndexer
from .searcher import BaseSearcher, CUDASearcher

__all__ = [
    "HiraDecodeStep", "hira_attention", "hira_decode_attention", "make_hira_attention", "register_hira_attention", "THRESHOLD_METHODS", "CacheOutput", "DeviceMode", "HiraCache",
    "HiraCacheLayer", "HiraConfig", "sample_max", "sample_mean_topk", "sample_kth", "BaseIndexer",
    "CUDAIndexer", "BaseSearcher", "CUDASearcher",
]
