from .hira_cache import CacheOutput, HiraCache, HiraCacheLayer
from .hira_config import DeviceMode, HiraConfig
from .threshold_finder import THRESHOLD_METHODS, sample_kth, sample_max, sample_mean_topk

__all__ = ["CacheOutput", "HiraCache", "HiraCacheLayer", "DeviceMode", "HiraConfig", "THRESHOLD_METHODS",
           "sample_max", "sample_mean_topk", "sample_kth"]
