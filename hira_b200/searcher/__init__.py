from .base import BaseSearcher
from .cuda import CUDASearcher

__all__ = ["BaseSearcher", "CUDASearcher"]
