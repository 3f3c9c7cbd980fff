from .base import BaseIndexer
from .cuda import CUDAIndexer

__all__ = ["BaseIndexer", "CUDAIndexer"]
