"""Searcher interface (reference: searcher/base.py:4-6)."""
from abc import ABC


class BaseSearcher(ABC):
    def search(self, query, threshold, indexer, scaling=None):
        raise NotImplementedError
