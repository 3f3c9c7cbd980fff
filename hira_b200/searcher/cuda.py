"""CUDASearcher: same entry point as the reference's (searcher/cuda.py:15-143), one
hand-written CUDA kernel underneath instead of the Triton wrappers.

`search` keeps the reference contract: returns the searcher's reusable dense
`(H_q, N_slots)` buffer (callers that keep a result must clone it,
tests/test_cuda_indexer_searcher.py:318-319) holding `scaling * (q.k)` where a key is
emitted and `output_fill_value` elsewhere; indices are child-slot indices of the blocked
layout.  The default gate/leaf rule is the reference GPU one (keep a node iff
`q.c + r > threshold`, emit every child of a kept parent); `gate="ge", leaf="ge"` gives
the reference CPU rule (exact leaf filter `q.k >= threshold`).

`search_compact` returns the compacted (slot, score) lists that `hira_attention` consumes.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib as L
from .. import index_state as S
from .base import BaseSearcher

DEFAULT_OUTPUT_FILL_VALUE = 0.0

_GATE = {"gt": L.HIRA_GATE_GT, "ge": L.HIRA_GATE_GE}
_LEAF = {"candidates": L.HIRA_LEAF_CANDIDATES, "ge": L.HIRA_LEAF_GE, "gt": L.HIRA_LEAF_GT}


class CUDASearcher(BaseSearcher):

    def __init__(self, block_c=None, output_fill_value: float = DEFAULT_OUTPUT_FILL_VALUE, *,
                 gate: str = "gt", leaf: str = "candidates", assume_unit_query: bool = True):
        super().__init__()
        self.block_c = block_c  # kept for signature parity; the kernel tiles by itself
        self.output_fill_value = float(output_fill_value)
        if gate not in _GATE or leaf not in _LEAF:
            raise ValueError(f"gate must be one of {list(_GATE)}, leaf one of {list(_LEAF)}")
        self.flags = _GATE[gate] | _LEAF[leaf]
        self.assume_unit_query = assume_unit_query
        self._tmp_out: Optional[torch.Tensor] = None
        self._compact: Optional[S.CompactResult] = None
        self._q2kv_cache = {}

    # ---- argument coercion (mirrors kernels/triton_search_wrappers.py:136-180) ----
    @staticmethod
    def _coerce_query(query: torch.Tensor, dim: int, device) -> torch.Tensor:
        if query.ndim == 4:
            if query.shape[0] != 1 or query.shape[2] != 1:
                raise ValueError(f"q must be (H_q,d) or (1,H_q,1,d); got {tuple(query.shape)}")
            query = query[0, :, 0, :]
        if query.ndim != 2 or query.shape[1] != dim:
            raise ValueError(f"q must be (H_q,{dim}) or (1,H_q,1,{dim}); got {tuple(query.shape)}")
        return query.to(device=device, dtype=torch.float32).contiguous()

    def _coerce_q2kv(self, q_head_to_kv, hq: int, hkv: int, device):
        """Returns (int32 device tensor or None for the default grouping, max_group)."""
        if q_head_to_kv is None:
            if hq % hkv != 0:
                raise ValueError(f"H_q={hq} must be divisible by H_kv={hkv} when q_head_to_kv is not given")
            return None, 0
        key = (q_head_to_kv.data_ptr(), q_head_to_kv._version, str(q_head_to_kv.device), hq, hkv)
        hit = self._q2kv_cache.get(key)
        if hit is not None:
            return hit
        host = q_head_to_kv.detach().to("cpu", torch.int64)
        if host.ndim != 1 or host.numel() != hq:
            raise ValueError(f"q_head_to_kv must have shape ({hq},), got {tuple(host.shape)}")
        if host.min() < 0 or host.max() >= hkv:
            raise ValueError("q_head_to_kv entries must lie in [0, H_kv)")
        if hq % hkv == 0 and torch.equal(host, torch.arange(hq) // (hq // hkv)):
            res = (None, 0)
        else:
            res = (host.to(device=device, dtype=torch.int32), int(torch.bincount(host, minlength=hkv).max()))
        self._q2kv_cache = {key: res}
        return res

    def _prepare(self, query, threshold, indexer, q_head_to_kv, scaling):
        st: S.IndexState = getattr(indexer, "state", None)
        if st is None:
            raise ValueError("Indexer is not built: missing children tensor.")
        if hasattr(indexer, "wait_pending_update"):
            indexer.wait_pending_update()                            # an update on a side stream
        st.active_parents = getattr(indexer, "active_parents", 0)   # empty capacity is not visited
        q = self._coerce_query(query, st.dim, st.device)
        hq = q.shape[0]
        threshold = torch.as_tensor(threshold)
        if threshold.shape != (hq,):
            raise ValueError(f"threshold must have shape ({hq},), got {tuple(threshold.shape)}")
        tau = threshold.to(device=st.device, dtype=torch.float32).contiguous()
        if scaling is not None:
            if scaling.shape != (hq,):
                raise ValueError(f"scaling must have shape ({hq},), got {tuple(scaling.shape)}")
            scaling = scaling.to(device=st.device, dtype=torch.float32).contiguous()
        q2kv, max_group = self._coerce_q2kv(q_head_to_kv, hq, st.n_heads, st.device)
        qnorm = None if self.assume_unit_query else q.norm(dim=-1).contiguous()
        return st, q, tau, scaling, q2kv, max_group, qnorm

    # ---- reference entry point ---------------------------------------------------
    def search(self, query, threshold, indexer, q_head_to_kv: Optional[torch.Tensor] = None,
               scaling: Optional[torch.Tensor] = None):
        st, q, tau, scaling, q2kv, max_group, qnorm = self._prepare(query, threshold, indexer, q_head_to_kv, scaling)
        hq = q.shape[0]
        if (self._tmp_out is None or self._tmp_out.device != st.device
                or tuple(self._tmp_out.shape) != (hq, st.cap_children)):
            self._tmp_out = torch.empty((hq, st.cap_children), dtype=torch.float32, device=st.device)
        S.search(st, q, tau, scaling=scaling, qnorm=qnorm, q2kv=q2kv, max_group=max_group, flags=self.flags,
                 out_dense=self._tmp_out)
        if self.output_fill_value != 0.0:
            self._tmp_out.masked_fill_(self._tmp_out == 0, self.output_fill_value)
        return self._tmp_out

    def search_compact(self, query, threshold, indexer, q_head_to_kv: Optional[torch.Tensor] = None,
                       scaling: Optional[torch.Tensor] = None, stats: Optional[torch.Tensor] = None) -> S.CompactResult:
        st, q, tau, scaling, q2kv, max_group, qnorm = self._prepare(query, threshold, indexer, q_head_to_kv, scaling)
        hq = q.shape[0]
        c = self._compact
        if c is None or c.idx.device != st.device or tuple(c.idx.shape) != (hq, st.cap_children):
            c = self._compact = S.alloc_compact(st, hq)
        S.search(st, q, tau, scaling=scaling, qnorm=qnorm, q2kv=q2kv, max_group=max_group, flags=self.flags,
                 compact=c, stats=stats)
        return c

    def synthetic_scanned_fraction(self, query, threshold, indexer, q_head_to_kv=None, scaling=None):
        """How much of the index one search reads (the reference declares this probe,
        searcher/cuda.py:145-239): per query head the child rows scanned and their share."""
        st, q, tau, scaling, q2kv, max_group, qnorm = self._prepare(query, threshold, indexer, q_head_to_kv, scaling)
        hq = q.shape[0]
        stats = S.new_stats(hq, st.device)
        c = S.alloc_compact(st, hq)
        S.search(st, q, tau, scaling=scaling, qnorm=qnorm, q2kv=q2kv, max_group=max_group, flags=self.flags,
                 compact=c, stats=stats)
        scanned = stats[:, 4].to(torch.int64)
        total = int(st.used[:, 2].max().item())
        frac = scanned.to(torch.float32) / float(max(1, total))
        return {
            "scanned_fraction_per_head": frac,
            "scanned_children_per_head": scanned,
            "total_children": total,
            "scanned_fraction_mean": float(frac.mean().item()),
            "raw": stats,
        }
