"""Threshold finders.  The reference declares `sample_max(samples, query)` and
`sample_mean_topk(samples, query, k)` and the `THRESHOLD_METHODS` table but both
functions raise NotImplementedError (cache/threshold_finder.py:1-14); here they run on
the device: score the sampled keys against the query, return the maximum, or the mean
of the k largest scores, per query head.

samples: (H_kv, S, D) or (1, H_kv, S, D), float32 or bfloat16 (S <= 4096)
query:   (H_q, D) or (1, H_q, 1, D)
returns: (H_q,) float32 thresholds on the same scale as `query . key`.
"""
from __future__ import annotations

import torch

from .. import _lib as L
from .. import index_state as S


def _prep(samples: torch.Tensor, query: torch.Tensor):
    if samples.ndim == 4:
        samples = samples[0]
    if query.ndim == 4:
        query = query[0, :, 0, :]
    if not samples.is_cuda:
        raise ValueError("samples must be a CUDA tensor (there is no CPU path)")
    q = query.to(device=samples.device, dtype=torch.float32).contiguous()
    if samples.dtype not in (torch.float32, torch.bfloat16):
        samples = samples.float()
    return samples.contiguous(), q


def sample_max(samples, query, q_head_to_kv=None):
    s, q = _prep(samples, query)
    return S.threshold(s, q, L.HIRA_TAU_SAMPLE_MAX, 1, q2kv=q_head_to_kv)


def sample_mean_topk(samples, query, k, q_head_to_kv=None):
    s, q = _prep(samples, query)
    return S.threshold(s, q, L.HIRA_TAU_SAMPLE_MEAN_TOPK, int(k), q2kv=q_head_to_kv)


def sample_kth(samples, query, k, q_head_to_kv=None):
    """k-th largest sample score (k/S estimates the fraction of keys above the threshold)."""
    s, q = _prep(samples, query)
    return S.threshold(s, q, L.HIRA_TAU_SAMPLE_KTH, int(k), q2kv=q_head_to_kv)


THRESHOLD_METHODS = {
    "sample_max": sample_max,
    "sample_mean_topk": sample_mean_topk,
    "sample_kth": sample_kth,
}
