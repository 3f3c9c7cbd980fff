"""Shared helpers for the parity tests: seeded inputs, device<->oracle index transfer."""
from __future__ import annotations

import numpy as np
import torch

from hira_b200 import index_state as S
from oracle import oracle as O


def make_keys(h, n, d, seed, dtype=torch.float32, normalize=True, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((h, n, d), generator=g)
    if normalize:
        x = x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    return x.to(dtype).to(device)


def make_queries(hq, d, seed, device="cuda", normalize=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((hq, d), generator=g)
    if normalize:
        q = q / q.norm(dim=-1, keepdim=True)
    return q.float().to(device)


def new_state(h, d, bf, depth, cap_parents, dtype, device="cuda", with_values=True):
    return S.IndexState(n_heads=h, dim=d, vdim=d, bf=bf, depth=depth, cap_parents=cap_parents, dtype=dtype,
                        vdtype=dtype, device=device, with_values=with_values)


def random_centres(h, n, k, seed, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(n, generator=g)[:k] for _ in range(h)]).to(torch.int32).to(device)


def build_both(h, n, d, bf, depth, dtype, seed, *, spare=0, n_iters=1, with_values=True):
    """Builds the same index with the CUDA library and with the oracle. Returns (state, oracle_index, keys, values)."""
    keys = make_keys(h, n, d, seed, dtype)
    vals = make_keys(h, n, d, seed + 1, dtype, normalize=False) if with_values else None
    k1 = -(-n // bf)
    k2 = -(-k1 // bf)
    cap = (k2 * bf if depth == 3 else k1) + spare
    st = new_state(h, d, bf, depth, cap, dtype, with_values=with_values)
    c1 = random_centres(h, n, k1, seed + 2)
    c2 = random_centres(h, k1, k2, seed + 3) if depth == 3 else None
    S.build(st, keys, vals, cent_idx1=c1, cent_idx2=c2, n_iters=n_iters, use_tensor_cores=False)
    torch.cuda.synchronize()
    code = O.HIRA_BF16 if dtype == torch.bfloat16 else O.HIRA_F32
    ox = O.OracleIndex(n_heads=h, dim=d, vdim=d, bf=bf, depth=depth, cap_parents=cap, dtype=code, vdtype=code,
                       with_values=with_values)
    O.build(ox, keys, vals, cent_idx1=c1, cent_idx2=c2, n_iters=n_iters)
    return st, ox, keys, vals


def assert_index_equal(st: S.IndexState, ox: O.OracleIndex, what=""):
    sd = st.state_dict()
    for name in O.OracleIndex.ARRAYS:
        a = getattr(ox, name)
        if a is None:
            continue
        b = O.to_host(sd[name])
        if a.dtype.kind == "f":
            same = np.array_equal(a.view(np.uint32), b.view(np.uint32))
        else:
            same = np.array_equal(a, b)
        if not same:
            bad = np.argwhere(a != b)
            raise AssertionError(f"{what}: array {name} differs at {len(bad)} places, first {bad[:5].tolist()} "
                                 f"oracle={a[tuple(bad[0])]} device={b[tuple(bad[0])]}")


def exact_tau(scores: np.ndarray, frac_keep: float) -> np.ndarray:
    """Per-row threshold = the k-th largest score itself (boundary case), k = ceil(frac*n)."""
    n = scores.shape[-1]
    k = max(1, int(np.ceil(frac_keep * n)))
    return np.sort(scores, axis=-1)[:, n - k].astype(np.float32)


def compact_sets(compact: S.CompactResult):
    """Per query head: (slots ndarray, scores ndarray) from a CompactResult."""
    return [(a.numpy(), b.numpy()) for a, b in compact.to_lists()]
