"""TEST / BASELINE INFRASTRUCTURE -- not a product path.

CPU restatement of the reference's CPU index and of the tensors its CPU searcher hands to
its C++ kernel, so that the reference's compiled `fused_tree_search_v3` (oracle/_ref) can be
driven where the reference's Python sources are not present (the GPU box):

  * `build_levels`  follows CPUIndexer.build (indexer/cpu.py:48-122): level 0 = the keys,
    level l+1 = k-means over the centres of level l with K = size // branching_factor
    (integer division, stop when it reaches 0 or `num_levels` levels exist), radii by the
    triangle inequality (`_refine_parent_ball_radii`, indexer/cpu.py:263-311: per parent the
    max over its children of ||child - parent|| + child radius, -inf for a centre nobody
    chose);
  * `update_levels` follows CPUIndexer.update (indexer/cpu.py:124-190) and
    `_extend_levels_to_depth` (:192-221): an independent sub-index over the new keys, padded
    with singleton levels to the same depth, concatenated level by level with the child->parent
    ids shifted;
  * `searcher_inputs` follows CPUSearcher._prepare_ext_level_data and
    _build_parent_child_adjacency (searcher/cpu.py:280-363): per level fp32 centres, radii,
    child->parent map, size, and the CSR (offsets, children) adjacency.

The k-means itself is faiss in the reference (indexer/cpu.py:223-261:
faiss.Kmeans(d, k, niter=max_iterations, seed=12345 + 9973*h, min_points_per_centroid=1),
then index.search(x, 1)); faiss is not installed and not pinned by the reference, so
`LloydKmeans` stands in for it -- plain Lloyd from `k` distinct random points.  The k-means
ARITHMETIC is therefore not the reference's (parity unpinned for that one call); everything
around it is pinned by tests/golden/cpu_indexer_levels.npz, produced by running the
reference's CPUIndexer with this same class installed as `faiss.Kmeans`.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch


class _FlatIndex:
    def __init__(self, c: np.ndarray):
        self.c = np.ascontiguousarray(c, dtype=np.float32)
        self.csq = (self.c * self.c).sum(1)

    def search(self, x: np.ndarray, k: int = 1, chunk: int = 8192):
        assert k == 1
        n = len(x)
        idx = np.empty(n, np.int64)
        dist = np.empty(n, np.float32)
        for lo in range(0, n, chunk):      # the (n, K) distance matrix is never held whole
            xb = x[lo:lo + chunk]
            d = (xb * xb).sum(1)[:, None] - 2.0 * (xb @ self.c.T) + self.csq[None, :]
            i = d.argmin(1)
            idx[lo:lo + chunk] = i
            dist[lo:lo + chunk] = d[np.arange(len(xb)), i]
        return dist[:, None], idx[:, None]


class LloydKmeans:
    """Drop-in for the subset of faiss.Kmeans the reference uses (constructor keywords,
    `train`, `centroids`, `index.search`)."""

    def __init__(self, d, k, niter=1, verbose=False, gpu=False, seed=0, min_points_per_centroid=1):
        self.d, self.k, self.niter, self.seed = int(d), int(k), int(niter), int(seed)
        self.centroids: Optional[np.ndarray] = None
        self.index: Optional[_FlatIndex] = None

    def train(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rng = np.random.default_rng(self.seed)
        c = x[rng.choice(len(x), self.k, replace=False)].copy()
        for _ in range(self.niter):
            a = _FlatIndex(c).search(x, 1)[1][:, 0]
            order = np.argsort(a, kind="stable")
            sa = a[order]
            starts = np.flatnonzero(np.r_[True, sa[1:] != sa[:-1]])
            sums = np.add.reduceat(x[order], starts, axis=0)
            counts = np.diff(np.r_[starts, len(sa)])
            c[sa[starts]] = sums / counts[:, None].astype(np.float32)   # empty clusters keep their centre
        self.centroids = c.astype(np.float32)
        self.index = _FlatIndex(self.centroids)


def _kmeans_level(x: np.ndarray, K: int, niter: int):
    """(H, L, D) -> centroids (H, K, D), assign (H, L); seeds as indexer/cpu.py:238-239."""
    H, L, D = x.shape
    cents = np.empty((H, K, D), np.float32)
    assign = np.empty((H, L), np.int64)
    for h in range(H):
        km = LloydKmeans(D, K, niter=max(int(niter), 1), seed=12345 + 9973 * h)
        km.train(x[h])
        cents[h] = km.centroids
        assign[h] = km.index.search(np.ascontiguousarray(x[h], np.float32), 1)[1].reshape(-1)
    return cents, assign


def _parent_radii(child_centers, child_radii, assign, parent_centroids):
    """The reference's torch ops, verbatim in meaning (indexer/cpu.py:286-311)."""
    cc, cr = torch.from_numpy(child_centers), torch.from_numpy(child_radii)
    a, pc = torch.from_numpy(assign), torch.from_numpy(parent_centroids)
    H, C, D = cc.shape
    K = pc.shape[1]
    pfc = pc.gather(1, a.unsqueeze(-1).expand(H, C, D))
    diff = (cc - pfc).float()
    contrib = torch.sqrt((diff * diff).sum(dim=-1)).to(cr.dtype) + cr
    out = torch.full((H, K), float("-inf"), dtype=contrib.dtype)
    out.scatter_reduce_(1, a, contrib, reduce="amax", include_self=True)
    return out.numpy()


def build_levels(keys, num_levels: int, branching_factor: int, max_iterations: int = 1) -> List[dict]:
    """keys (H, N, D) fp32 array/tensor -> levels [{centers (H,K,D), radii (H,K), size, c2p (H,K)|None}]."""
    keys = np.ascontiguousarray(torch.as_tensor(keys).float().numpy() if torch.is_tensor(keys) else keys, np.float32)
    H, N, D = keys.shape
    levels = [dict(centers=keys, radii=np.zeros((H, N), np.float32), size=N, c2p=None)]
    size, idx, centers = N, 0, keys
    while True:
        size = size // branching_factor
        if size < 1 or idx + 1 >= num_levels:
            break
        centers, assign = _kmeans_level(centers, size, max_iterations)
        child = levels[idx]
        child["c2p"] = assign
        radii = _parent_radii(child["centers"], child["radii"], assign, centers)
        levels.append(dict(centers=centers, radii=radii, size=centers.shape[1], c2p=None))
        idx += 1
    return levels


def _extend_to_depth(levels: List[dict], depth: int, max_iterations: int):
    while len(levels) < depth:
        child = levels[-1]
        pc, assign = _kmeans_level(child["centers"], 1, max_iterations)
        child["c2p"] = assign
        levels.append(dict(centers=pc, radii=_parent_radii(child["centers"], child["radii"], assign, pc), size=1,
                           c2p=None))


def update_levels(levels: List[dict], new_keys, branching_factor: int, max_iterations: int = 1) -> List[dict]:
    """Appends `new_keys` (H, m, D) as CPUIndexer.update does; returns the same list, modified."""
    depth = len(levels)
    old_sizes = [lv["size"] for lv in levels]
    sub = build_levels(new_keys, depth, branching_factor, max_iterations)
    _extend_to_depth(sub, depth, max_iterations)
    for i in range(depth):
        dst, src = levels[i], sub[i]
        dst["centers"] = np.concatenate([dst["centers"], src["centers"]], axis=1)
        dst["radii"] = np.concatenate([dst["radii"], src["radii"]], axis=1)
        dst["size"] = dst["centers"].shape[1]
        if i >= depth - 1:
            continue
        shifted = src["c2p"] + old_sizes[i + 1]
        dst["c2p"] = shifted if dst["c2p"] is None else np.concatenate([dst["c2p"], shifted], axis=1)
    return levels


def searcher_inputs(levels: List[dict]):
    """The argument lists of fused_tree_search_v3 after the keys/query/threshold:
    (centers, radii, c2p, sizes, offsets, children) as lists of torch tensors."""
    centers, radii, c2ps, sizes, offsets, children = [], [], [], [], [], []
    H = levels[0]["centers"].shape[0]
    for l, lv in enumerate(levels):
        centers.append(torch.from_numpy(np.ascontiguousarray(lv["centers"], np.float32)))
        radii.append(torch.from_numpy(np.ascontiguousarray(lv["radii"], np.float32)))
        sizes.append(int(lv["size"]))
        if lv["c2p"] is None:
            c2ps.append(torch.empty(0, dtype=torch.long))
            offsets.append(torch.empty(0, dtype=torch.long))
            children.append(torch.empty(0, dtype=torch.long))
            continue
        c2p = np.ascontiguousarray(lv["c2p"], np.int64)
        P = levels[l + 1]["size"]
        off = np.empty((H, P + 1), np.int64)
        ch = np.empty((H, c2p.shape[1]), np.int64)
        for h in range(H):
            ch[h] = np.argsort(c2p[h], kind="stable")
            off[h, 0] = 0
            off[h, 1:] = np.bincount(c2p[h], minlength=P).cumsum()
        c2ps.append(torch.from_numpy(c2p))
        offsets.append(torch.from_numpy(off))
        children.append(torch.from_numpy(ch))
    return centers, radii, c2ps, sizes, offsets, children


def load_reference_kernel(root):
    """The reference's fused_tree_search_v3 extension built by oracle/Makefile, or None."""
    import importlib.util
    from pathlib import Path
    so = Path(root) / "oracle" / "_ref" / "hira_torch_ext_v3.so"
    if not so.exists():
        return None
    try:
        spec = importlib.util.spec_from_file_location("hira_torch_ext_v3", str(so))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        return m
    except Exception:
        return None


def reference_search(ext, levels: List[dict], q_hat, tau, scaling=None, q2kv=None, prepared=None):
    """CPUSearcher.search (searcher/cpu.py:44-101) with strategy fused_v3: q_hat (H_q, D) unit
    queries, tau (H_q,), optional scaling (H_q,).  Returns the dense (H_q, N) score tensor."""
    q_hat = torch.as_tensor(q_hat).float().contiguous()
    tau = torch.as_tensor(tau).float().contiguous()
    hq = q_hat.shape[0]
    H = levels[0]["centers"].shape[0]
    if scaling is None:
        scaling = torch.ones((hq,), dtype=torch.float32)
    if q2kv is None:
        q2kv = torch.arange(hq, dtype=torch.long) // (hq // H)
    cs, rs, c2ps, sizes, offs, chs = prepared if prepared is not None else searcher_inputs(levels)
    return ext.fused_tree_search_v3(cs[0], q_hat, tau, cs, rs, c2ps, sizes, offs, chs,
                                    torch.as_tensor(q2kv).long().contiguous(),
                                    torch.as_tensor(scaling).float().contiguous())
