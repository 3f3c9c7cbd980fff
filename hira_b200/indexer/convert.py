"""Conversion of a CPU-format index (the reference CPUIndexer's levels: centres, radii and
child->parent maps with clusters of any size, indexer/cpu.py:12-22,48-122) into the blocked
arrays the CUDA kernels search.  The block size becomes the largest cluster of any level;
smaller clusters leave free slots (count < block size).  Radii are taken over as stored,
so the search visits exactly the nodes the reference CPU search visits.

A CPU index may be deeper than the blocked layout's three levels (CPUIndexer builds any depth,
indexer/cpu.py:79-120; HiraConfig.num_levels defaults to 5).  Its levels above the third are then
left out: every ball encloses all of its descendants (the radii are triangle-inequality bounds,
indexer/cpu.py:263-311), so a key with q.k >= tau passes every ancestor's gate whatever the depth,
and the selected set under the leaf-tested rule is the same -- the upper levels could only have
skipped whole grandparent blocks earlier.
"""
from __future__ import annotations

import numpy as np


def blocked_from_levels(centers, radii, c2p, values=None):
    """centers[l] (H, K_l, D), radii[l] (H, K_l), c2p[l] (H, K_l) for l < n_levels-1; level 0 = keys.
    Returns a dict of numpy arrays keyed like IndexState.ARRAYS plus "meta" (2 or 3 levels)."""
    centers = [np.asarray(c, dtype=np.float32) for c in centers]
    radii = [np.asarray(r, dtype=np.float32) for r in radii]
    c2p = [np.asarray(c, dtype=np.int64) for c in c2p]
    if len(centers) < 2:
        raise ValueError(f"Unsupported depth {len(centers)}: the blocked index has 2 or 3 levels")
    if len(centers) > 3:          # deeper trees: the lowest three levels select the same keys (see above)
        centers, radii, c2p = centers[:3], radii[:3], c2p[:2]
    n_levels = len(centers)
    H, N, D = centers[0].shape
    K1 = centers[1].shape[1]
    bf = 1
    for l in range(n_levels - 1):
        for h in range(H):
            bf = max(bf, int(np.bincount(c2p[l][h], minlength=centers[l + 1].shape[1]).max()))
    depth = n_levels
    if depth == 3:
        K2 = centers[2].shape[1]
        cap_gp, cap_p = K2, K2 * bf
    else:
        K2, cap_gp, cap_p = 0, 0, K1
    cap_c = cap_p * bf
    V = values.shape[-1] if values is not None else 0
    out = {
        "children": np.zeros((H, cap_c, D), np.float32),
        "values": np.zeros((H, cap_c, V), np.float32) if values is not None else None,
        "slot2token": np.full((H, cap_c), -1, np.int32),
        "parents": np.zeros((H, cap_p, D), np.float32),
        "parent_radii": np.zeros((H, cap_p), np.float32),
        "parent_sqnorm": np.zeros((H, cap_p), np.float32),
        "child_counts": np.zeros((H, cap_p), np.int32),
        "grand_parents": np.zeros((H, cap_gp, D), np.float32) if depth == 3 else None,
        "gp_radii": np.zeros((H, cap_gp), np.float32) if depth == 3 else None,
        "gp_sqnorm": np.zeros((H, cap_gp), np.float32) if depth == 3 else None,
        "gp_counts": np.zeros((H, cap_gp), np.int32) if depth == 3 else None,
        "used": np.zeros((H, 4), np.int32),
    }
    for h in range(H):
        if depth == 3:
            pslot = np.empty(K1, np.int64)
            fill = np.zeros(K2, np.int64)
            for p in range(K1):            # ascending parent id inside each grandparent
                g = c2p[1][h, p]
                pslot[p] = g * bf + fill[g]
                fill[g] += 1
            out["grand_parents"][h] = centers[2][h]
            r2 = radii[2][h]
            out["gp_radii"][h] = np.where(np.isfinite(r2), r2, 0.0)
            out["gp_counts"][h] = fill
            out["used"][h] = (K2 * bf, K2, N, 0)
        else:
            pslot = np.arange(K1, dtype=np.int64)
            out["used"][h] = (K1, 0, N, 0)
        out["parents"][h, pslot] = centers[1][h]
        r1 = radii[1][h]
        out["parent_radii"][h, pslot] = np.where(np.isfinite(r1), r1, 0.0)
        cfill = np.zeros(K1, np.int64)
        for i in range(N):                 # ascending token id inside each parent
            p = c2p[0][h, i]
            s = pslot[p] * bf + cfill[p]
            cfill[p] += 1
            out["children"][h, s] = centers[0][h, i]
            out["slot2token"][h, s] = i
            if values is not None:
                out["values"][h, s] = values[h, i]
        out["child_counts"][h, pslot] = cfill
    out["meta"] = dict(n_heads=H, dim=D, vdim=V, bf=bf, depth=depth, cap_parents=cap_p,
                       dtype="torch.float32", vdtype="torch.float32")
    return out
