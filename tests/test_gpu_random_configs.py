"""Seeded random configurations (depth, branching, dimension, dtype, GQA group, threshold quantile,
gate / leaf rule, number of appends, attention splits): search, appends through the scan folded into
the search, and sparse attention against the CPU oracle.  Index sets and index contents bit-exact,
attention within the dtype's tolerance."""
import random

import numpy as np
import pytest
import torch

from hira_b200 import _lib as L
from hira_b200 import index_state as S
from oracle import oracle as O

from util import assert_index_equal, build_both, exact_tau, make_keys, make_queries
from test_gpu_parity import FLAG_CASES, _run_search_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", list(range(24)))
def test_random_configuration(seed):
    rng = random.Random(1000 + seed)
    depth = rng.choice([2, 3, 3])
    bf = rng.choice([1, 2, 4, 5, 8, 12, 16, 32, 32, 48, 64])
    d = rng.choice([16, 32, 64, 96, 128, 128, 192, 256])
    dtype = rng.choice([torch.float32, torch.bfloat16, torch.bfloat16])
    h = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 3, 4, 4, 5, 8])
    n = rng.choice([37, 200, 777, 1500, 4096, 5000]) if bf > 1 else rng.choice([37, 200, 300])
    steps = rng.choice([0, 5, 17])
    frac = rng.choice([0.0, 0.02, 0.1, 0.5, 1.0])
    flags = rng.choice(FLAG_CASES)
    st, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=100 + seed, spare=(steps + 2) * bf)
    hq = h * group
    q = make_queries(hq, d, seed=seed)
    all_d, all_k = O.search(ox, q, np.full((hq,), -np.inf, np.float32), flags=O.GATE_GT)
    if frac == 0.0:
        tau_np = np.full((hq,), 1e30, np.float32)
    elif frac == 1.0:
        tau_np = np.full((hq,), -np.inf, np.float32)
    else:
        tau_np = np.stack([exact_tau(all_d[i][all_k[i] > 0][None, :], frac)[0] for i in range(hq)])
    tau = torch.from_numpy(tau_np).cuda()
    scaling = torch.linspace(0.5, 2.0, hq, device="cuda")
    _run_search_case(st, ox, q, tau, flags, scaling=scaling)
    if steps:
        new_k = make_keys(h, steps, d, 500 + seed, dtype)
        new_v = make_keys(h, steps, d, 600 + seed, dtype, normalize=False)
        scan = S.new_scan_slots(st)
        comp = S.alloc_compact(st, hq)
        for i in range(steps):
            S.search(st, q, tau, flags=flags, compact=comp, scan_key=new_k[:, i], scan_out=scan)
            S.append_scanned(st, new_k[:, i:i + 1], new_v[:, i:i + 1], scan)
            O.append(ox, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())
        torch.cuda.synchronize()
        assert int(st.status.item()) == int(ox.status[0])
        assert_index_equal(st, ox, "appends through the folded scan")
        _run_search_case(st, ox, q, tau, flags, scaling=scaling)
    fl = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
    _, compact = S.search(st, q, tau, scaling=scaling, flags=fl, want_compact=True)
    out = S.sparse_attn(st, q, scaling, compact, n_splits=rng.choice([1, 2, 5, None]))
    torch.cuda.synchronize()
    o_dense, o_keep = O.search(ox, q, tau_np, scaling=scaling, flags=O.GATE_GE | O.LEAF_GE)
    want, _ = O.attention(ox, q, scaling, o_dense, o_keep)
    got = out.cpu().numpy()
    denom = np.abs(want).max(axis=-1, keepdims=True) + 1e-6
    assert np.max(np.abs(got - want) / denom) < (1e-5 if dtype == torch.float32 else 2e-3)
