"""The CPU oracle against outputs of the reference's own code (tests/golden/*.npz, made by
tests/golden/make_golden.py from the reference's Triton kernels run in the Triton
interpreter, its CUDAIndexer radius/update routines run on CPU tensors, and its C++
fused_tree_search_v3).  These pin the oracle; the GPU tests then pin the CUDA library to the
oracle bit for bit, and `test_cuda_matches_reference_fixtures` closes the loop directly.

Sets (which slots are emitted, where an appended key lands) must match exactly; scores and
radii within 1e-5 (the reference fixes no summation order, the oracle does).
"""
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return dict(np.load(GOLDEN / f"{name}.npz"))


def used_blocks(children, values, parents, radii, counts, bf):
    """Per head, the parent blocks that hold at least one key, in slot order.  With several
    heads the reference pads every head to the same number of parent blocks (an all-zero
    block where a head needed none, indexer/cuda.py:729-750), so the same blocks can sit at
    different slots; the blocks themselves and their order must agree."""
    out = []
    for h in range(children.shape[0]):
        keep = np.nonzero(counts[h] > 0)[0]
        c = children[h].reshape(-1, bf, children.shape[-1])[keep]
        v = values[h].reshape(-1, bf, values.shape[-1])[keep]
        out.append((c, v, parents[h][keep], radii[h][keep], counts[h][keep]))
    return out


def index_from(rec) -> O.OracleIndex:
    ox = O.OracleIndex(n_heads=int(rec["H"]), dim=int(rec["D"]), vdim=int(rec["D"]), bf=int(rec["bf"]),
                       depth=int(rec["depth"]), cap_parents=int(rec["cap_parents"]))
    for name in O.OracleIndex.ARRAYS:
        key = f"ix_{name}"
        if key in rec and getattr(ox, name) is not None:
            assert rec[key].shape == getattr(ox, name).shape, name
            setattr(ox, name, np.ascontiguousarray(rec[key]))
    return ox


@pytest.mark.parametrize("name", ["search_triton_l2", "search_triton_l3"])
def test_blocked_search_matches_reference_triton_kernels(name):
    rec = load(name)
    ox = index_from(rec)
    dense, keep = O.search(ox, rec["q"], rec["tau"], scaling=rec["scaling"], q2kv=rec["q2kv"],
                           flags=O.GATE_GT | O.LEAF_CANDIDATES)
    want = rec["expected_dense"]
    n = want.shape[1]
    # the reference marks "emitted" only by a non-zero score
    assert np.array_equal(dense[:, :n] != 0, want != 0)
    assert np.array_equal(keep[:, :n] != 0, want != 0)
    np.testing.assert_allclose(dense[:, :n], want, atol=1e-5, rtol=1e-5)
    assert 0 < (want != 0).sum() < want.size      # the thresholds prune some parents but not all


@pytest.mark.parametrize("name", ["append_l2", "append_l3", "append_l2_free"])
def test_radii_and_append_match_reference_indexer(name):
    rec = load(name)
    ox = index_from(rec)
    H, bf, depth = int(rec["H"]), int(rec["bf"]), int(rec["depth"])
    up, ug = int(ox.used[0, 0]), int(ox.used[0, 1])
    # radii recomputed from the layout (indexer/cuda.py:114-198)
    O.recompute_radii(ox)
    np.testing.assert_allclose(ox.parent_radii[:, :up], rec["radii_parent_from_layout"], atol=1e-5)
    if depth == 3:
        np.testing.assert_allclose(ox.gp_radii[:, :ug], rec["radii_gp_from_layout"], atol=1e-5)
    assert np.array_equal(ox.child_counts[:, :up], rec["init_child_counts"])
    # one key per call, as the decode loop does (indexer/cuda.py:544-701)
    m = rec["new_k"].shape[1]
    for i in range(m):
        O.append(ox, np.ascontiguousarray(rec["new_k"][:, i:i + 1]), np.ascontiguousarray(rec["new_v"][:, i:i + 1]))
    assert int(ox.status[0]) == 0
    P = rec["after_parents"].shape[1]
    mine = used_blocks(ox.children, ox.values, ox.parents, ox.parent_radii, ox.child_counts, bf)
    ref = used_blocks(rec["after_children"], rec["after_values"], rec["after_parents"], rec["after_parent_radii"],
                      rec["after_child_counts"], bf)
    for h in range(H):
        for a, b in zip(mine[h][:3] + mine[h][4:], ref[h][:3] + ref[h][4:]):
            assert np.array_equal(a, b)
        np.testing.assert_allclose(mine[h][3], ref[h][3], atol=1e-5)
    if depth == 3:
        assert np.array_equal(ox.children[:, :P * bf], rec["after_children"])
        assert np.array_equal(ox.child_counts[:, :P], rec["after_child_counts"])
        G = rec["after_gps"].shape[1]
        assert np.array_equal(ox.grand_parents[:, :G], rec["after_gps"])
        assert np.array_equal(ox.gp_counts[:, :G], rec["after_gp_counts"])
        np.testing.assert_allclose(ox.gp_radii[:, :G], rec["after_gp_radii"], atol=1e-5)


def csr_from_c2p(c2p, P):
    H, C = c2p.shape
    off = np.zeros((H, P + 1), np.int64)
    ch = np.zeros((H, C), np.int64)
    for h in range(H):
        ch[h] = np.argsort(c2p[h], kind="stable")
        off[h, 1:] = np.cumsum(np.bincount(c2p[h], minlength=P))
    return off, ch


def levels_of(rec):
    L = int(rec["n_levels"])
    centers = [rec[f"centers_{l}"] for l in range(L)]
    radii = [rec[f"radii_{l}"] for l in range(L)]
    c2p = [rec[f"c2p_{l}"] for l in range(L - 1)]
    return centers, radii, c2p


@pytest.mark.parametrize("name", ["search_cpu_v3_l2", "search_cpu_v3_l3"])
def test_csr_search_matches_reference_cpp_kernel(name):
    rec = load(name)
    centers, radii, c2p = levels_of(rec)
    sizes = [c.shape[1] for c in centers]
    offs, chs = [], []
    for l in range(len(centers) - 1):
        o, c = csr_from_c2p(c2p[l], sizes[l + 1])
        offs.append(o)
        chs.append(c)
    offs.append(None)
    chs.append(None)
    G = int(rec["G"])
    hq = rec["q"].shape[0]
    q2kv = (np.arange(hq) // G).astype(np.int32)
    out, keep = O.search_csr(centers, radii, offs, chs, sizes, rec["q"], rec["tau"], scaling=rec["scaling"], q2kv=q2kv)
    want = rec["expected_dense"]
    assert np.array_equal(out != 0, want != 0)
    np.testing.assert_allclose(out, want, atol=1e-5, rtol=1e-5)
    assert (want != 0).sum() > 0


@pytest.mark.parametrize("name", ["search_cpu_v3_l2", "search_cpu_v3_l3"])
def test_blocked_conversion_of_cpu_index_selects_the_same_tokens(name):
    """A CPU-format index converted to the blocked layout and searched with the CPU rule
    (gate >=, leaf >=) selects exactly the tokens the reference CPU kernel selects."""
    from hira_b200.indexer.convert import blocked_from_levels
    rec = load(name)
    centers, radii, c2p = levels_of(rec)
    arrays = blocked_from_levels(centers, radii, c2p)
    ox = O.OracleIndex.from_arrays(arrays)
    G = int(rec["G"])
    hq = rec["q"].shape[0]
    dense, keep = O.search(ox, rec["q"], rec["tau"], scaling=rec["scaling"], flags=O.GATE_GE | O.LEAF_GE)
    want = rec["expected_dense"]
    for qh in range(hq):
        h = qh // G
        slots = np.nonzero(keep[qh])[0]
        toks = ox.slot2token[h, slots]
        assert sorted(toks.tolist()) == np.nonzero(want[qh])[0].tolist()
        np.testing.assert_allclose(dense[qh, slots], want[qh, toks], atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["search_triton_l2", "search_triton_l3", "search_cpu_v3_l2", "search_cpu_v3_l3",
                                  "append_l2", "append_l3", "append_l2_free"])
def test_cuda_matches_reference_fixtures(name):
    """The CUDA library, through the C ABI, directly against the reference's outputs."""
    import torch
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200.indexer.convert import blocked_from_levels
    rec = load(name)
    if name.startswith("search_cpu"):
        centers, radii, c2p = levels_of(rec)
        arrays = blocked_from_levels(centers, radii, c2p)
        flags, q2kv = L.HIRA_GATE_GE | L.HIRA_LEAF_GE, None
    else:
        arrays = index_from(rec).arrays()
        flags = L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES
        q2kv = torch.from_numpy(rec["q2kv"]).cuda() if "q2kv" in rec else None
    m = arrays["meta"]
    st = S.IndexState(n_heads=m["n_heads"], dim=m["dim"], vdim=m["vdim"] or m["dim"], bf=m["bf"], depth=m["depth"],
                      cap_parents=m["cap_parents"], dtype=torch.float32, vdtype=torch.float32, device="cuda",
                      with_values=arrays.get("values") is not None)
    st.load_arrays(arrays)
    if name.startswith("append"):
        k, v = torch.from_numpy(rec["new_k"]).cuda(), torch.from_numpy(rec["new_v"]).cuda()
        for i in range(k.shape[1]):
            S.append(st, k[:, i:i + 1].contiguous(), v[:, i:i + 1].contiguous())
        torch.cuda.synchronize()
        bf, P = m["bf"], rec["after_parents"].shape[1]
        mine = used_blocks(st.children.cpu().numpy(), st.values.cpu().numpy(), st.parents.cpu().numpy(),
                           st.parent_radii.cpu().numpy(), st.child_counts.cpu().numpy(), bf)
        ref = used_blocks(rec["after_children"], rec["after_values"], rec["after_parents"],
                          rec["after_parent_radii"], rec["after_child_counts"], bf)
        for h in range(m["n_heads"]):
            for a, b in zip(mine[h][:3] + mine[h][4:], ref[h][:3] + ref[h][4:]):
                assert np.array_equal(a, b)
            np.testing.assert_allclose(mine[h][3], ref[h][3], atol=1e-5)
        if m["depth"] == 3:
            G = rec["after_gps"].shape[1]
            np.testing.assert_allclose(st.gp_radii[:, :G].cpu().numpy(), rec["after_gp_radii"], atol=1e-5)
        return
    q = torch.from_numpy(rec["q"]).cuda()
    tau = torch.from_numpy(rec["tau"]).cuda()
    scaling = torch.from_numpy(rec["scaling"]).cuda()
    hq = q.shape[0]
    dense = torch.empty((hq, st.cap_children), device="cuda")
    S.search(st, q, tau, scaling=scaling, q2kv=q2kv, max_group=0, flags=flags, out_dense=dense)
    torch.cuda.synchronize()
    d = dense.cpu().numpy()
    want = rec["expected_dense"]
    if name.startswith("search_cpu"):
        s2t = st.slot2token.cpu().numpy()
        G = int(rec["G"])
        for qh in range(hq):
            slots = np.nonzero(d[qh])[0]
            toks = s2t[qh // G, slots]
            assert sorted(toks.tolist()) == np.nonzero(want[qh])[0].tolist()
            np.testing.assert_allclose(d[qh, slots], want[qh, toks], atol=1e-5, rtol=1e-5)
    else:
        n = want.shape[1]
        assert np.array_equal(d[:, :n] != 0, want != 0)
        np.testing.assert_allclose(d[:, :n], want, atol=1e-5, rtol=1e-5)
