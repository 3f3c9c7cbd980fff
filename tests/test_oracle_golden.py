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


# ---------------------------------------------------------------------------------------
# bf16 keys of the decode workload's distribution, D = 128, branching 32
# ---------------------------------------------------------------------------------------
BF16_FIXTURES = ["search_triton_l2_bf16_d128_bf32", "search_triton_l3_bf16_d128_bf32"]


def bf16_fixture_index(rec):
    """The fixture stores the bf16 keys and the initial centres; the oracle's (deterministic)
    build lays the index out exactly as it did when the fixture was made."""
    import torch
    H, n, D, bf, depth = (int(rec[k]) for k in ("H", "n", "D", "bf", "depth"))
    keys = torch.from_numpy(rec["keys_bf16"]).view(torch.bfloat16)
    vals = torch.zeros_like(keys)
    ox = O.OracleIndex(n_heads=H, dim=D, vdim=D, bf=bf, depth=depth, cap_parents=int(rec["cap_parents"]),
                       dtype=O.HIRA_BF16, vdtype=O.HIRA_BF16)
    O.build(ox, keys, vals, cent_idx1=rec["cent_idx1"], cent_idx2=rec["cent_idx2"] if depth == 3 else None)
    return ox, keys, vals


@pytest.mark.parametrize("name", BF16_FIXTURES)
def test_blocked_search_matches_reference_triton_kernels_on_bf16_keys(name):
    rec = load(name)
    ox, _, _ = bf16_fixture_index(rec)
    dense, keep = O.search(ox, rec["q"], rec["tau"], scaling=rec["scaling"], q2kv=rec["q2kv"],
                           flags=O.GATE_GT | O.LEAF_CANDIDATES)
    n = int(rec["n"])
    want = np.unpackbits(rec["expected_mask"], axis=-1)[:, :n].astype(bool)
    assert np.array_equal(keep[:, :n] != 0, want)
    np.testing.assert_allclose(dense[:, :n].sum(axis=-1), rec["expected_sum"], rtol=1e-4)
    per_head = want.sum(axis=-1)
    assert per_head[0] == n and 0 < per_head[1] < n     # workload threshold: no pruning; median gate: some


@pytest.mark.gpu
@pytest.mark.parametrize("name", BF16_FIXTURES)
def test_cuda_matches_reference_triton_kernels_on_bf16_keys(name):
    import torch
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    rec = load(name)
    H, n, D, bf, depth = (int(rec[k]) for k in ("H", "n", "D", "bf", "depth"))
    keys = torch.from_numpy(rec["keys_bf16"]).view(torch.bfloat16).cuda()
    st = S.IndexState(n_heads=H, dim=D, vdim=D, bf=bf, depth=depth, cap_parents=int(rec["cap_parents"]),
                      dtype=torch.bfloat16, vdtype=torch.bfloat16, device="cuda")
    S.build(st, keys, torch.zeros_like(keys), cent_idx1=torch.from_numpy(rec["cent_idx1"]).cuda(),
            cent_idx2=torch.from_numpy(rec["cent_idx2"]).cuda() if depth == 3 else None, use_tensor_cores=False)
    q, tau = torch.from_numpy(rec["q"]).cuda(), torch.from_numpy(rec["tau"]).cuda()
    _, compact = S.search(st, q, tau, scaling=torch.from_numpy(rec["scaling"]).cuda(),
                          q2kv=torch.from_numpy(rec["q2kv"]).cuda(), flags=L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES,
                          want_compact=True)
    torch.cuda.synchronize()
    want = np.unpackbits(rec["expected_mask"], axis=-1)[:, :n].astype(bool)
    for qh, (slots, scores) in enumerate(compact.to_lists()):
        assert np.array_equal(slots.numpy(), np.nonzero(want[qh])[0])
        np.testing.assert_allclose(float(scores.sum()), rec["expected_sum"][qh], rtol=1e-4)


# ---------------------------------------------------------------------------------------
# the CPU index restatement (oracle/cpu_index.py) against the reference's CPUIndexer
# ---------------------------------------------------------------------------------------
def test_cpu_index_restatement_matches_reference_cpu_indexer():
    from oracle import cpu_index as CI
    rec = load("cpu_indexer_levels")
    bf, nl, it = int(rec["bf"]), int(rec["num_levels"]), int(rec["max_iterations"])
    levels = CI.build_levels(rec["keys"], nl, bf, it)

    def check(tag):
        assert len(levels) == int(rec[f"{tag}_n_levels"])
        for l, lv in enumerate(levels):
            assert np.array_equal(lv["centers"], rec[f"{tag}_centers_{l}"]), (tag, l)
            np.testing.assert_allclose(lv["radii"], rec[f"{tag}_radii_{l}"], rtol=1e-6, atol=1e-6)
            if lv["c2p"] is not None:
                assert np.array_equal(lv["c2p"], rec[f"{tag}_c2p_{l}"]), (tag, l)
            else:
                assert f"{tag}_c2p_{l}" not in rec
    check("built")
    CI.update_levels(levels, rec["new_keys"], bf, it)
    check("updated")
    assert [lv["size"] for lv in levels] == [620, 77, 10]


# ---------------------------------------------------------------------------------------
# the reference's own compiled kernels, run live (oracle/_ref, built from its sources)
# ---------------------------------------------------------------------------------------
ROOT = Path(__file__).resolve().parents[1]


def _two_level_omp():
    import ctypes as C
    so = ROOT / "oracle" / "_ref" / "libtwo_level_filter_omp.so"
    if not so.exists():
        pytest.skip("oracle/_ref/libtwo_level_filter_omp.so is not built (make -C oracle ref REF=...)")
    lib = C.CDLL(str(so))
    lib.two_level_filter_omp.restype = None
    lib.two_level_filter_omp.argtypes = [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_float, C.c_int32]
    return lib


def test_two_level_search_matches_reference_omp_kernel_at_cfg1_width():
    """benchmark_area/cpu_bench/archive/two_level_filter_omp.cpp is the reference's CPU statement
    of the Triton two-level rule (skip a parent when dot + r <= t, else write every child's
    score).  Decode-workload keys, D = 128, branching 32, 32,768 keys of one head."""
    import torch
    from hira_b200 import workloads as W
    lib = _two_level_omp()
    n, D, bf = 32768, 128, 32
    keys, vals = W.make_kv(1, n, 41, "cpu", dist="rope_outlier", dtype=torch.float32)
    ox = O.OracleIndex(n_heads=1, dim=D, vdim=D, bf=bf, depth=2, cap_parents=n // bf)
    O.build(ox, keys, vals, cent_idx1=W.random_centres(1, n, n // bf, 3, "cpu"))
    q = W.make_queries(2, 8, "cpu", pos=n)
    q = (q / q.norm(dim=-1, keepdim=True)).numpy()
    gates = ox.parents[0] @ q.T + ox.parent_radii[0][:, None]            # (parents, 2)
    for j, frac in enumerate((0.5, 0.9)):                               # thresholds inside the gate range
        gv = np.sort(gates[:, j].astype(np.float64))
        i = int(frac * len(gv))
        while gv[i + 1] - gv[i] < 1e-3:
            i += 1
        t = np.float32(0.5 * (gv[i] + gv[i + 1]))
        out = np.zeros(n, np.float32)
        qj = np.ascontiguousarray(q[j])
        lib.two_level_filter_omp(ox.children.ctypes.data, ox.parents.ctypes.data, ox.parent_radii.ctypes.data,
                                 qj.ctypes.data, out.ctypes.data, n, n // bf, D, t, bf)
        dense, keep = O.search(ox, qj[None], np.array([t], np.float32), q2kv=np.zeros(1, np.int32),
                               flags=O.GATE_GT | O.LEAF_CANDIDATES)
        assert np.array_equal(keep[0] != 0, out != 0)
        assert 0 < (out != 0).sum() < n
        np.testing.assert_allclose(dense[0], out, atol=2e-5, rtol=1e-5)


def cfg0_case():
    """BASELINE configuration 0 whole: fp32, 8 heads x 4,096 keys (per-channel scaled Gaussian),
    one query per head, 2 levels of branching 64 with 10 k-means iterations; thresholds: the
    exact 128th largest score per head (a key sits on it) and the midpoint below it."""
    import torch
    from hira_b200 import workloads as W
    from oracle import cpu_index as CI
    ext = CI.load_reference_kernel(ROOT)
    if ext is None:
        pytest.skip("oracle/_ref/hira_torch_ext_v3.so is not built (make -C oracle ref REF=...)")
    w = W.CFG0
    keys, vals, q = W.make_inputs(w, "cpu")
    levels = CI.build_levels(keys.numpy(), w.levels, w.branching, 10)
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    sc = torch.einsum("hd,hnd->hn", q_hat, keys)
    srt = torch.sort(sc, dim=-1, descending=True).values
    tau_exact = srt[:, w.kth - 1].contiguous()
    tau_mid = W.guard_banded_tau(sc, w.kth)
    return ext, levels, keys, vals, q_hat, sc, tau_exact, tau_mid


def check_against_reference_cpu_kernel(search_blocked, slot2token, ext, levels, keys, q_hat, sc, tau_exact, tau_mid):
    """search_blocked(tau) -> per query head (slots, scores) of the blocked index searched with
    gate >=, leaf >=; compared with the reference kernel's dense token-order output."""
    from oracle import cpu_index as CI
    prepared = CI.searcher_inputs(levels)
    hq = q_hat.shape[0]
    # (1) midpoint threshold: the sets must be equal
    want = CI.reference_search(ext, levels, q_hat, tau_mid, prepared=prepared).numpy()
    got = search_blocked(tau_mid)
    for qh in range(hq):
        slots, scores = got[qh]
        toks = slot2token[qh][slots]
        assert sorted(toks.tolist()) == np.nonzero(want[qh])[0].tolist()
        np.testing.assert_allclose(scores, want[qh][toks], atol=1e-4, rtol=1e-5)
        assert len(toks) == 128
    # (2) the exact 128th largest score: only keys whose score is within rounding of the
    # threshold may differ (the reference kernel sums in compiler-chosen SIMD order)
    want = CI.reference_search(ext, levels, q_hat, tau_exact, prepared=prepared).numpy()
    got = search_blocked(tau_exact)
    n_boundary = 0
    for qh in range(hq):
        toks = set(slot2token[qh][got[qh][0]].tolist())
        ref = set(np.nonzero(want[qh])[0].tolist())
        for t in toks ^ ref:
            bound = 2.0 ** -20 * float(np.linalg.norm(keys[qh, t]))
            assert abs(float(sc[qh, t]) - float(tau_exact[qh])) <= bound, (qh, t)
            n_boundary += 1
        assert 126 <= len(toks) <= 129
    return n_boundary


def test_cfg0_blocked_search_matches_reference_cpu_kernel():
    from hira_b200.indexer.convert import blocked_from_levels
    ext, levels, keys, vals, q_hat, sc, tau_exact, tau_mid = cfg0_case()
    arrays = blocked_from_levels([lv["centers"] for lv in levels], [lv["radii"] for lv in levels],
                                 [lv["c2p"] for lv in levels[:-1]], values=vals.numpy())
    ox = O.OracleIndex.from_arrays(arrays)
    assert [lv["size"] for lv in levels] == [4096, 64]

    def search_blocked(tau):
        dense, keep = O.search(ox, q_hat.numpy(), tau.numpy(), flags=O.GATE_GE | O.LEAF_GE)
        return [(np.nonzero(keep[qh])[0], dense[qh][np.nonzero(keep[qh])[0]]) for qh in range(q_hat.shape[0])]
    check_against_reference_cpu_kernel(search_blocked, ox.slot2token, ext, levels, keys.numpy(), q_hat, sc.numpy(),
                                       tau_exact, tau_mid)


@pytest.mark.gpu
def test_cfg0_cuda_search_matches_reference_cpu_kernel():
    import torch
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200.indexer.convert import blocked_from_levels
    ext, levels, keys, vals, q_hat, sc, tau_exact, tau_mid = cfg0_case()
    arrays = blocked_from_levels([lv["centers"] for lv in levels], [lv["radii"] for lv in levels],
                                 [lv["c2p"] for lv in levels[:-1]], values=vals.numpy())
    m = arrays["meta"]
    st = S.IndexState(n_heads=m["n_heads"], dim=m["dim"], vdim=m["vdim"], bf=m["bf"], depth=m["depth"],
                      cap_parents=m["cap_parents"], dtype=torch.float32, vdtype=torch.float32, device="cuda")
    st.load_arrays(arrays)
    qd = q_hat.cuda()

    def search_blocked(tau):
        _, compact = S.search(st, qd, tau.cuda(), flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
        torch.cuda.synchronize()
        return [(a.numpy(), b.numpy()) for a, b in compact.to_lists()]
    check_against_reference_cpu_kernel(search_blocked, arrays["slot2token"], ext, levels, keys.numpy(), q_hat,
                                       sc.numpy(), tau_exact, tau_mid)
    # attention over V of the selected keys (fp32): against softmax over exactly those tokens
    scaling = torch.full((q_hat.shape[0],), 1.0, device="cuda")
    _, compact = S.search(st, qd, tau_mid.cuda(), scaling=scaling, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE,
                          want_compact=True)
    out = S.sparse_attn(st, qd, scaling, compact).cpu()
    mask = sc >= tau_mid[:, None]
    w = torch.softmax(torch.where(mask, sc, torch.full_like(sc, float("-inf"))).double(), dim=-1)
    want = torch.einsum("hn,hnd->hd", w, vals.double()).float()
    assert float((out - want).abs().max() / want.abs().max()) < 1e-5


def test_five_level_cpu_index_converts_to_three_levels_with_the_same_selection():
    """A CPU-format index of 5 levels (HiraConfig's default depth) searched by the reference C++ kernel
    selects exactly the tokens that the blocked conversion of its lowest three levels selects."""
    import torch
    from hira_b200 import workloads as W
    from hira_b200.indexer.convert import blocked_from_levels
    from oracle import cpu_index as CI
    ext = CI.load_reference_kernel(ROOT)
    if ext is None:
        pytest.skip("oracle/_ref/hira_torch_ext_v3.so is not built (make -C oracle ref REF=...)")
    keys, vals = W.make_kv(2, 4096, 17, "cpu", dist="clustered", dtype=torch.float32)
    levels = CI.build_levels(keys.numpy(), 5, 4, 2)
    assert [lv["size"] for lv in levels] == [4096, 1024, 256, 64, 16]
    q = W.make_queries(4, 3, "cpu")
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    sc = torch.einsum("hgd,hnd->hgn", q_hat.view(2, 2, 128), keys).reshape(4, 4096)
    tau = W.guard_banded_tau(sc, 40)
    want = CI.reference_search(ext, levels, q_hat, tau).numpy()
    arrays = blocked_from_levels([lv["centers"] for lv in levels], [lv["radii"] for lv in levels],
                                 [lv["c2p"] for lv in levels[:-1]])
    assert arrays["meta"]["depth"] == 3
    ox = O.OracleIndex.from_arrays(arrays)
    dense, keep = O.search(ox, q_hat.numpy(), tau.numpy(), flags=O.GATE_GE | O.LEAF_GE)
    for qh in range(4):
        toks = ox.slot2token[qh // 2][np.nonzero(keep[qh])[0]]
        assert sorted(toks.tolist()) == np.nonzero(want[qh])[0].tolist()
        assert len(toks) == 40
    # the five-level search pruned at its upper levels, the conversion did not need them
    assert (want != 0).sum() == 160
