"""CUDA library vs CPU oracle on the same seeded inputs, through the C ABI.  Integer and
index results (selected slots, layouts, counts) and fp32 scores must be bit-exact;
attention outputs within the stated tolerances (1e-5 fp32, 2e-3 relative bf16)."""
import numpy as np
import pytest
import torch

from hira_b200 import _lib as L
from hira_b200 import index_state as S
from oracle import oracle as O

from util import (assert_index_equal, build_both, compact_sets, exact_tau, make_keys, make_queries, new_state,
                  random_centres)

pytestmark = pytest.mark.gpu

BUILD_CASES = [
    # h, n, d, bf, depth, dtype, n_iters
    (2, 256, 32, 8, 2, torch.float32, 1),
    (3, 1000, 64, 8, 3, torch.float32, 1),
    (2, 777, 128, 16, 3, torch.bfloat16, 1),
    (2, 1024, 128, 32, 3, torch.bfloat16, 2),
    (1, 130, 16, 10, 2, torch.float32, 3),
    (2, 4096, 128, 64, 2, torch.float32, 1),
    (1, 300, 256, 4, 3, torch.bfloat16, 1),
]


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,n_iters", BUILD_CASES)
def test_build_matches_oracle(h, n, d, bf, depth, dtype, n_iters):
    st, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=7, n_iters=n_iters, spare=2 * bf)
    assert_index_equal(st, ox, "build")
    # structural invariants the reference's tests pin (tests/test_cuda_indexer_searcher.py:134-195)
    assert int((st.slot2token >= 0).sum()) == h * n
    assert int(st.child_counts.sum()) == h * n
    assert int(st.child_counts.max()) <= bf


SEARCH_CASES = [
    # h, n, d, bf, depth, dtype, group
    (2, 512, 32, 8, 2, torch.float32, 1),
    (2, 1000, 64, 8, 3, torch.float32, 2),
    (2, 2048, 128, 32, 3, torch.bfloat16, 4),
    (1, 4096, 128, 64, 3, torch.bfloat16, 8),
    (2, 900, 128, 16, 2, torch.bfloat16, 3),
    (1, 640, 128, 4, 3, torch.float32, 12),
    (2, 700, 256, 10, 3, torch.float32, 4),
    (1, 300, 64, 1, 2, torch.float32, 2),
    (1, 6000, 64, 48, 3, torch.bfloat16, 2),      # three 16-parent tiles per grandparent (not a power of two)
]
FLAG_CASES = [
    L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES,
    L.HIRA_GATE_GE | L.HIRA_LEAF_GE,
    L.HIRA_GATE_GT | L.HIRA_LEAF_GT,
]


def _run_search_case(st, ox, q, tau, flags, scaling=None, qnorm=None, q2kv=None, max_group=0):
    hq = q.shape[0]
    dense = torch.full((hq, st.cap_children), float("nan"), device="cuda")
    stats = S.new_stats(hq, "cuda")
    _, compact = S.search(st, q, tau, scaling=scaling, qnorm=qnorm, q2kv=q2kv, max_group=max_group, flags=flags,
                          out_dense=dense, want_compact=True, stats=stats)
    torch.cuda.synchronize()
    o_dense, o_keep, o_stats = O.search(ox, q, tau, scaling=scaling, qnorm=qnorm, q2kv=q2kv, flags=flags,
                                        want_stats=True)
    d = dense.cpu().numpy()
    assert np.array_equal(d.view(np.uint32), o_dense.view(np.uint32)), "dense output differs from the oracle"
    sets = compact_sets(compact)
    for qh in range(hq):
        slots, scores = sets[qh]
        want = np.nonzero(o_keep[qh])[0]
        assert np.array_equal(slots, want), f"head {qh}: selected slots differ ({len(slots)} vs {len(want)})"
        assert np.array_equal(scores.view(np.uint32), o_dense[qh, want].view(np.uint32))
    s = stats.cpu().numpy().astype(np.uint32)
    assert np.array_equal(s[:, :6], o_stats[:, :6]), "visit counters differ"
    return o_keep


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,group", SEARCH_CASES)
@pytest.mark.parametrize("flags", FLAG_CASES)
def test_search_matches_oracle(h, n, d, bf, depth, dtype, group, flags):
    st, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=11, spare=bf)
    hq = h * group
    q = make_queries(hq, d, seed=5)
    sc = torch.einsum("hnd,hgd->hgn", keys.float(), q.view(h, group, d)).reshape(hq, n).cpu().numpy()
    # threshold = one of the canonical scores themselves (the 10% boundary), so that the
    # >= / > edge is exercised with a key sitting exactly on it
    all_d, all_k = O.search(ox, q, np.full((hq,), -np.inf, np.float32), flags=O.GATE_GT)
    tau_np = np.stack([exact_tau(all_d[i][all_k[i] > 0][None, :], 0.10)[0] for i in range(hq)])
    tau = torch.from_numpy(tau_np).cuda()
    scaling = torch.linspace(0.5, 2.0, hq, device="cuda")
    keep = _run_search_case(st, ox, q, tau, flags, scaling=scaling)
    if flags & L.HIRA_LEAF_GE:
        # against brute force in token space, away from the boundary: every key with
        # score > tau + eps is selected, none with score < tau - eps
        s2t = ox.slot2token
        for qh in range(hq):
            toks = set(s2t[qh // group, np.nonzero(keep[qh])[0]].tolist())
            must = set(np.nonzero(sc[qh] > tau[qh].item() + 1e-5)[0].tolist())
            never = set(np.nonzero(sc[qh] < tau[qh].item() - 1e-5)[0].tolist())
            assert must <= toks and not (toks & never)


def test_search_explicit_map_qnorm_and_empty():
    h, n, d, bf = 2, 1536, 128, 16
    st, ox, keys, _ = build_both(h, n, d, bf, 3, torch.bfloat16, seed=21, spare=bf)
    hq = 6
    q = make_queries(hq, d, seed=9, normalize=False)
    q2kv = torch.tensor([1, 0, 1, 1, 0, 1], dtype=torch.int32, device="cuda")  # non-monotone, uneven groups
    qn = q.norm(dim=-1).contiguous()
    tau = torch.tensor([0.5, 1.0, -1e30, 1e30, 0.0, 2.0], device="cuda")  # includes keep-all and keep-none
    for flags in FLAG_CASES:
        _run_search_case(st, ox, q, tau, flags, qnorm=qn, q2kv=q2kv, max_group=4)
        _run_search_case(st, ox, q, tau, flags, qnorm=None, q2kv=q2kv, max_group=0)


def test_search_is_deterministic():
    st, ox, keys, _ = build_both(2, 2048, 128, 32, 3, torch.bfloat16, seed=3)
    q = make_queries(8, 128, seed=1)
    tau = torch.full((8,), 0.05, device="cuda")
    outs = []
    for _ in range(2):
        _, c = S.search(st, q, tau, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
        torch.cuda.synchronize()
        outs.append((c.idx.clone(), c.score.clone(), c.count.clone()))
    assert torch.equal(outs[0][2], outs[1][2])
    for (a, b) in zip(compact_sets(S.CompactResult(*outs[0], c.tile_parents, c.tile_rows)),
                      compact_sets(S.CompactResult(*outs[1], c.tile_parents, c.tile_rows))):
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


APPEND_CASES = [
    (2, 256, 32, 8, 2, torch.float32, 40),
    (2, 500, 64, 8, 3, torch.float32, 70),
    (3, 1024, 128, 32, 3, torch.bfloat16, 100),
    (1, 100, 128, 4, 3, torch.bfloat16, 60),
]


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,m", APPEND_CASES)
def test_append_matches_oracle(h, n, d, bf, depth, dtype, m):
    st, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=31, spare=(m + 1) * bf)
    new_k = make_keys(h, m, d, 77, dtype)
    new_v = make_keys(h, m, d, 78, dtype, normalize=False)
    # one key per call (the decode pattern), then a batch
    half = m // 2
    for i in range(half):
        S.append(st, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())
        O.append(ox, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())
    S.append(st, new_k[:, half:].contiguous(), new_v[:, half:].contiguous())
    O.append(ox, new_k[:, half:].contiguous(), new_v[:, half:].contiguous())
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0 and int(ox.status[0]) == 0
    assert_index_equal(st, ox, "append")
    assert int((st.slot2token >= 0).sum()) == h * (n + m)
    # incrementally widened radii bound the radii recomputed from the layout
    r_inc = st.parent_radii.clone()
    S.recompute_radii(st)
    O.recompute_radii(ox)
    torch.cuda.synchronize()
    assert_index_equal(st, ox, "radii")
    assert bool((r_inc >= st.parent_radii - 1e-6).all())
    # search after append still equals the oracle
    q = make_queries(h * 2, d, seed=4)
    tau = torch.full((h * 2,), 0.1, device="cuda")
    _run_search_case(st, ox, q, tau, L.HIRA_GATE_GE | L.HIRA_LEAF_GE)


def test_append_with_and_without_workspace_agree():
    # the scan spread over the GPU (two kernels, scratch) and the one-CTA-per-head path give the same index
    h, n, d, bf = 2, 8192, 128, 32
    a, ox, keys, vals = build_both(h, n, d, bf, 3, torch.bfloat16, seed=61, spare=40 * bf)
    b, _, _, _ = build_both(h, n, d, bf, 3, torch.bfloat16, seed=61, spare=40 * bf)
    new_k = make_keys(h, 24, d, 62, torch.bfloat16)
    new_v = make_keys(h, 24, d, 63, torch.bfloat16, normalize=False)
    for lo, hi in ((0, 1), (1, 2), (2, 10), (10, 24)):
        S.append(a, new_k[:, lo:hi].contiguous(), new_v[:, lo:hi].contiguous(), use_workspace=True)
        S.append(b, new_k[:, lo:hi].contiguous(), new_v[:, lo:hi].contiguous(), use_workspace=False)
        O.append(ox, new_k[:, lo:hi].contiguous(), new_v[:, lo:hi].contiguous())
    torch.cuda.synchronize()
    assert int(L.load().hira_append_workspace_bytes(a.struct, 1)) > 0
    assert_index_equal(a, ox, "append with workspace")
    assert_index_equal(b, ox, "append without workspace")


SCAN_CASES = [
    # h, n, d, bf, depth, dtype, group, steps
    (2, 256, 32, 8, 2, torch.float32, 1, 30),
    (2, 500, 64, 8, 3, torch.float32, 2, 40),
    (3, 4096, 128, 32, 3, torch.bfloat16, 4, 40),
    (2, 2048, 128, 32, 3, torch.bfloat16, 8, 20),     # two 4-head chunks per kv head: only the first scans
    (1, 100, 128, 4, 3, torch.bfloat16, 1, 50),       # many parents per tile (the gate loop beyond the staged rows)
    (2, 700, 256, 16, 3, torch.float32, 2, 20),
]


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,group,steps", SCAN_CASES)
def test_search_with_fused_parent_scan_equals_search_then_append(h, n, d, bf, depth, dtype, group, steps):
    """search + append against search-with-scan + append-from-scan on twin indexes, key after key:
    the same keys are selected and the indexes stay bit-identical to the oracle's."""
    a, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=71, spare=(steps + 1) * bf)
    b, _, _, _ = build_both(h, n, d, bf, depth, dtype, seed=71, spare=(steps + 1) * bf)
    new_k = make_keys(h, steps, d, 72, dtype)
    new_v = make_keys(h, steps, d, 73, dtype, normalize=False)
    hq = h * group
    q = make_queries(hq, d, seed=74)
    tau = torch.full((hq,), 0.15, device="cuda")
    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
    ca, cb = S.alloc_compact(a, hq), S.alloc_compact(b, hq)
    scan = S.new_scan_slots(b)
    for i in range(steps):
        k1, v1 = new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous()
        S.search(a, q, tau, flags=flags, compact=ca)
        S.append(a, k1, v1)
        S.search(b, q, tau, flags=flags, compact=cb, scan_key=new_k[:, i], scan_out=scan)
        S.append_scanned(b, new_k[:, i:i + 1], new_v[:, i:i + 1], scan)       # strided views are fine
        O.append(ox, k1, v1)
        if i % 7 == 0 or i == steps - 1:
            torch.cuda.synchronize()
            la, lb = ca.to_lists(), cb.to_lists()
            for x, y in zip(la, lb):
                assert torch.equal(x[0], y[0]) and torch.equal(x[1], y[1])
    torch.cuda.synchronize()
    assert bool((scan == -1).all())                    # every slot was consumed and reset
    assert int(a.status.item()) == 0 and int(b.status.item()) == 0
    assert_index_equal(a, ox, "search then append")
    assert_index_equal(b, ox, "search with scan, append from scan")


def test_fused_scan_rejects_explicit_head_map():
    st, _, _, _ = build_both(2, 256, 32, 8, 2, torch.float32, seed=75, spare=16)
    q = make_queries(2, 32, seed=76)
    with pytest.raises(ValueError):
        S.search(st, q, torch.zeros(2, device="cuda"), q2kv=torch.tensor([1, 0], dtype=torch.int32, device="cuda"),
                 want_compact=True, scan_key=make_keys(2, 1, 32, 77)[:, 0], scan_out=S.new_scan_slots(st))


def test_append_capacity_status():
    h, n, d, bf = 1, 64, 32, 8
    st, ox, keys, vals = build_both(h, n, d, bf, 2, torch.float32, seed=5, spare=2)
    new_k = make_keys(h, 8, d, 91) * 50.0  # far from everything: each becomes its own parent
    new_v = make_keys(h, 8, d, 92)
    S.append(st, new_k, new_v)
    O.append(ox, new_k, new_v)
    torch.cuda.synchronize()
    assert int(st.status.item()) == int(ox.status[0]) != 0
    assert_index_equal(st, ox, "append at capacity")


ATTN_CASES = [
    (2, 2048, 128, 32, 3, torch.float32, 4, 0, 1e-5),
    (2, 2048, 128, 32, 3, torch.bfloat16, 4, 5, 2e-3),
    (1, 4096, 64, 8, 2, torch.bfloat16, 2, 0, 2e-3),
    (2, 600, 128, 16, 3, torch.float32, 1, 33, 1e-5),
]


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,group,n_queued,tol", ATTN_CASES)
@pytest.mark.parametrize("n_splits", [1, 3, None])
def test_sparse_attention_matches_oracle(h, n, d, bf, depth, dtype, group, n_queued, tol, n_splits):
    st, ox, keys, vals = build_both(h, n, d, bf, depth, dtype, seed=41)
    hq = h * group
    q = make_queries(hq, d, seed=6)
    sc = torch.einsum("hnd,hgd->hgn", keys.float(), q.view(h, group, d)).reshape(hq, n).cpu().numpy()
    tau = torch.from_numpy(exact_tau(sc, 0.05)).cuda()
    scaling = torch.full((hq,), 8.0, device="cuda")
    _, compact = S.search(st, q, tau, scaling=scaling, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
    qk = make_keys(h, n_queued, d, 55, dtype) if n_queued else None
    qv = make_keys(h, n_queued, d, 56, dtype, normalize=False) if n_queued else None
    ml = torch.zeros((hq, 2), device="cuda")
    out = S.sparse_attn(st, q, scaling, compact, queued_k=qk, queued_v=qv, n_splits=n_splits, out_ml=ml)
    torch.cuda.synchronize()
    o_dense, o_keep = O.search(ox, q, tau, scaling=scaling, flags=O.GATE_GE | O.LEAF_GE)
    want, want_ml = O.attention(ox, q, scaling, o_dense, o_keep, queued_k=qk, queued_v=qv)
    got = out.cpu().numpy()
    denom = np.abs(want).max(axis=-1, keepdims=True) + 1e-6
    assert np.max(np.abs(got - want) / denom) < tol
    got_ml = ml.cpu().numpy()
    np.testing.assert_allclose(got_ml[:, 0], want_ml[:, 0], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(got_ml[:, 1], want_ml[:, 1], rtol=1e-4)


@pytest.mark.parametrize("n_splits", [1, 2])
def test_attention_over_every_key_equals_dense_softmax(n_splits):
    """Keep-all threshold: every tile emits all its rows, so a block of tiles overflows the staging
    list many times over (the chunked path), and the result must be plain softmax attention."""
    h, n, d, bf, group = 2, 8192, 128, 32, 2
    st, ox, keys, vals = build_both(h, n, d, bf, 3, torch.bfloat16, seed=43)
    hq = h * group
    q = make_queries(hq, d, seed=7)
    tau = torch.full((hq,), float("-inf"), device="cuda")
    scaling = torch.full((hq,), 6.0, device="cuda")
    _, compact = S.search(st, q, tau, scaling=scaling, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
    out = S.sparse_attn(st, q, scaling, compact, n_splits=n_splits)
    torch.cuda.synchronize()
    assert int(compact.count.sum()) == hq * n
    logits = torch.einsum("hnd,hgd->hgn", keys.double(), q.view(h, group, d).double()) * 6.0
    want = torch.einsum("hgn,hnd->hgd", torch.softmax(logits, dim=-1), vals.double()).reshape(hq, d)
    err = (out.double() - want).abs().max() / want.abs().max()
    assert float(err) < 2e-3


def test_decode_attention_entry_equals_the_three_calls():
    h, n, d, bf, group = 2, 2048, 128, 32, 4
    st, ox, keys, vals = build_both(h, n, d, bf, 3, torch.bfloat16, seed=44)
    hq = h * group
    g = torch.Generator().manual_seed(8)
    q_raw = (torch.randn((hq, d), generator=g) * 3.0).cuda()
    tau = torch.full((hq,), 0.12, device="cuda")
    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
    q_hat, ls = S.prepare_query(q_raw, d ** -0.5)
    _, ca = S.search(st, q_hat, tau, scaling=ls, flags=flags, want_compact=True)
    n_splits = S.attn_splits(st, hq, ca.tile_parents)
    ws = torch.empty((hq * n_splits * (d + 2),), device="cuda")
    out_a = S.sparse_attn(st, q_hat, ls, ca, n_splits=n_splits, workspace=ws)
    cb = S.alloc_compact(st, hq)
    qh2, ls2 = torch.empty_like(q_hat), torch.empty_like(ls)
    out_b = torch.empty_like(out_a)
    S.decode_attention(st, q_raw, d ** -0.5, tau, cb, qh2, ls2, flags=flags, n_splits=n_splits,
                       workspace=torch.empty_like(ws), out=out_b)
    torch.cuda.synchronize()
    assert torch.equal(q_hat, qh2) and torch.equal(ls, ls2)
    assert torch.equal(ca.count, cb.count) and torch.equal(out_a, out_b)
    la, lb = ca.to_lists(), cb.to_lists()
    assert all(torch.equal(x[0], y[0]) and torch.equal(x[1], y[1]) for x, y in zip(la, lb))


def test_attention_with_nothing_selected_is_zero():
    st, ox, keys, vals = build_both(1, 512, 128, 16, 3, torch.bfloat16, seed=1)
    q = make_queries(2, 128, seed=2)
    tau = torch.full((2,), 1e30, device="cuda")
    _, compact = S.search(st, q, tau, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
    out = S.sparse_attn(st, q, None, compact)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0


def test_merge_partials_matches_oracle():
    g = torch.Generator().manual_seed(0)
    po = torch.randn((4, 6, 128), generator=g)
    pml = torch.stack([torch.randn((4, 6), generator=g) * 5, torch.rand((4, 6), generator=g) * 100 + 1], dim=-1)
    pml[1, 2, 0] = float("-inf")
    pml[1, 2, 1] = 0.0
    ml = torch.zeros((6, 2), device="cuda")
    out = S.merge_partials(po.cuda().contiguous(), pml.cuda().contiguous(), out_ml=ml)
    torch.cuda.synchronize()
    want, want_ml = O.merge_partials(po, pml)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ml.cpu().numpy(), want_ml, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("s,k", [(1000, 16), (64, 64), (4096, 1), (37, 5)])
def test_threshold_matches_oracle(dtype, s, k):
    h, d, group = 2, 128, 3
    samples = make_keys(h, s, d, 13, dtype)
    q = make_queries(h * group, d, seed=14)
    for method in (L.HIRA_TAU_SAMPLE_MAX, L.HIRA_TAU_SAMPLE_MEAN_TOPK, L.HIRA_TAU_SAMPLE_KTH):
        got = S.threshold(samples, q, method, k).cpu().numpy()
        want = O.threshold(samples, q, method, k)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"method {method}"


def test_kth_score_is_exact():
    h, n, d, bf, group = 2, 3000, 128, 32, 2
    st, ox, keys, _ = build_both(h, n, d, bf, 3, torch.bfloat16, seed=17)
    hq = h * group
    q = make_queries(hq, d, seed=18)
    tau = torch.full((hq,), float("-inf"), device="cuda")
    _, compact = S.search(st, q, tau, flags=L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES, want_compact=True)
    k = torch.tensor([1, 60, 3000, 3001], dtype=torch.int32, device="cuda")
    got = S.kth_score(st, compact, k).cpu().numpy()
    o_dense, o_keep = O.search(ox, q, tau, flags=O.GATE_GT)
    for qh in range(hq):
        s = np.sort(o_dense[qh][o_keep[qh] > 0])[::-1]
        kk = int(k[qh])
        want = s[kk - 1] if kk <= len(s) else -np.inf
        assert got[qh] == want


def test_assign_matches_oracle():
    for dtype in (torch.float32, torch.bfloat16):
        pts = make_keys(2, 700, 128, 23, dtype)
        cents = make_keys(2, 90, 128, 24, dtype)
        idx, d2 = S.assign(pts, cents, use_tensor_cores=False)
        torch.cuda.synchronize()
        o_idx, o_d2 = O.assign(pts, cents)
        assert np.array_equal(idx.cpu().numpy(), o_idx)
        assert np.array_equal(d2.cpu().numpy().view(np.uint32), o_d2.view(np.uint32))


@pytest.mark.parametrize("h,n,k", [(1, 128, 128), (3, 1000, 300), (2, 4096, 128), (1, 50, 7)])
def test_assign_tensor_cores(h, n, k):
    # tcgen05 accumulates in hardware order, so a near-tie may resolve differently from the
    # fp32 FMA chain: the chosen centroid must be (numerically) a nearest one
    torch.backends.cuda.matmul.allow_tf32 = False
    pts = make_keys(h, n, 128, 71, torch.bfloat16, normalize=False)
    cents = make_keys(h, k, 128, 72, torch.bfloat16, normalize=False)
    idx, d2 = S.assign(pts, cents, use_tensor_cores=True)
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and int(idx.max()) < k, "the kernel reported a timeout (-1) or an out-of-range centroid"
    full = torch.cdist(pts.float(), cents.float()) ** 2                     # (h, n, k)
    best = full.min(dim=2).values
    chosen = full.gather(2, idx.long().unsqueeze(-1)).squeeze(-1)
    assert float((chosen - best).max()) <= 1e-3 * float(best.max())
    torch.testing.assert_close(d2, best, atol=2e-2, rtol=1e-4)
    cc_idx, _ = S.assign(pts, cents, use_tensor_cores=False)
    assert float((idx == cc_idx).float().mean()) > 0.999


def test_build_with_tensor_cores_gives_a_valid_index():
    h, n, d, bf = 2, 4096, 128, 32
    keys = make_keys(h, n, d, 81, torch.bfloat16)
    vals = make_keys(h, n, d, 82, torch.bfloat16, normalize=False)
    st = new_state(h, d, bf, 3, (n // bf // bf) * bf, torch.bfloat16)
    S.build(st, keys, vals, n_iters=2, use_tensor_cores=True)
    torch.cuda.synchronize()
    assert int((st.slot2token >= 0).sum()) == h * n and int(st.child_counts.sum()) == h * n
    tok = st.slot2token.clamp_min(0).long()
    ok = st.slot2token >= 0
    assert torch.equal(st.children[ok], keys.gather(1, tok.unsqueeze(-1).expand(-1, -1, d))[ok])
    # radii really bound their children
    pc = st.children.float().view(h, -1, bf, d)
    dist = (pc - st.parents.float()[:, :, None, :]).norm(dim=-1)
    slot_ok = torch.arange(bf, device="cuda")[None, None, :] < st.child_counts[:, :, None]
    assert bool((dist[slot_ok] <= st.parent_radii[:, :, None].expand_as(dist)[slot_ok] + 1e-4).all())
    # and the search over it still equals brute force
    q = make_queries(h * 4, d, seed=83)
    sc = torch.einsum("hnd,hgd->hgn", keys.float(), q.view(h, 4, d)).reshape(h * 4, n)
    tau = torch.sort(sc, dim=-1).values[:, int(n * 0.95)].contiguous()
    _, c = S.search(st, q, tau, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
    sets = compact_sets(c)
    s2t = st.slot2token.cpu().numpy()
    for qh in range(h * 4):
        got = set(s2t[qh // 4, sets[qh][0]].tolist())
        must = set(torch.nonzero(sc[qh] > tau[qh] + 1e-4).flatten().tolist())
        never = set(torch.nonzero(sc[qh] < tau[qh] - 1e-4).flatten().tolist())
        assert must <= got and not (got & never)


@pytest.mark.parametrize("h,n,d,bf,depth,dtype,n_iters,rounds", [
    (2, 1000, 32, 8, 3, torch.float32, 1, 1),
    (1, 4096, 128, 32, 3, torch.bfloat16, 1, 3),
    (2, 777, 64, 16, 2, torch.float32, 3, 2),
    (3, 300, 16, 5, 3, torch.float32, 1, 8),
])
def test_balanced_build_matches_oracle(h, n, d, bf, depth, dtype, n_iters, rounds):
    """Capacity-aware assignment rounds: the layout, the counts and the radii equal the oracle's, every
    key is stored once, and the balls are no larger on average than with the reference's rule."""
    keys = make_keys(h, n, d, 91, dtype, normalize=False)
    vals = make_keys(h, n, d, 92, dtype, normalize=False)
    k1 = -(-n // bf)
    k2 = -(-k1 // bf)
    cap = k2 * bf if depth == 3 else k1
    c1 = random_centres(h, n, k1, 93)
    c2 = random_centres(h, k1, k2, 94) if depth == 3 else None
    code = O.HIRA_BF16 if dtype == torch.bfloat16 else O.HIRA_F32
    radii = []
    for r in (0, rounds):
        st = new_state(h, d, bf, depth, cap, dtype)
        S.build(st, keys, vals, cent_idx1=c1, cent_idx2=c2, n_iters=n_iters, balance_rounds=r, use_tensor_cores=False)
        torch.cuda.synchronize()
        ox = O.OracleIndex(n_heads=h, dim=d, vdim=d, bf=bf, depth=depth, cap_parents=cap, dtype=code, vdtype=code)
        O.build(ox, keys, vals, cent_idx1=c1, cent_idx2=c2, n_iters=n_iters, balance_rounds=r)
        assert_index_equal(st, ox, f"balance_rounds={r}")
        tok = st.slot2token[st.slot2token >= 0].reshape(h, n).sort(dim=1).values.cpu()
        assert torch.equal(tok, torch.arange(n).expand(h, n).to(tok.dtype))
        radii.append(float(st.parent_radii[:, :k1 if depth == 2 else k2 * bf].mean()))
    assert radii[1] <= radii[0] * 1.0001, radii


def test_export_roundtrip():
    st, ox, keys, vals = build_both(2, 500, 64, 8, 3, torch.bfloat16, seed=29)
    k, v = S.export(st, 500)
    torch.cuda.synchronize()
    assert torch.equal(k, keys) and torch.equal(v, vals)


def test_bad_arguments_raise():
    st = new_state(1, 32, 8, 2, 4, torch.float32)
    q = make_queries(2, 32, seed=1)
    tau = torch.zeros((2,), device="cuda")
    with pytest.raises(ValueError):
        S.search(st, q, tau, flags=0x40, want_compact=True)
    with pytest.raises(ValueError):
        S.search(st, q, tau, flags=0)  # no output buffer
    st2 = new_state(2, 32, 8, 2, 4, torch.float32)
    with pytest.raises(ValueError):  # 3 query heads over 2 kv heads without a map
        S.search(st2, make_queries(3, 32, seed=1), torch.zeros((3,), device="cuda"), want_compact=True)
