"""The int8 tensor-core pre-filter of the search (csrc/search_q8.cu) must not change a single
emitted slot or score: every case runs the search three ways on the same index -- through the
pre-filter, through the plain streaming kernel (side copy switched off) and in the CPU oracle --
and compares bit for bit.  Cases cover the branching factors whose tiles are whole 128-row stages,
both depths and dtypes, GQA groups 1-8, partially filled tiles, thresholds from keep-all to
keep-none and on a key's own score, indexes after appends (the appends maintain the side copy),
and keys with outlier channels."""
import numpy as np
import pytest
import torch

from hira_b200 import _lib as L
from hira_b200 import index_state as S
from hira_b200 import workloads as W
from oracle import oracle as O

from util import compact_sets

pytestmark = pytest.mark.gpu
RULES = [L.HIRA_GATE_GE | L.HIRA_LEAF_GE, L.HIRA_GATE_GT | L.HIRA_LEAF_GT, L.HIRA_GATE_GT | L.HIRA_LEAF_GE]


def _build(h, n, bf, depth, dtype, dist, seed, spare=0):
    keys, vals = W.make_kv(h, n, seed, "cuda", dist=dist, dtype=dtype)
    k1 = -(-n // bf)
    k2 = -(-k1 // bf)
    tp = {8: 128, 16: 64, 32: 32, 64: 16, 128: 8}[bf]
    cap = (k2 + spare) * bf if depth == 3 else -(-(k1 + spare) // tp) * tp
    st = S.IndexState(n_heads=h, dim=128, vdim=128, bf=bf, depth=depth, cap_parents=cap, dtype=dtype, vdtype=dtype,
                      device="cuda")
    assert st.int8_copy
    S.build(st, keys, vals, cent_idx1=W.random_centres(h, n, k1, seed + 1, "cuda"),
            cent_idx2=W.random_centres(h, k1, k2, seed + 2, "cuda") if depth == 3 else None, use_tensor_cores=False)
    return st, keys


def _three_ways(st, q_hat, tau, flags, scaling=None, q2kv=None, max_group=0):
    hq = q_hat.shape[0]
    stats = S.new_stats(hq, "cuda")
    st.enable_int8_copy(True)
    _, c8 = S.search(st, q_hat, tau, scaling=scaling, q2kv=q2kv, max_group=max_group, flags=flags, want_compact=True,
                     stats=stats)
    st.enable_int8_copy(False)
    stats_p = S.new_stats(hq, "cuda")
    _, cp = S.search(st, q_hat, tau, scaling=scaling, q2kv=q2kv, max_group=max_group, flags=flags, want_compact=True,
                     stats=stats_p)
    st.enable_int8_copy(True)
    torch.cuda.synchronize()
    ox = O.OracleIndex.from_arrays(st.state_dict())
    o_dense, o_keep = O.search(ox, q_hat, tau, scaling=scaling, q2kv=q2kv, flags=flags)
    a, b = compact_sets(c8), compact_sets(cp)
    total = 0
    for qh in range(hq):
        want = np.nonzero(o_keep[qh])[0]
        assert np.array_equal(a[qh][0], want), f"query head {qh}: pre-filter path selects other slots than the oracle"
        assert np.array_equal(b[qh][0], want), f"query head {qh}: streaming path selects other slots than the oracle"
        assert np.array_equal(a[qh][1].view(np.uint32), o_dense[qh][want].view(np.uint32))
        assert np.array_equal(a[qh][1].view(np.uint32), b[qh][1].view(np.uint32))
        total += len(want)
    s8, sp = stats.cpu().numpy(), stats_p.cpu().numpy()
    assert np.array_equal(s8[:, :8], sp[:, :8]), "visit counters differ between the two kernels"
    assert (sp[:, 8:] == 0).all()
    return total, s8


@pytest.mark.parametrize("h,n,bf,depth,dtype,group,dist", [
    (2, 8192, 32, 3, torch.bfloat16, 4, "rope_outlier"),
    (1, 16384, 64, 3, torch.bfloat16, 8, "rope_outlier"),
    (2, 4096, 16, 3, torch.float32, 2, "aniso"),
    (3, 2048, 8, 2, torch.bfloat16, 1, "aniso"),
    (1, 5000, 32, 3, torch.bfloat16, 4, "rope_outlier"),      # last grandparent and parents partly filled
    (2, 3000, 128, 2, torch.float32, 3, "aniso"),              # group of 3: one head slot of the CTA unused
    (1, 2048, 64, 2, torch.bfloat16, 6, "rope_outlier"),       # two CTAs per tile (4 + 2 heads)
])
def test_prefilter_equals_streaming_kernel_and_oracle(h, n, bf, depth, dtype, group, dist):
    st, keys = _build(h, n, bf, depth, dtype, dist, seed=11 * bf + depth)
    hq = h * group
    q = W.make_queries(hq, 5, "cuda", pos=n if dist == "rope_outlier" else None)
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    sc = torch.einsum("hgd,hnd->hgn", q_hat.view(h, group, 128), keys.float()).reshape(hq, n)
    srt = torch.sort(sc, dim=-1, descending=True).values
    scaling = torch.rand((hq,), device="cuda") + 0.5
    for keep in (0.02, 0.3):
        tau = srt[:, max(0, int(keep * n) - 1)].contiguous()
        for flags in RULES:
            total, s8 = _three_ways(st, q_hat, tau, flags, scaling=scaling)
            assert total > 0
            cand, scored = int(s8[:, 8].sum()), int(s8[:, 9].sum())
            assert scored > 0 and cand >= 1
    # a threshold that sits exactly on a key's canonical score, keep-all and keep-none
    compact = S.alloc_compact(st, hq)
    S.search(st, q_hat, torch.full((hq,), float("-inf"), device="cuda"), flags=0, compact=compact)
    tau_on = S.kth_score(st, compact, torch.full((hq,), 17, dtype=torch.int32, device="cuda")).clone()
    total, _ = _three_ways(st, q_hat, tau_on, RULES[0])
    assert total == 17 * hq
    total, _ = _three_ways(st, q_hat, tau_on, RULES[1])
    assert total == 16 * hq
    total, _ = _three_ways(st, q_hat, torch.full((hq,), float("-inf"), device="cuda"), RULES[0])
    assert total == n * group * h
    total, _ = _three_ways(st, q_hat, torch.full((hq,), float("inf"), device="cuda"), RULES[0])
    assert total == 0
    # that search's gates kept nothing, so the next one streams only what its gates keep
    assert int(st.q8_chan_scale.view(torch.int32)[0, 134]) == 1    # not decided yet: decided when the next search starts
    total, _ = _three_ways(st, q_hat, tau_on, RULES[0])
    assert total == 17 * hq
    assert int(st.q8_chan_scale.view(torch.int32)[0, 134]) == 0
    total, _ = _three_ways(st, q_hat, tau_on, RULES[0])
    assert total == 17 * hq and int(st.q8_chan_scale.view(torch.int32)[0, 134]) == 1


def test_mode_flips_between_back_to_back_searches_never_cost_a_fallback():
    """The search kernel starts while the kernel that prepares its query terms (and decides the streaming
    mode from the last search's gates) may still be running.  Searches whose gates keep everything and
    searches whose gates keep nothing alternate without a pause, so the mode word flips before every other
    launch: every CTA must still agree with itself on the stages requested up front -- no bounded wait may
    run out (no CTA takes the exact fallback), and the results are those of the streaming kernel."""
    h, n, bf, group = 4, 32768, 32, 4
    st, keys = _build(h, n, bf, 3, torch.bfloat16, "rope_outlier", 77)
    hq = h * group
    q = W.make_queries(hq, 78, "cuda", pos=n)
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    scores = torch.einsum("hgd,hnd->hgn", q_hat.view(h, group, 128), keys.float()).reshape(hq, n)
    tau_mid = W.guard_banded_tau(scores, 600)
    tau_all = torch.full((hq,), float("-inf"), device="cuda")
    tau_none = torch.full((hq,), float("inf"), device="cuda")
    flags = RULES[0]
    st.enable_int8_copy(False)
    _, want = S.search(st, q_hat, tau_mid, flags=flags, want_compact=True)
    want_sets = compact_sets(want)
    st.enable_int8_copy(True)
    before = S.q8_fallback_count()
    compact = S.alloc_compact(st, hq)
    other = S.alloc_compact(st, hq)
    for i in range(40):                       # no synchronisation inside: the launches follow one another
        S.search(st, q_hat, tau_all if i % 2 == 0 else tau_none, flags=flags, compact=other)
        S.search(st, q_hat, tau_mid, flags=flags, compact=compact)
    torch.cuda.synchronize()
    assert S.q8_fallback_count() == before
    got_sets = compact_sets(compact)
    for qh in range(hq):
        assert np.array_equal(got_sets[qh][0], want_sets[qh][0])
        assert np.array_equal(got_sets[qh][1].view(np.uint32), want_sets[qh][1].view(np.uint32))


def test_prefilter_prunes_the_exact_pass_to_a_few_per_cent():
    """On the decode workload (RoPE + outlier channels, tau at 2 %) the union of candidates over a
    group of 4 query heads stays near the union of the true survivors."""
    st, keys = _build(2, 32768, 32, 3, torch.bfloat16, "rope_outlier", seed=3)
    q = W.make_queries(8, 21, "cuda", pos=32768)
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    sc = torch.einsum("hgd,hnd->hgn", q_hat.view(2, 4, 128), keys.float()).reshape(8, 32768)
    tau = torch.sort(sc, dim=-1, descending=True).values[:, 654].contiguous()
    total, s8 = _three_ways(st, q_hat, tau, RULES[0])
    assert abs(total - 8 * 655) <= 8      # tau comes from torch's scores, the kernels use the canonical ones
    cand, scored = int(s8[:, 8].sum()), int(s8[:, 9].sum())
    assert scored == 2 * 32768
    assert total / 4 <= cand <= 0.15 * scored, (cand, scored)


def test_appends_keep_the_side_copy_in_step():
    """Keys appended one at a time (into free slots, new parents, new grandparents) are found through
    the pre-filter like any other key; explicit query-head maps work as well."""
    st, keys = _build(2, 4096, 32, 3, torch.bfloat16, "rope_outlier", seed=9, spare=40)
    new_k, new_v = W.make_kv(2, 24, 77, "cuda", dist="rope_outlier", dtype=torch.bfloat16, first_pos=4096)
    for i in range(24):
        S.append(st, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0
    hq = 4
    # queries aligned with appended keys, so that those keys are among the selected ones
    q = torch.cat([new_k[0, 5:6], new_k[0, 20:21], new_k[1, 0:1], new_k[1, 23:24]]).float()
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    allk = torch.cat([keys, new_k], dim=1).float()
    sc = torch.stack([allk[i // 2] @ q_hat[i] for i in range(hq)])
    tau = torch.sort(sc, dim=-1, descending=True).values[:, 40].contiguous()
    total, s8 = _three_ways(st, q_hat, tau, RULES[0])
    assert abs(total - 41 * hq) <= hq      # tau comes from torch's scores, the kernels use the canonical ones
    assert int(s8[:, 9].sum()) > 0         # the pre-filter ran
    ox = O.OracleIndex.from_arrays(st.state_dict())
    _, keep = O.search(ox, q_hat, tau, flags=RULES[0])
    for i, j in enumerate((5, 20, 0, 23)):                      # the appended key each query was taken from is selected
        slot = int((st.slot2token[i // 2] == 4096 + j).nonzero()[0])
        assert keep[i][slot]
    # an explicit query-head map takes the streaming kernel (the pre-filter serves the default grouping)
    q2kv = torch.tensor([1, 0, 1, 0], dtype=torch.int32, device="cuda")
    total2, s8b = _three_ways(st, q_hat, tau, RULES[0], q2kv=q2kv, max_group=2)
    assert int(s8b[:, 9].sum()) == 0 and total2 > 0
    # every filled row of the side copy (built or appended) equals a torch restatement of the
    # quantiser: k' = k / s, step = max |k'| / 127, k~ = rint(k' / step), chunk j of slot r at j ^ (r & 7)
    chan = st.q8_chan_scale[:, :128].clone()
    kp = st.children.float() / chan[:, None, :]
    step = kp.abs().amax(dim=-1) / 127.0
    h16 = step.half()                                      # the step is stored as fp16, rounded up
    h16 = torch.where(h16.float() < step, torch.nextafter(h16, torch.full_like(h16, float("inf"))), h16)
    step16 = h16.float()
    filled = st.slot2token >= 0
    assert int(filled.sum()) == 2 * (4096 + 24)
    meta = st.children_q8_meta
    got_step = (meta & 0xffff).to(torch.int16).view(torch.float16).float()
    got_err = ((meta >> 16) & 0xffff).to(torch.int16).view(torch.float16).float()
    assert torch.equal(got_step[filled], step16[filled])
    kq = torch.round(kp / step16[..., None]).clamp(-127, 127).to(torch.int8)
    capC = st.cap_children
    swz = (torch.arange(capC, device="cuda") & 7)[:, None]
    phys = (torch.arange(8, device="cuda")[None, :] ^ swz)                        # (capC, 8): where logical chunk j sits
    stored = st.children_q8.view(2, capC, 8, 16).gather(2, phys[None, :, :, None].expand(2, -1, -1, 16)).reshape(2, capC, 128)
    assert torch.equal(stored[filled], kq[filled])
    err = (kp - kq.float() * step16[..., None]).norm(dim=-1)
    assert bool((got_err[filled] >= err[filled]).all())
