"""Parity at the shapes and on the data the decode path is measured on (hira_b200/workloads.py):
bf16, D = 128, un-normalised keys with RoPE and outlier channels, 32,768 / 131,072 keys per head,
branching 32 and 64, GQA groups of 4 and 8 -- the CUDA library through its C ABI against the CPU
oracle, bit for bit (selected sets, scores, slot contents), and against the candidate sets the
reference's own GPU searcher produced on a B200 (tests/golden/search_triton_gpu_*.npz).
"""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from hira_b200 import _lib as L
from hira_b200 import index_state as S
from hira_b200 import workloads as W
from oracle import oracle as O

from util import assert_index_equal, compact_sets

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
CPU_RULE = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
GPU_RULE = L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES


def build_workload(w: W.Workload, n_heads=None, spare_gp=0, n_iters=1):
    """Index of the first `n_heads` (batch, kv head) groups of `w`, built on the device from
    device-generated data; returns (state, keys, values, unit queries)."""
    keys, vals, q = W.make_inputs(w, "cuda", n_heads=n_heads)
    h, n, d = keys.shape
    bf = w.branching
    k1 = n // bf
    k2 = -(-k1 // bf)
    st = S.IndexState(n_heads=h, dim=d, vdim=d, bf=bf, depth=w.levels, cap_parents=(k2 + spare_gp) * bf,
                      dtype=w.dtype, vdtype=w.dtype, device="cuda")
    S.build(st, keys, vals, cent_idx1=W.random_centres(h, n, k1, 7, "cuda"),
            cent_idx2=W.random_centres(h, k1, k2, 8, "cuda"), n_iters=n_iters, use_tensor_cores=False)
    q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0
    return st, keys, vals, q_hat


def exact_tau(st, q_hat, kth):
    """tau = the kth largest canonical score of each query head: a key sits exactly on it."""
    hq = q_hat.shape[0]
    compact = S.alloc_compact(st, hq)
    S.search(st, q_hat, torch.full((hq,), float("-inf"), device="cuda"), flags=GPU_RULE, compact=compact)
    return S.kth_score(st, compact, torch.full((hq,), kth, dtype=torch.int32, device="cuda")).clone()


def assert_search_equals_oracle(st, ox, q_hat, tau, scaling, flags, expect_selected=None):
    hq = q_hat.shape[0]
    stats = S.new_stats(hq, "cuda")
    _, compact = S.search(st, q_hat, tau, scaling=scaling, flags=flags, want_compact=True, stats=stats)
    torch.cuda.synchronize()
    o_dense, o_keep, o_stats = O.search(ox, q_hat, tau, scaling=scaling, flags=flags, want_stats=True)
    total = 0
    for qh, (slots, scores) in enumerate(compact_sets(compact)):
        want = np.nonzero(o_keep[qh])[0]
        assert np.array_equal(slots, want), f"query head {qh}: selected slots differ"
        assert np.array_equal(scores.view(np.uint32), o_dense[qh][want].view(np.uint32)), f"query head {qh}: scores differ"
        total += len(slots)
    assert np.array_equal(stats.cpu().numpy().astype(np.uint32)[:, :6], o_stats[:, :6]), "visit counters differ"
    if expect_selected is not None:
        assert total == expect_selected
    return compact, o_dense, o_keep


def test_cfg1_build_matches_oracle_at_full_context():
    """2 of the 8 KV heads (the oracle's assignment is the slow part), 32,768 keys each."""
    w = W.CFG1
    st, keys, vals, _ = build_workload(w, n_heads=2)
    h, n, d = keys.shape
    ox = O.OracleIndex(n_heads=h, dim=d, vdim=d, bf=w.branching, depth=3, cap_parents=st.cap_parents,
                       dtype=O.HIRA_BF16, vdtype=O.HIRA_BF16)
    O.build(ox, keys, vals, cent_idx1=W.random_centres(h, n, n // w.branching, 7, "cuda"),
            cent_idx2=W.random_centres(h, n // w.branching, n // w.branching ** 2, 8, "cuda"))
    assert_index_equal(st, ox, "cfg1 build")


def test_cfg1_search_and_attention_match_oracle():
    """BASELINE configuration 1 whole: 8 KV x 32,768 bf16 keys, 32 query heads, 3 levels of
    branching 32, tau = the exact 2 % score (a key on the boundary in every head)."""
    w = W.CFG1
    st, keys, vals, q_hat = build_workload(w)
    ox = O.OracleIndex.from_arrays(st.state_dict())
    hq = q_hat.shape[0]
    tau = exact_tau(st, q_hat, w.kth)
    scaling = (torch.rand((hq,), device="cuda") + 0.5) * W.DIM ** -0.5 * 19.0
    compact, o_dense, o_keep = assert_search_equals_oracle(st, ox, q_hat, tau, scaling, CPU_RULE,
                                                           expect_selected=hq * w.kth)
    assert_search_equals_oracle(st, ox, q_hat, tau, scaling, GPU_RULE)
    assert_search_equals_oracle(st, ox, q_hat, tau, None, L.HIRA_GATE_GT | L.HIRA_LEAF_GT, expect_selected=hq * (w.kth - 1))
    out = S.sparse_attn(st, q_hat, scaling, compact)
    want, _ = O.attention(ox, q_hat, scaling, o_dense, o_keep)
    err = np.abs(out.cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 2e-3, err


@pytest.mark.parametrize("cfg", ["cfg2", "cfg4"])
def test_long_context_step_with_appends_matches_oracle(cfg):
    """One batch item of configuration 2 (8 KV x 131,072 keys, branching 32, groups of 4) and
    one sequence shard of configuration 4 (branching 64, groups of 8): 16 decode steps, each a
    search whose parent read also finds the nearest parent of the key appended right after;
    the index then equals the oracle's after 16 appends and the final search selects the same
    keys, bit for bit."""
    w = W.CONFIGS[cfg]
    st, keys, vals, q_hat = build_workload(w, n_heads=w.kv_heads, spare_gp=40)
    ox = O.OracleIndex.from_arrays(st.state_dict())
    h, n, d = keys.shape
    hq = q_hat.shape[0]
    tau = exact_tau(st, q_hat, w.kth)
    scaling = torch.full((hq,), 19.0 * W.DIM ** -0.5, device="cuda")
    st.active_parents = (n // w.branching // w.branching + 34) * w.branching   # bound grown by the worst case
    new_k, new_v = W.make_kv(h, 16, 9000, "cuda", dist=w.dist, dtype=w.dtype, first_pos=n)
    compact = S.alloc_compact(st, hq)
    scan = S.new_scan_slots(st)
    for i in range(16):
        S.search(st, q_hat, tau, scaling=scaling, flags=CPU_RULE, compact=compact,
                 scan_key=new_k[:, i].contiguous(), scan_out=scan)
        S.append_scanned(st, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous(), scan)
        O.append(ox, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0 and int(ox.status[0]) == 0
    assert_index_equal(st, ox, f"{cfg} after 16 appends")
    st.active_parents = 0
    compact, o_dense, o_keep = assert_search_equals_oracle(st, ox, q_hat, tau, scaling, CPU_RULE)
    out = S.sparse_attn(st, q_hat, scaling, compact)
    want, _ = O.attention(ox, q_hat, scaling, o_dense, o_keep)
    assert np.abs(out.cpu().numpy() - want).max() / np.abs(want).max() < 2e-3


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("cfg", ["cfg1", "cfg4"])
def test_candidate_sets_equal_the_reference_gpu_searcher(cfg):
    """The reference's CUDASearcher (its Triton kernels, on a B200) was run on this index --
    same seeds, same build -- by tests/golden/make_golden.py --gpu; the fixture holds its
    candidate bitmaps.  hira_search with the reference GPU rule (gate >, every child of a kept
    parent) must produce the same sets.  Even query heads carry the workload's 2 % threshold
    (nothing is pruned on this data), odd ones the median gate value (about half is)."""
    path = GOLDEN / f"search_triton_gpu_{cfg}.npz"
    if not path.exists():
        pytest.skip(f"{path.name} has not been generated (needs the reference checkout and a GPU)")
    rec = dict(np.load(path))
    w = W.CONFIGS[cfg]
    st, keys, vals, q_hat = build_workload(w, n_heads=w.kv_heads)
    if _sha(keys) != str(rec["keys_sha"]) or _sha(q_hat) != str(rec["q_sha"]):
        pytest.skip("the device-generated inputs differ from the ones the fixture was made on "
                    "(another torch / GPU generation): regenerate the fixture")
    assert _sha(st.children) == str(rec["children_sha"]), "the build laid the index out differently"
    tau = torch.from_numpy(rec["tau"]).cuda()
    _, compact = S.search(st, q_hat, tau, flags=GPU_RULE, want_compact=True)
    torch.cuda.synchronize()
    n = int(rec["n"])
    want = np.unpackbits(rec["expected_mask"], axis=-1)[:, :n].astype(bool)
    assert bool(rec["equal_when_generated"])
    for qh, (slots, _) in enumerate(compact_sets(compact)):
        assert np.array_equal(slots, np.nonzero(want[qh])[0]), f"query head {qh}"
    per_head = want.sum(axis=-1)
    assert (per_head[0::2] == n).all() and (per_head[1::2] < n).all() and (per_head[1::2] > 0).all()
