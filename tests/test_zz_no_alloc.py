"""The allocation-free attention entry point against the regular one.

`hira_sparse_attn_noalloc` serves callers that cannot hand the library a device
workspace (no cudaMalloc allowed after warm-up, plugin hosts that only pass inputs and
outputs, plain C hosts): its split-KV partials live in an array inside the library.  It
must give the same attention output as `hira_sparse_attn`, also on a second call that
finds the first call's partials still in the array.  The file name sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from hira_b200 import _lib as L
from hira_b200 import index_state as S

pytestmark = pytest.mark.gpu


def _case(seed, h=2, n=2048, d=128, bf=32, group=4, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    keys = torch.randn((h, n, d), generator=g).to(dtype).cuda()
    vals = torch.randn((h, n, d), generator=g).to(dtype).cuda()
    q = torch.randn((h * group, d), generator=g)
    q = (q / q.norm(dim=-1, keepdim=True)).cuda()
    st = S.IndexState(n_heads=h, dim=d, vdim=d, bf=bf, depth=3, cap_parents=n // bf, dtype=dtype, vdtype=dtype,
                      device="cuda")
    S.build(st, keys, vals, use_tensor_cores=False)
    tau = torch.full((h * group,), 0.12, device="cuda")
    scaling = torch.full((h * group,), 6.0, device="cuda")
    _, compact = S.search(st, q, tau, scaling=scaling, flags=L.HIRA_GATE_GE | L.HIRA_LEAF_GE, want_compact=True)
    qk = torch.randn((h, 3, d), generator=g).to(dtype).cuda()
    qv = torch.randn((h, 3, d), generator=g).to(dtype).cuda()
    return st, q, scaling, compact, qk, qv


def _noalloc(st, q, scaling, compact, qk, qv, n_splits):
    lib = L.load()
    hq = q.shape[0]
    out = torch.empty((hq, st.vdim), dtype=torch.float32, device="cuda")
    ml = torch.empty((hq, 2), dtype=torch.float32, device="cuda")
    rc = lib.hira_sparse_attn_noalloc(st.struct, L.ptr(q), L.ptr(scaling), None, hq, compact.tile_parents,
                                      L.ptr(compact.idx), L.ptr(compact.score), L.ptr(compact.count), L.ptr(qk),
                                      L.ptr(qv), qk.shape[1], qk.shape[1] * st.dim, n_splits, L.ptr(out), L.ptr(ml),
                                      0, 0, L.current_stream())
    return rc, out, ml


def test_noalloc_attention_matches_workspace_attention_twice():
    for call, seed in enumerate((101, 202)):          # two calls in a row, different data
        st, q, scaling, compact, qk, qv = _case(seed)
        n_splits = 3
        ml_ref = torch.empty((q.shape[0], 2), dtype=torch.float32, device="cuda")
        ref = S.sparse_attn(st, q, scaling, compact, queued_k=qk, queued_v=qv, n_splits=n_splits, out_ml=ml_ref)
        rc, out, ml = _noalloc(st, q, scaling, compact, qk, qv, n_splits)
        torch.cuda.synchronize()
        assert rc == 0, L.load().hira_last_error()
        # both entry points launch the same kernels in the same order; only the address of the
        # partials differs, so the results are the same bits
        assert torch.equal(out, ref), f"call {call}: outputs differ"
        assert torch.equal(ml, ml_ref), f"call {call}: (max, denominator) differ"


def test_noalloc_attention_rejects_oversized_requests():
    st, q, scaling, compact, qk, qv = _case(7)
    too_many = L.NOALLOC_SCRATCH_FLOATS // (q.shape[0] * (st.vdim + 2)) + 1
    rc, _, _ = _noalloc(st, q, scaling, compact, qk, qv, too_many)
    assert rc == L.HIRA_ERR_CAPACITY
    assert b"exceed the built-in scratch" in L.load().hira_last_error()
