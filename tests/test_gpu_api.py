"""The reference-facing Python classes on a GPU, written after the reference's own tests
(tests/test_cuda_indexer_searcher.py, tests/test_customized.py, tests/test_cuda_pipeline.py):
structure invariants of the blocked index, exact selected sets with a midpoint threshold,
scaling / GQA behaviour, value alignment, update == rebuild recall, cache + attention end to end."""
import numpy as np
import pytest
import torch

from hira_b200 import (CUDAIndexer, CUDASearcher, HiraCache, HiraConfig, hira_attention, hira_decode_attention,
                       sample_max, sample_mean_topk)

pytestmark = pytest.mark.gpu


def _keys(h, n, d, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((1, h, n, d), generator=g)
    return (x / x.norm(dim=-1, keepdim=True)).to(dtype).cuda()


def _query(hq, d, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((1, hq, 1, d), generator=g)
    return (q / q.norm(dim=-1, keepdim=True)).cuda()


def _half_threshold(scores):
    s = torch.sort(scores, dim=-1).values
    n = s.shape[-1]
    return 0.5 * (s[:, n // 2 - 1] + s[:, n // 2])


def _valid_slots(ix):
    return ix.slot2token >= 0


@pytest.mark.parametrize("levels,h,n,d,bf", [(2, 2, 256, 32, 8), (3, 2, 1000, 64, 8), (3, 4, 2048, 128, 32), (2, 1, 130, 16, 10)])
def test_index_structure_invariants(levels, h, n, d, bf):
    keys, vals = _keys(h, n, d, 1), _keys(h, n, d, 2)
    ix = CUDAIndexer(levels, 1, bf).build(keys, vals)
    m = -(-n // bf)
    if levels == 3:
        g = -(-m // bf)
        assert tuple(ix.grand_parents.shape) == (h, g, d) and tuple(ix.grand_parent_radii.shape) == (h, g)
        assert tuple(ix.parents.shape) == (h, g * bf, d) and tuple(ix.children.shape) == (h, g * bf * bf, d)
        assert ix._gp_child_counts.min() >= 0 and ix._gp_child_counts.max() <= bf
    else:
        assert tuple(ix.parents.shape) == (h, m, d) and tuple(ix.children.shape) == (h, m * bf, d)
    assert tuple(ix.values.shape) == (1, h, ix.children.shape[1], d)
    assert int(_valid_slots(ix).sum()) == h * n
    assert ix._child_counts.dtype == torch.int32 and 0 <= int(ix._child_counts.min()) and int(ix._child_counts.max()) <= bf
    assert ix._parent_valid.dtype == torch.bool and int(ix._child_counts[~ix._parent_valid].sum()) == 0
    # pad rows are zero, values follow their keys
    pad = ~_valid_slots(ix)
    assert float(ix.children[pad].abs().sum()) == 0.0 and float(ix.values[0][pad].abs().sum()) == 0.0
    tok = ix.slot2token.clamp_min(0).long()
    gathered_k = keys[0].gather(1, tok.unsqueeze(-1).expand(-1, -1, d))
    gathered_v = vals[0].gather(1, tok.unsqueeze(-1).expand(-1, -1, d))
    assert torch.equal(ix.children[~pad], gathered_k[~pad]) and torch.equal(ix.values[0][~pad], gathered_v[~pad])
    # radii equal the radii recomputed from the layout, torch-side (indexer/cuda.py:114-150)
    pc = ix.children.float().view(h, -1, bf, d)
    dist = (pc - ix.parents.float()[:, :, None, :]).norm(dim=-1)
    slot_ok = torch.arange(bf, device="cuda")[None, None, :] < ix._child_counts[:, :, None]
    want = torch.where(slot_ok, dist, torch.full_like(dist, float("-inf"))).max(dim=2).values.clamp_min(0)
    torch.testing.assert_close(ix.parent_radii, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("layout", ["4d", "2d"])
@pytest.mark.parametrize("h,hq,n,d", [(1, 1, 128, 32), (2, 2, 256, 64), (2, 4, 192, 32)])
def test_exact_set_with_midpoint_threshold_bf1(h, hq, n, d, layout):
    # every key its own parent, radius 0: the tree search must equal thresholded brute force
    keys = _keys(h, n, d, 11)
    ix = CUDAIndexer(2, 1, 1).build(keys)
    q = _query(hq, d, 111)
    kk = ix.children.index_select(0, torch.arange(hq, device="cuda") // (hq // h))
    gt = torch.einsum("hd,hnd->hn", q[0, :, 0], kk)
    tau = _half_threshold(gt)
    pred = CUDASearcher(block_c=1).search(q if layout == "4d" else q[0, :, 0].contiguous(), tau, ix)
    mask = gt > tau[:, None]
    assert torch.equal(pred != 0, mask)
    torch.testing.assert_close(pred, torch.where(mask, gt, torch.zeros_like(gt)), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("levels,bf", [(2, 8), (3, 8), (3, 32)])
def test_search_recall_scaling_and_gqa(levels, bf):
    h, hq, n, d = 2, 8, 4096, 128
    keys = _keys(h, n, d, 21)
    ix = CUDAIndexer(levels, 1, bf).build(keys)
    q = _query(hq, d, 22)
    q2kv = torch.arange(hq) // (hq // h)
    kk = ix.children.index_select(0, q2kv.cuda())
    gt = torch.einsum("hd,hnd->hn", q[0, :, 0], kk)
    tau = torch.sort(gt, dim=-1).values[:, int(n * 0.9)]
    s = CUDASearcher(block_c=bf)
    out = s.search(q, tau, ix).clone()
    true = gt > tau[:, None] + 1e-5
    assert bool(((out != 0) | ~true).all())                                 # recall 1: no true key missed
    torch.testing.assert_close(out[true], gt[true], atol=1e-4, rtol=1e-4)   # returned scores are the dot products
    # tau = -2 on unit vectors: everything is emitted and equals brute force on valid rows
    allout = s.search(q, torch.full((hq,), -2.0, device="cuda"), ix).clone()
    valid = _valid_slots(ix).index_select(0, q2kv.cuda())
    torch.testing.assert_close(allout[valid], gt[valid], atol=1e-4, rtol=1e-4)
    # scaling multiplies scores and never changes the set; zero scaling gives all zeros
    sc = torch.linspace(0.5, 3.0, hq, device="cuda")
    scaled = s.search(q, tau, ix, scaling=sc).clone()
    assert torch.equal(scaled != 0, out != 0)
    torch.testing.assert_close(scaled, out * sc[:, None], atol=1e-5, rtol=1e-5)
    assert float(s.search(q, tau, ix, scaling=torch.zeros(hq, device="cuda")).abs().max()) == 0.0
    # explicit, non-monotone head map
    m = torch.tensor([1, 0, 1, 0, 0, 1, 1, 0])
    mapped = s.search(q, tau, ix, q_head_to_kv=m).clone()
    for qh in range(hq):
        ref = torch.einsum("d,nd->n", q[0, qh, 0], ix.children[m[qh]])
        sel = mapped[qh] != 0
        torch.testing.assert_close(mapped[qh][sel], ref[sel], atol=1e-4, rtol=1e-4)
        assert bool((sel | ~(ref > tau[qh] + 1e-5)).all())
    # the CPU rule returns exactly the thresholded set
    exact = CUDASearcher(block_c=bf, gate="ge", leaf="ge").search(q, tau, ix)
    assert bool(((exact != 0) == ((gt >= tau[:, None]) & valid))[((gt - tau[:, None]).abs() > 1e-5)].all())


def test_bad_inputs_raise_value_error():
    ix = CUDAIndexer(2, 1, 8).build(_keys(2, 64, 32, 1))
    s = CUDASearcher(block_c=8)
    with pytest.raises(ValueError):
        s.search(torch.randn(3, 16).cuda(), torch.zeros(3).cuda(), ix)          # wrong dim
    with pytest.raises(ValueError):
        s.search(_query(2, 32, 1), torch.zeros(3).cuda(), ix)                   # wrong threshold length
    with pytest.raises(ValueError):
        ix.update(torch.randn(2, 2, 7, 32).cuda()[0])                           # not 4-D
    with pytest.raises(ValueError):
        CUDASearcher(block_c=8).search(_query(2, 32, 1), torch.zeros(2).cuda(), CUDAIndexer(2, 1, 8))  # not built
    with pytest.raises(ValueError):
        CUDAIndexer(1, 1, 8)                                                    # fewer than 2 levels
    deep = CUDAIndexer(5, 1, 8)                                                 # deeper trees are served by 3 levels
    assert deep.requested_levels == 5 and deep.depth == CUDAIndexer.DEPTH.THREE_LEVELS


@pytest.mark.parametrize("levels", [2, 3])
@pytest.mark.parametrize("max_context", [None, 700])
def test_update_matches_brute_force_and_keeps_values_aligned(levels, max_context):
    h, n, d, bf, extra = 2, 512, 64, 8, 96
    keys, vals = _keys(h, n + extra, d, 31), _keys(h, n + extra, d, 32)
    vals[..., 0] = torch.arange(n + extra, device="cuda")[None, None, :]        # tag every value with its token id
    ix = CUDAIndexer(levels, 1, bf, max_context=max_context).build(keys[:, :, :n], vals[:, :, :n])
    pos = n
    for m in (1, 1, 6, 24, 64):
        ix.update(keys[:, :, pos:pos + m], vals[:, :, pos:pos + m])
        pos += m
    ix.check_status()
    assert int(_valid_slots(ix).sum()) == h * (n + extra)
    valid = _valid_slots(ix)
    tok = ix.slot2token.long()
    assert torch.equal(ix.values[0][..., 0][valid], tok[valid].float())
    assert torch.equal(ix.children[valid], keys[0].gather(1, tok.clamp_min(0).unsqueeze(-1).expand(-1, -1, d))[valid])
    q = _query(h, d, 33)
    gt = torch.einsum("hd,hnd->hn", q[0, :, 0], keys[0])
    tau = _half_threshold(gt)
    out = CUDASearcher(block_c=bf, gate="ge", leaf="ge").search(q, tau, ix)
    for hh in range(h):
        got = set(tok[hh][out[hh] != 0].tolist())
        assert got == set(torch.nonzero(gt[hh] > tau[hh]).flatten().tolist())
    # a full rebuild over the stored keys selects the same tokens; with pre-allocated room the arrays
    # are reused, and whatever the old layout held beyond the new one is cleared
    before = ix.state
    ix.rebuild()
    if max_context is not None:
        assert ix.state is before
    out2 = CUDASearcher(block_c=bf, gate="ge", leaf="ge").search(q, tau, ix)
    for hh in range(h):
        assert set(ix.slot2token[hh][out2[hh] != 0].tolist()) == set(torch.nonzero(gt[hh] > tau[hh]).flatten().tolist())
    valid = _valid_slots(ix)
    assert int(valid.sum()) == h * (n + extra)
    assert float(ix.children[~valid].abs().sum()) == 0.0 and float(ix.values[0][~valid].abs().sum()) == 0.0
    assert int(ix._child_counts.sum()) == h * (n + extra)
    ix.update(keys[:, :, :3], vals[:, :, :3])               # and the rebuilt index takes appends again
    ix.check_status()
    assert int(_valid_slots(ix).sum()) == h * (n + extra + 3)


def test_state_dict_roundtrip():
    ix = CUDAIndexer(3, 1, 8).build(_keys(2, 300, 32, 5), _keys(2, 300, 32, 6))
    sd = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in ix.state_dict().items()}
    ix2 = CUDAIndexer.from_state_dict(sd)
    q, tau = _query(2, 32, 7), torch.zeros(2).cuda()
    assert torch.equal(CUDASearcher(8).search(q, tau, ix).clone(), CUDASearcher(8).search(q, tau, ix2))


def test_threshold_finders():
    samples, q = _keys(2, 500, 64, 41)[0], _query(4, 64, 42)
    sc = torch.einsum("hgd,hsd->hgs", q[0, :, 0].view(2, 2, 64), samples).reshape(4, 500)
    torch.testing.assert_close(sample_max(samples, q), sc.max(dim=1).values, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(sample_mean_topk(samples, q, 16), sc.topk(16, dim=1).values.mean(dim=1), atol=1e-5, rtol=1e-5)


class _ModelCfg:
    num_hidden_layers = 2

    def get_text_config(self, decoder=True):
        return self


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_cache_and_attention_end_to_end(dtype, tol):
    b, hkv, hq, n, d = 2, 2, 4, 1024, 64
    cfg = HiraConfig(device_mode="cuda_only", update_every=4, num_levels=3, branching_factor=16, max_context=1200)
    cache = HiraCache(_ModelCfg(), cfg)
    g = torch.Generator().manual_seed(0)
    k = torch.randn((b, hkv, n + 6, d), generator=g).to(dtype).cuda()
    v = torch.randn((b, hkv, n + 6, d), generator=g).to(dtype).cuda()
    qp = torch.randn((b, hq, n, d), generator=g).to(dtype).cuda()
    out, _ = cache.update(k[:, :, :n], v[:, :, :n], 0)
    pre, _ = hira_attention(None, qp, out, None, None, scaling=d ** -0.5)
    ref = torch.nn.functional.scaled_dot_product_attention(qp, k[:, :, :n], v[:, :, :n], is_causal=True, enable_gqa=True)
    torch.testing.assert_close(pre, ref.transpose(1, 2), atol=tol, rtol=tol)
    for t in range(6):                      # decode: 4 queued keys are flushed into the index, 2 stay queued
        out, _ = cache.update(k[:, :, n + t:n + t + 1], v[:, :, n + t:n + t + 1], 0)
    assert cache.get_seq_length(0) == n + 6 and out.queued_keys.shape[2] == 2
    out.indexer.check_status()
    q = torch.randn((b, hq, 1, d), generator=g).to(dtype).cuda()
    # a threshold below every score: sparse attention over everything == dense attention
    low = torch.full((b * hq,), -1e30, device="cuda")
    got = hira_decode_attention(q, out, scaling=d ** -0.5, threshold=low)
    dense = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), enable_gqa=True)
    torch.testing.assert_close(got, dense, atol=tol, rtol=tol)
    # with the on-device threshold finder: equals softmax restricted to the selected keys
    got2, compact = hira_decode_attention(q, out, scaling=d ** -0.5, threshold_method="sample_mean_topk", topk=32,
                                          sample_size=256, return_compact=True)
    ix = out.indexer
    sets = compact.to_lists()
    qf = q.float().reshape(b * hq, d)
    for qh in range(b * hq):
        h = qh // (hq // hkv)
        slots = sets[qh][0].long().cuda()
        kk = torch.cat([ix.children[h][slots].float(), out.queued_keys.reshape(b * hkv, -1, d)[h].float()])
        vv = torch.cat([ix.values[0][h][slots].float(), out.queued_values.reshape(b * hkv, -1, d)[h].float()])
        w = torch.softmax((kk @ qf[qh]) * d ** -0.5, dim=0)
        torch.testing.assert_close(got2.reshape(b * hq, d)[qh], w @ vv, atol=tol, rtol=tol)
    a, _ = hira_attention(None, q, out, None, None, scaling=d ** -0.5, hira_config=cfg)
    assert tuple(a.shape) == (b, 1, hq, d) and a.dtype == dtype


def test_patched_llama_generates_like_dense_attention():
    """A (tiny, random) Hugging Face Llama with `hira` registered as its attention and a
    HiraCache as `past_key_values`: with the threshold switched off the index must reproduce
    dense attention, token for token, through prefill, queued keys and index appends."""
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM
    from hira_b200 import register_hira_attention
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=2048)
    model = LlamaForCausalLM(cfg).cuda().eval()
    ids = torch.randint(0, 512, (1, 300), device="cuda")
    hcfg = HiraConfig(device_mode="cuda_only", update_every=3, num_levels=3, branching_factor=8, max_context=400,
                      threshold_method="none")
    name = register_hira_attention(hcfg)
    with torch.no_grad():
        model.config._attn_implementation = "sdpa"
        ref_cache = DynamicCache(config=cfg)
        ref = [model(ids, past_key_values=ref_cache, use_cache=True).logits[:, -1]]
        model.config._attn_implementation = name
        cache = HiraCache(cfg, hcfg)
        got = [model(ids, past_key_values=cache, use_cache=True).logits[:, -1]]
        tok = ref[0].argmax(-1, keepdim=True)
        for _ in range(7):
            model.config._attn_implementation = "sdpa"
            ref.append(model(tok, past_key_values=ref_cache, use_cache=True).logits[:, -1])
            model.config._attn_implementation = name
            got.append(model(tok, past_key_values=cache, use_cache=True).logits[:, -1])
            tok = ref[-1].argmax(-1, keepdim=True)
    assert cache.get_seq_length(0) == 307
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, atol=2e-3, rtol=2e-3)
        assert torch.equal(a.argmax(-1), b.argmax(-1))


@pytest.mark.parametrize("levels", [2, 3])
def test_active_bound_skips_empty_capacity_without_changing_results(levels):
    """An index sized for a long context visits only the tiles that can hold keys: the host's
    bound (tightened from the device counters by an asynchronous copy) leaves selected sets,
    scores and attention output unchanged."""
    from hira_b200 import index_state as S
    from hira_b200.cache import CacheOutput
    h, hq, n, d, bf = 2, 4, 2048, 64, 8
    keys, vals = _keys(h, n, d, 41), _keys(h, n, d, 42)
    ix = CUDAIndexer(levels, 1, bf, max_context=n + 4096, reserve_worst_case=True).build(keys, vals)
    more_k, more_v = _keys(h, 24, d, 43), _keys(h, 24, d, 44)
    for i in range(24):
        ix.update(more_k[:, :, i:i + 1], more_v[:, :, i:i + 1])
    torch.cuda.synchronize()
    ix.update(_keys(h, 1, d, 45), _keys(h, 1, d, 46))       # reads the counters copied back meanwhile
    ix.check_status()
    st = ix.state
    bound = ix.active_parents
    used = st.used.max(dim=0).values.tolist()
    in_use = used[1] * bf if levels == 3 else used[0]
    assert in_use <= bound < st.cap_parents // 2            # tight, far below the capacity
    q = _query(hq, d, 47)
    tau = torch.full((hq,), 0.1, device="cuda")
    srch = CUDASearcher(bf, gate="ge", leaf="ge")
    empty = torch.empty((1, h, 0, d), device="cuda")
    co = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=ix,
                     searcher=srch)
    out_b, comp_b = hira_decode_attention(q, co, threshold=tau, return_compact=True)
    assert st.active_parents == bound and comp_b.n_tiles_active < comp_b.count.shape[1]
    lists_b = comp_b.to_lists()
    kth_b = S.kth_score(st, comp_b, torch.full((hq,), 5, dtype=torch.int32, device="cuda")).clone()
    out_b = out_b.clone()
    # the same with the bound switched off
    ix._gp_bound, ix._parents_bound = st.cap_gp, st.cap_parents
    out_f, comp_f = hira_decode_attention(q, co, threshold=tau, return_compact=True)
    assert st.active_parents == 0 and comp_f.n_tiles_active is None
    lists_f = comp_f.to_lists()
    kth_f = S.kth_score(st, comp_f, torch.full((hq,), 5, dtype=torch.int32, device="cuda"))
    assert sum(len(a[0]) for a in lists_f) > 0
    for a, b in zip(lists_b, lists_f):
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # the split of the tile range over CTAs differs, so the output may differ in the last bits
    assert torch.allclose(out_b, out_f, rtol=1e-5, atol=1e-6) and torch.equal(kth_b, kth_f)


@pytest.mark.parametrize("levels", [2, 3])
def test_scanned_update_through_the_public_classes(levels):
    """hira_decode_attention(append_key=k) + update(k, v, scanned=True) leaves the same index and
    the same attention output as the plain decode_attention + update."""
    from hira_b200.cache import CacheOutput
    h, hq, n, d, bf = 2, 4, 1024, 64, 8
    keys, vals = _keys(h, n, d, 51), _keys(h, n, d, 52)
    a = CUDAIndexer(levels, 1, bf, max_context=n + 64, seed=3).build(keys, vals)
    b = CUDAIndexer(levels, 1, bf, max_context=n + 64, seed=3).build(keys, vals)
    more_k, more_v = _keys(h, 20, d, 53), _keys(h, 20, d, 54)
    tau = torch.full((hq,), 0.1, device="cuda")
    empty = torch.empty((1, h, 0, d), device="cuda")
    ca = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=a,
                     searcher=CUDASearcher(bf))
    cb = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=b,
                     searcher=CUDASearcher(bf))
    for i in range(20):
        q = _query(hq, d, 60 + i)
        k, v = more_k[:, :, i:i + 1], more_v[:, :, i:i + 1]
        oa = hira_decode_attention(q, ca, threshold=tau)
        a.update(k, v)
        ob = hira_decode_attention(q, cb, threshold=tau, append_key=k)
        b.update(k, v, scanned=True)
        assert torch.equal(oa, ob)
    a.check_status(), b.check_status()
    for name in a.state.ARRAYS:
        x, y = getattr(a.state, name), getattr(b.state, name)
        assert x is None and y is None or torch.equal(x, y), name
    with pytest.raises(ValueError):
        b.update(more_k[:, :, :1], more_v[:, :, :1], scanned=True)      # no search scanned for this key


def test_update_on_a_side_stream_beside_the_attention():
    """update(..., stream=side) runs the append while the decode step's attention is still going;
    index and attention output stay identical to the one-stream order, step after step."""
    from hira_b200.cache import CacheOutput
    h, hq, n, d, bf = 2, 4, 4096, 64, 16
    keys, vals = _keys(h, n, d, 81), _keys(h, n, d, 82)
    a = CUDAIndexer(3, 1, bf, max_context=n + 64, seed=5).build(keys, vals)
    b = CUDAIndexer(3, 1, bf, max_context=n + 64, seed=5).build(keys, vals)
    more_k, more_v = _keys(h, 30, d, 83).cpu().pin_memory(), _keys(h, 30, d, 84).cpu().pin_memory()
    tau = torch.full((hq,), 0.1, device="cuda")
    empty = torch.empty((1, h, 0, d), device="cuda")
    ca = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=a,
                     searcher=CUDASearcher(bf))
    cb = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=b,
                     searcher=CUDASearcher(bf))
    side = torch.cuda.Stream()
    for i in range(30):
        q = _query(hq, d, 90 + i)
        oa = hira_decode_attention(q, ca, threshold=tau)
        a.update(more_k[:, :, i:i + 1].cuda(), more_v[:, :, i:i + 1].cuda())
        ob = hira_decode_attention(q, cb, threshold=tau)
        with torch.cuda.stream(side):
            k = more_k[:, :, i:i + 1].to("cuda", non_blocking=True)
            v = more_v[:, :, i:i + 1].to("cuda", non_blocking=True)
        b.update(k, v, stream=side)
        assert torch.equal(oa, ob)
    a.check_status(), b.check_status()
    for name in a.state.ARRAYS:
        x, y = getattr(a.state, name), getattr(b.state, name)
        assert x is None and y is None or torch.equal(x, y), name


@pytest.mark.parametrize("levels", [3, 2])
def test_decode_step_replayed_from_cuda_graphs_equals_the_plain_step(levels):
    """HiraDecodeStep(graph_steps=5): the library call recorded into a CUDA graph per set of host buffers
    and replayed while the host refills the buffers in place, recorded anew every 5 appends (12 steps:
    three recordings, two buffer sets) -- same outputs and the same index as the plain step."""
    from hira_b200 import HiraDecodeStep
    h, hq, n, d, bf = 2, 8, 4096, 128, 16
    keys, vals = _keys(h, n, d, 211, torch.bfloat16), _keys(h, n, d, 212, torch.bfloat16)
    a = CUDAIndexer(levels, 1, bf, max_context=n + 64, reserve_worst_case=True, seed=9).build(keys, vals)
    b = CUDAIndexer(levels, 1, bf, max_context=n + 64, reserve_worst_case=True, seed=9).build(keys, vals)
    plain, graphed = HiraDecodeStep(a, hq), HiraDecodeStep(b, hq, graph_steps=5)
    steps = 12
    more_k = _keys(h, steps, d, 213, torch.bfloat16)[0].transpose(0, 1).contiguous().cpu()   # (steps, h, d)
    more_v = _keys(h, steps, d, 214, torch.bfloat16)[0].transpose(0, 1).contiguous().cpu()
    tau = torch.full((hq,), 0.12, device="cuda")
    bufs = [dict(q=torch.empty((hq, d)).pin_memory(), k=torch.empty((h, d), dtype=torch.bfloat16).pin_memory(),
                 v=torch.empty((h, d), dtype=torch.bfloat16).pin_memory(), o=torch.empty((hq, d)).pin_memory())
            for _ in range(2)]
    out_plain = torch.empty((hq, d), dtype=torch.float32).pin_memory()
    g = torch.Generator().manual_seed(6)
    for i in range(steps):
        s = bufs[i % 2]
        s["q"].copy_(torch.randn((hq, d), generator=g))
        s["k"].copy_(more_k[i])
        s["v"].copy_(more_v[i])
        plain(s["q"], out_plain, threshold=tau, k_host=s["k"], v_host=s["v"])
        plain.synchronize()
        graphed(s["q"], s["o"], threshold=tau, k_host=s["k"], v_host=s["v"])
        graphed.synchronize()
        assert torch.allclose(out_plain, s["o"], rtol=1e-5, atol=1e-6), i
    assert len(graphed._graphs) <= 2
    a.check_status(), b.check_status()
    for name in a.state.ARRAYS:
        x, y = getattr(a.state, name), getattr(b.state, name)
        assert x is None and y is None or torch.equal(x, y), name


@pytest.mark.parametrize("levels,fused", [(3, False), (3, True), (2, False)])
def test_decode_step_from_host_buffers_equals_the_separate_calls(levels, fused):
    """HiraDecodeStep (one hira_decode_step call per token: host query in, host output out, the
    append beside it on a second stream) against hira_decode_attention + update with device
    tensors: same attention output, same index, step after step; also with the threshold found
    on the device inside the step."""
    from hira_b200 import HiraDecodeStep
    from hira_b200.cache import CacheOutput
    h, hq, n, d, bf = 2, 8, 4096, 128, 16
    keys, vals = _keys(h, n, d, 111, torch.bfloat16), _keys(h, n, d, 112, torch.bfloat16)
    a = CUDAIndexer(levels, 1, bf, max_context=n + 64, reserve_worst_case=True, seed=9).build(keys, vals)
    b = CUDAIndexer(levels, 1, bf, max_context=n + 64, reserve_worst_case=True, seed=9).build(keys, vals)
    steps = 12
    more_k = _keys(h, steps, d, 113, torch.bfloat16)[0].transpose(0, 1).contiguous().cpu().pin_memory()   # (steps, h, d)
    more_v = _keys(h, steps, d, 114, torch.bfloat16)[0].transpose(0, 1).contiguous().cpu().pin_memory()
    tau = torch.full((hq,), 0.12, device="cuda")
    empty = torch.empty((1, h, 0, d), dtype=torch.bfloat16, device="cuda")
    ca = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=a,
                     searcher=CUDASearcher(bf))
    step = HiraDecodeStep(b, hq, fused_scan=fused)
    out_host = torch.empty((hq, d), dtype=torch.float32).pin_memory()
    g = torch.Generator().manual_seed(5)
    for i in range(steps):
        q = torch.randn((hq, d), generator=g).pin_memory()
        oa = hira_decode_attention(q.cuda().view(1, hq, 1, d), ca, threshold=tau)
        a.update(more_k[i].cuda().view(1, h, 1, d), more_v[i].cuda().view(1, h, 1, d))
        step(q, out_host, threshold=tau, k_host=more_k[i], v_host=more_v[i])
        step.synchronize()
        assert torch.allclose(oa.view(hq, d).cpu(), out_host, rtol=1e-5, atol=1e-6), i
    a.check_status(), b.check_status()
    for name in a.state.ARRAYS:
        x, y = getattr(a.state, name), getattr(b.state, name)
        assert x is None and y is None or torch.equal(x, y), name
    # threshold found inside the step: equals sample_mean_topk on the same samples + the given-tau step
    from hira_b200.attention.hira_attention import _samples_for
    q = torch.randn((hq, d), generator=g).pin_memory()
    q_hat = (q / q.norm(dim=-1, keepdim=True)).cuda()
    tau2 = sample_mean_topk(_samples_for(b, 1000), q_hat, 16)
    step(q, out_host)
    step.synchronize()
    got = out_host.clone()
    step(q, out_host, threshold=tau2)
    step.synchronize()
    assert torch.equal(got, out_host)
