"""hira_attention: range-searching sparse attention for decode, in the shape of a
Hugging Face attention function (see AttentionInterface in transformers.modeling_utils;
the reference ships only that pointer, attention/hira_attention.py:1-3, and the hook in
examples/patch_llama.py:59-74).

`key` is what `HiraCache.update` returned: a `CacheOutput`.  Prefill (`prefill_keys`
present) attends densely over the prompt; a decode step
  1. normalises the query (the tree bound assumes a unit query, searcher/cpu.py:61-63)
     and folds its norm and the softmax scale into the per-head `scaling`,
  2. finds a threshold on the device (THRESHOLD_METHODS) unless one is given,
  3. searches the index for the keys with `q.k >= threshold`,
  4. runs softmax over those keys plus the not-yet-indexed queue and multiplies by the
     slot-aligned values.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib as L
from .. import index_state as S
from ..cache.threshold_finder import THRESHOLD_METHODS
from ..searcher import CUDASearcher


def _samples_for(indexer, sample_size: int) -> torch.Tensor:
    """(H_kv, S, D) key rows drawn once per built index from its filled slots."""
    st = indexer.state
    cached = getattr(indexer, "_tau_samples", None)
    if cached is not None and cached[0] is st and cached[1].shape[1] == min(sample_size, 4096):
        return cached[1]
    s = min(sample_size, 4096)
    g = torch.Generator(device=st.device)
    g.manual_seed(getattr(indexer, "seed", 0) + 17)
    filled = st.slot2token >= 0                                   # (H, capC)
    # random filled slots per head: top-s of random scores masked to filled slots
    r = torch.rand(filled.shape, generator=g, device=st.device).masked_fill_(~filled, -1.0)
    n_filled = int(filled.sum(dim=1).min().item())
    s = max(1, min(s, n_filled))
    slots = r.topk(s, dim=1).indices                              # (H, s)
    rows = st.children.gather(1, slots.unsqueeze(-1).expand(-1, -1, st.dim)).contiguous()
    indexer._tau_samples = (st, rows)
    return rows


def _attn_searcher(searcher, gate: str) -> CUDASearcher:
    s = getattr(searcher, "_attn_searcher", None)
    if s is None:
        s = CUDASearcher(getattr(searcher, "block_c", None), gate=gate, leaf=gate)
        try:
            searcher._attn_searcher = s
        except AttributeError:
            pass
    return s


def hira_decode_attention(query: torch.Tensor, cache_output, *, scaling: Optional[float] = None,
                          threshold: Optional[torch.Tensor] = None, threshold_method: str = "sample_mean_topk",
                          sample_size: int = 1000, topk: int = 16, gate: str = "ge",
                          q_head_to_kv: Optional[torch.Tensor] = None, return_compact: bool = False,
                          append_key: Optional[torch.Tensor] = None):
    """query (B, H_q, 1, D) -> (B, H_q, 1, V) float32.  `threshold` (B*H_q,) is on the scale of
    `q_hat . k` with `q_hat = q / ||q||`.

    `append_key` (B, H_kv, 1, D): the key the caller appends right after this call with
    `indexer.update(append_key, value, scanned=True)`.  The search then scores the parent rows it
    reads against that key as well, and the update needs no parent scan of its own."""
    indexer, searcher = cache_output.indexer, cache_output.searcher
    st: S.IndexState = indexer.state
    b, hq, lq, d = query.shape
    if lq != 1:
        raise NotImplementedError("hira_decode_attention handles one query token per step")
    q = query.reshape(b * hq, d)
    if q.device != st.device or q.dtype not in (torch.float32, torch.bfloat16):
        q = q.to(device=st.device, dtype=torch.float32)
    sm_scale = float(scaling) if scaling is not None else d ** -0.5
    bufs = getattr(searcher, "_decode_bufs", None)
    if bufs is None or bufs[0].shape != (b * hq, d) or bufs[0].device != st.device:
        bufs = (torch.empty((b * hq, d), dtype=torch.float32, device=st.device),
                torch.empty((b * hq,), dtype=torch.float32, device=st.device))
        try:
            searcher._decode_bufs = bufs
        except AttributeError:
            pass
    srch = _attn_searcher(searcher, gate)
    n_q = b * hq
    q2kv, max_group = srch._coerce_q2kv(q_head_to_kv, n_q, st.n_heads, st.device)
    if hasattr(indexer, "wait_pending_update"):
        indexer.wait_pending_update()                            # an update still running on a side stream
    st.active_parents = getattr(indexer, "active_parents", 0)   # empty capacity is not visited
    compact = srch._compact
    if compact is None or compact.idx.device != st.device or tuple(compact.idx.shape) != (n_q, st.cap_children):
        compact = srch._compact = S.alloc_compact(st, n_q)
    qk = cache_output.queued_keys
    queued_k = queued_v = None
    if qk is not None and qk.shape[-2] > 0:
        queued_k = qk.reshape(-1, qk.shape[-2], qk.shape[-1]).to(st.dtype).contiguous()
        qv = cache_output.queued_values
        queued_v = qv.reshape(-1, qv.shape[-2], qv.shape[-1]).to(st.vdtype).contiguous()
    n_splits = S.attn_splits(st, n_q, compact.tile_parents)
    ws = getattr(srch, "_attn_ws", None)
    need = n_q * n_splits * (st.vdim + 2)
    if ws is None or ws.numel() < need or ws.device != st.device:
        ws = srch._attn_ws = torch.empty((need,), dtype=torch.float32, device=st.device)
    out = torch.empty((n_q, st.vdim), dtype=torch.float32, device=st.device)
    q = q.contiguous()
    scan_key = scan_out = None
    if append_key is not None:
        if q2kv is not None:
            raise ValueError("append_key needs the default query-head grouping")
        scan_key, scan_out = indexer.begin_scanned_update(append_key)
    if threshold is not None and threshold_method != "none":
        # the usual decode step: the threshold is known, one library call does the rest
        tau = threshold
        if tau.shape != (n_q,):
            raise ValueError(f"threshold must have shape ({n_q},), got {tuple(tau.shape)}")
        if tau.device != st.device or tau.dtype != torch.float32 or not tau.is_contiguous():
            tau = tau.to(device=st.device, dtype=torch.float32).contiguous()
        S.decode_attention(st, q, sm_scale, tau, compact, bufs[0], bufs[1], q2kv=q2kv, max_group=max_group,
                           flags=srch.flags, queued_k=queued_k, queued_v=queued_v, n_splits=n_splits, workspace=ws,
                           out=out, scan_key=scan_key, scan_out=scan_out,
                           searched_event=indexer.searched_event() if hasattr(indexer, "searched_event") else None)
    else:
        q_hat, logit_scale = S.prepare_query(q, sm_scale, bufs[0], bufs[1])
        if threshold is None and threshold_method == "none":
            threshold = torch.full((n_q,), float("-inf"), device=st.device)      # keep every key: dense-equivalent
        if threshold is None:
            samples = _samples_for(indexer, sample_size)
            fn = THRESHOLD_METHODS[threshold_method]
            if threshold_method == "sample_max":
                threshold = fn(samples, q_hat, q_head_to_kv)
            else:
                threshold = fn(samples, q_hat, min(topk, samples.shape[1]), q_head_to_kv)
        tau = torch.as_tensor(threshold).to(device=st.device, dtype=torch.float32).contiguous()
        if tau.shape != (n_q,):
            raise ValueError(f"threshold must have shape ({n_q},), got {tuple(tau.shape)}")
        S.search(st, q_hat, tau, scaling=logit_scale, q2kv=q2kv, max_group=max_group, flags=srch.flags,
                 compact=compact, scan_key=scan_key, scan_out=scan_out)
        if hasattr(indexer, "searched_event"):
            indexer.searched_event()
            indexer._searched.record(torch.cuda.current_stream(st.device))
        S.sparse_attn(st, q_hat, logit_scale, compact, q2kv=q2kv, queued_k=queued_k, queued_v=queued_v,
                      n_splits=n_splits, workspace=ws, out=out)
    out = out.reshape(b, hq, 1, st.vdim)
    return (out, compact) if return_compact else out


def hira_attention(module, query: torch.Tensor, key, value=None, attention_mask: Optional[torch.Tensor] = None,
                   dropout: float = 0.0, scaling: Optional[float] = None, **kwargs):
    """Hugging Face attention-function signature.  Returns (attn_output (B, L_q, H_q, V), None)."""
    from ..cache.hira_cache import CacheOutput
    if not isinstance(key, CacheOutput):
        raise TypeError("hira_attention expects the CacheOutput returned by HiraCache.update as `key`")
    if key.prefill_keys is not None:
        k, v = key.prefill_keys, key.prefill_values
        is_causal = attention_mask is None and query.shape[2] > 1
        out = torch.nn.functional.scaled_dot_product_attention(
            query, k, v, attn_mask=attention_mask, dropout_p=0.0, is_causal=is_causal, scale=scaling,
            enable_gqa=query.shape[1] != k.shape[1])
        return out.transpose(1, 2).contiguous(), None
    cfg = kwargs.get("hira_config")
    opts = {}
    if cfg is not None:
        opts = dict(threshold_method=cfg.threshold_method, sample_size=cfg.sample_size,
                    topk=getattr(cfg, "topk", 16), gate=getattr(cfg, "gate", "ge"))
    out = hira_decode_attention(query, key, scaling=scaling, threshold=kwargs.get("threshold"), **opts)
    return out.to(query.dtype).transpose(1, 2).contiguous(), None


def make_hira_attention(hira_config=None, threshold: Optional[torch.Tensor] = None):
    """An attention function bound to a HiraConfig, for `AttentionInterface.register`."""
    def fn(module, query, key, value=None, attention_mask=None, dropout: float = 0.0, scaling=None, **kwargs):
        kwargs.setdefault("hira_config", hira_config)
        if threshold is not None:
            kwargs.setdefault("threshold", threshold)
        return hira_attention(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, **kwargs)
    return fn


def register_hira_attention(hira_config=None, name: str = "hira"):
    """Registers `name` as an attention implementation of Hugging Face models, so that
    `model.config._attn_implementation = name` (or `attn_implementation=name` at load time)
    routes every attention layer through the index when `past_key_values` is a HiraCache
    (the patching the reference sketches in examples/patch_llama.py:22-100).  Masks are built
    as for SDPA; decode steps ignore them (one sequence, no padding)."""
    from transformers import AttentionInterface
    AttentionInterface.register(name, make_hira_attention(hira_config))
    try:
        from transformers.masking_utils import AttentionMaskInterface, sdpa_mask
        AttentionMaskInterface.register(name, sdpa_mask)
    except Exception:  # older transformers: no separate mask registry
        pass
    return name


class HiraDecodeStep:
    """One library call per decode step and layer, host buffers in and out (`hira_decode_step`):
    the query is copied to the device, the threshold taken or found there, the index searched,
    the selected keys attended, the output copied back, and the token's new key / value appended
    beside all that on a second stream.  The Python classes above do the same in several calls
    with device tensors; this is the path for a serving loop that holds its activations in
    pinned host memory and wants no interpreter work between the launches.

        step = HiraDecodeStep(indexer, n_qheads=B * H_q, threshold_method="sample_mean_topk")
        step(q_host, out_host, k_host=k, v_host=v)          # (B*H_q, D), (B*H_q, V), (B*H_kv, D) ...
        step.synchronize()                                   # out_host is ready, the key is indexed

    The indexer must have been built with room for the appends (`max_context`): the step never
    reallocates.

    `graph_steps=G` (> 0) replays the step from CUDA graphs: the first call with a given set of host
    buffers (and threshold tensor) records the library call into a graph, later calls with the same
    buffers replay it -- the host refills its buffers in place, nothing else is launched.  Grids are
    frozen in a graph, so a recording covers the slots the index can reach within the next G appends
    (a few empty tiles are visited meanwhile) and is made anew after G appends.  Worth it when the step
    is short (small batch per GPU), where the launches rather than the kernels bound it."""

    def __init__(self, indexer, n_qheads: int, *, q_dtype: torch.dtype = torch.float32, gate: str = "ge",
                 scaling: Optional[float] = None, threshold_method: str = "sample_mean_topk", sample_size: int = 1000,
                 topk: int = 16, fused_scan: bool = False, side_stream: Optional["torch.cuda.Stream"] = None,
                 graph_steps: int = 0):
        st: S.IndexState = indexer.state
        if st is None:
            raise ValueError("Indexer is not built")
        self.indexer = indexer
        flags = (L.HIRA_GATE_GE | L.HIRA_LEAF_GE) if gate == "ge" else (L.HIRA_GATE_GT | L.HIRA_LEAF_GT)
        methods = {"sample_max": L.HIRA_TAU_SAMPLE_MAX, "sample_mean_topk": L.HIRA_TAU_SAMPLE_MEAN_TOPK,
                   "sample_kth": L.HIRA_TAU_SAMPLE_KTH}
        samples = _samples_for(indexer, sample_size) if threshold_method in methods else None
        self._step = S.DecodeStep(st, n_qheads, q_dtype, flags=flags, fused_scan=fused_scan, tau_samples=samples,
                                  tau_method=methods.get(threshold_method, L.HIRA_TAU_SAMPLE_MEAN_TOPK),
                                  tau_k=1 if samples is None else min(topk, samples.shape[1]))
        self.sm_scale = float(scaling) if scaling is not None else st.dim ** -0.5
        self.side = side_stream if side_stream is not None else torch.cuda.Stream(device=st.device)
        self.graph_steps = int(graph_steps)
        self._graphs = {}            # addresses of the caller's buffers -> recorded step
        self._graph_left = 0         # appends the recorded grids still cover
        self._graph_active = 0       # the bound on the slots in use they were recorded with

    def _run_graphed(self, q_host, out_host, threshold, k_host, v_host):
        ix, st = self.indexer, self.indexer.state
        if self._graph_left <= 0 or ix.active_parents > self._graph_active:
            # record anew, for the slots the index can reach within the next graph_steps appends
            self._graphs.clear()
            saved = ix._parents_bound, ix._gp_bound
            ix._parents_bound += self.graph_steps
            ix._gp_bound += self.graph_steps
            self._graph_active = ix.active_parents
            ix._parents_bound, ix._gp_bound = saved
            self._graph_left = self.graph_steps
        key = (q_host.data_ptr(), out_host.data_ptr(), 0 if threshold is None else threshold.data_ptr(),
               0 if k_host is None else k_host.data_ptr(), 0 if v_host is None else v_host.data_ptr())
        g = self._graphs.get(key)
        if g is None:
            st.active_parents = self._graph_active
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step.run(q_host, out_host, sm_scale=self.sm_scale, tau=threshold, k_host=k_host, v_host=v_host,
                               side_stream=self.side)
            self._graphs[key] = g
        g.replay()
        if k_host is not None:
            self._graph_left -= 1

    def __call__(self, q_host: torch.Tensor, out_host: torch.Tensor, *, threshold: Optional[torch.Tensor] = None,
                 k_host: Optional[torch.Tensor] = None, v_host: Optional[torch.Tensor] = None):
        ix = self.indexer
        st = ix.state
        if st is not self._step.st:
            raise RuntimeError("the index was reallocated since this step was created: build it with max_context")
        ix.wait_pending_update()
        if k_host is not None:
            need_g, need_p = ix._gp_bound + 1, ix._parents_bound + 1
            if (st.depth == 3 and need_g > st.cap_gp) or (st.depth == 2 and need_p > st.cap_parents):
                ix._tighten_bounds()
                raise RuntimeError("no pre-allocated room left for this append: raise max_context (or rebuild)")
            ix._parents_bound += 1          # the append may open a new parent and a new grandparent
            ix._gp_bound += 1
        st.active_parents = ix.active_parents
        if self.graph_steps > 0:
            self._run_graphed(q_host, out_host, threshold, k_host, v_host)
        else:
            self._step.run(q_host, out_host, sm_scale=self.sm_scale, tau=threshold, k_host=k_host, v_host=v_host,
                           side_stream=self.side)
        if k_host is not None:
            ix._n_keys += 1
            ix._appended += 1
            if ix._snapshot is not None or ix._appended % ix.BOUND_REFRESH_EVERY == 0:
                ix._tighten_bounds()

    def synchronize(self):
        torch.cuda.current_stream(self.indexer.state.device).synchronize()
