"""Device-resident index arrays and thin typed wrappers over the C ABI.

`IndexState` owns the torch tensors behind one `hira_index_t` (torch only supplies
memory and the stream); the functions below forward to libhira_b200.so.  Names of
the arrays follow the reference's CUDAIndexer attributes (indexer/cuda.py:40-54).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib as L


class IndexState:
    def __init__(self, *, n_heads: int, dim: int, vdim: int, bf: int, depth: int, cap_parents: int,
                 dtype: torch.dtype, vdtype: Optional[torch.dtype], device, with_values: bool = True,
                 int8_copy: Optional[bool] = None):
        if depth not in (2, 3):
            raise ValueError(f"Unsupported depth {depth}")
        self.n_heads, self.dim, self.vdim, self.bf, self.depth = n_heads, dim, vdim if with_values else 0, bf, depth
        self.dtype, self.vdtype = dtype, (vdtype if with_values else dtype)
        self.device = torch.device(device)
        if depth == 3:
            self.cap_gp = max(1, -(-cap_parents // bf))
            self.cap_parents = self.cap_gp * bf
        else:
            self.cap_gp = 0
            self.cap_parents = max(1, cap_parents)
        capC = self.cap_parents * bf
        dev = self.device
        z = torch.zeros
        self.children = z((n_heads, capC, dim), dtype=dtype, device=dev)
        self.values = z((n_heads, capC, self.vdim), dtype=self.vdtype, device=dev) if with_values else None
        self.slot2token = torch.full((n_heads, capC), -1, dtype=torch.int32, device=dev)
        self.parents = z((n_heads, self.cap_parents, dim), dtype=dtype, device=dev)
        self.parent_radii = z((n_heads, self.cap_parents), dtype=torch.float32, device=dev)
        self.parent_sqnorm = z((n_heads, self.cap_parents), dtype=torch.float32, device=dev)
        self.child_counts = z((n_heads, self.cap_parents), dtype=torch.int32, device=dev)
        if depth == 3:
            self.grand_parents = z((n_heads, self.cap_gp, dim), dtype=dtype, device=dev)
            self.gp_radii = z((n_heads, self.cap_gp), dtype=torch.float32, device=dev)
            self.gp_sqnorm = z((n_heads, self.cap_gp), dtype=torch.float32, device=dev)
            self.gp_counts = z((n_heads, self.cap_gp), dtype=torch.int32, device=dev)
        else:
            self.grand_parents = self.gp_radii = self.gp_sqnorm = self.gp_counts = None
        self.used = z((n_heads, 4), dtype=torch.int32, device=dev)
        # int8 side copy of the children for the tensor-core pre-filter of the search (D = 128):
        # +52 % on the bf16 keys' memory (128 B + 4 B per slot), about half the search's traffic
        if int8_copy is None:
            int8_copy = dim == 128 and self.device.type == "cuda"
        if int8_copy and dim != 128:
            raise ValueError("the int8 side copy needs dim == 128")
        self.int8_copy = bool(int8_copy)
        if self.int8_copy:
            self.children_q8 = z((n_heads, capC, 128), dtype=torch.int8, device=dev)
            self.children_q8_meta = z((n_heads, capC), dtype=torch.int32, device=dev)   # (step, error bound) as two fp16
            self.q8_chan_scale = torch.ones((n_heads, L.Q8_CHAN), dtype=torch.float32, device=dev)
            self.q8_query_scratch = z((n_heads, L.Q8_QUERY_BYTES), dtype=torch.uint8, device=dev)
        else:
            self.children_q8 = self.children_q8_meta = self.q8_chan_scale = self.q8_query_scratch = None
        self.status = z((1,), dtype=torch.int32, device=dev)
        self._struct = None
        self._active_parents = 0
        self.refresh_struct()

    ARRAYS = ("children", "values", "slot2token", "parents", "parent_radii", "parent_sqnorm", "child_counts",
              "grand_parents", "gp_radii", "gp_sqnorm", "gp_counts", "used")
    # derived from `children` (and scratch): not part of a checkpoint
    Q8_ARRAYS = ("children_q8", "children_q8_meta", "q8_chan_scale", "q8_query_scratch")

    @property
    def cap_children(self) -> int:
        return self.cap_parents * self.bf

    def refresh_struct(self):
        s = L.HiraIndexStruct()
        s.dtype = L.dtype_code(self.dtype)
        s.vdtype = L.dtype_code(self.vdtype)
        s.depth, s.bf, s.dim, s.vdim = self.depth, self.bf, self.dim, self.vdim
        s.n_heads, s.cap_parents, s.cap_gp = self.n_heads, self.cap_parents, self.cap_gp
        s.active_parents = self._active_parents
        for name in self.ARRAYS + self.Q8_ARRAYS:
            setattr(s, name, L.ptr(getattr(self, name)))
        self._struct = s
        return s

    @property
    def active_parents(self) -> int:
        """Host's upper bound on the parent slots in use; 0 = unknown (all of cap_parents).
        Search, sparse attention and kth_score skip the tiles beyond it."""
        return self._active_parents

    @active_parents.setter
    def active_parents(self, n: int):
        n = int(n)
        if n < 0 or n >= self.cap_parents:
            n = 0
        self._active_parents = n
        self._struct.active_parents = n

    @property
    def struct(self):
        return C.byref(self._struct)

    def state_dict(self) -> dict:
        d = {name: getattr(self, name) for name in self.ARRAYS if getattr(self, name) is not None}
        d["meta"] = dict(n_heads=self.n_heads, dim=self.dim, vdim=self.vdim, bf=self.bf, depth=self.depth,
                         cap_parents=self.cap_parents, dtype=str(self.dtype), vdtype=str(self.vdtype))
        return d

    def load_arrays(self, arrays: dict):
        """Copies host/device arrays with matching shapes into the index (checkpoint import,
        moving an index between the oracle and the device)."""
        for name in self.ARRAYS:
            dst = getattr(self, name)
            if dst is None or name not in arrays or arrays[name] is None:
                continue
            src = arrays[name]
            if not torch.is_tensor(src):
                src = torch.as_tensor(src)
            if src.dtype == torch.uint16 or (dst.dtype == torch.bfloat16 and src.dtype == torch.int16):
                src = src.view(torch.bfloat16)
            dst.copy_(src.reshape(dst.shape).to(dst.dtype))
        self.refresh_int8_copy()

    def enable_int8_copy(self, on: bool = True):
        """Switches the search between the int8 pre-filter (when the index carries the side copy)
        and the plain streaming kernel; results are identical either way."""
        for name in self.Q8_ARRAYS:
            setattr(self._struct, name, L.ptr(getattr(self, name)) if (on and self.int8_copy) else None)

    def refresh_int8_copy(self):
        """Recomputes the int8 side copy from the children as stored now."""
        if self.int8_copy and self.device.type == "cuda":
            L.check(L.load().hira_q8_refresh(self.struct, L.current_stream(self.device)), "hira_q8_refresh")

    def grown(self, new_cap_parents: int) -> "IndexState":
        """A copy with more parent slots (and grandparent slots); existing slots keep their positions."""
        new = IndexState(n_heads=self.n_heads, dim=self.dim, vdim=self.vdim, bf=self.bf, depth=self.depth,
                         cap_parents=new_cap_parents, dtype=self.dtype, vdtype=self.vdtype, device=self.device,
                         with_values=self.values is not None, int8_copy=self.int8_copy)
        for name in self.ARRAYS + self.Q8_ARRAYS:
            src = getattr(self, name)
            if src is None or name == "used":
                continue
            if name in ("q8_chan_scale", "q8_query_scratch"):
                getattr(new, name).copy_(src)
                continue
            getattr(new, name)[:, : src.shape[1]].copy_(src)
        new.used.copy_(self.used)
        new.status.copy_(self.status)
        return new


@dataclass
class CompactResult:
    """Compacted search output (see hira_search in include/hira_b200.h)."""
    idx: torch.Tensor      # (H_q, cap_children) int32, slot ids, valid in the first count entries of each tile segment
    score: torch.Tensor    # (H_q, cap_children) float32
    count: torch.Tensor    # (H_q, n_tiles) int32
    tile_parents: int
    tile_rows: int
    n_tiles_active: Optional[int] = None   # tiles the last search wrote (None: all)

    def to_lists(self):
        """Per query head: (slots, scores) as 1-D CPU tensors, ascending slot order."""
        idx, score, count = self.idx.cpu(), self.score.cpu(), self.count.cpu()
        out = []
        for qh in range(idx.shape[0]):
            sl, sc = [], []
            for t in range(count.shape[1] if self.n_tiles_active is None else self.n_tiles_active):
                c = int(count[qh, t])
                if c:
                    b = t * self.tile_rows
                    sl.append(idx[qh, b:b + c])
                    sc.append(score[qh, b:b + c])
            out.append((torch.cat(sl) if sl else torch.empty(0, dtype=torch.int32),
                        torch.cat(sc) if sc else torch.empty(0)))
        return out


def tile_parents(st: IndexState) -> int:
    tp = getattr(st, "_tile_parents", None)
    if tp is None:   # depends on bf, depth and the capacity only: fixed for the life of the state
        tp = st._tile_parents = int(L.load().hira_search_tile_parents(st.struct))
    return tp


def n_tiles(st: IndexState, tp: Optional[int] = None) -> int:
    tp = tp or tile_parents(st)
    return -(-st.cap_parents // tp)


def _f32(t: Optional[torch.Tensor], dev) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.to(device=dev, dtype=torch.float32).contiguous()


def search(st: IndexState, q: torch.Tensor, tau: torch.Tensor, *, scaling=None, qnorm=None, q2kv=None,
           max_group: int = 0, flags: int = 0, out_dense=None, compact: Optional[CompactResult] = None,
           want_compact: bool = False, stats=None, tp: Optional[int] = None, scan_key=None, scan_out=None):
    """q (H_q, D) fp32, tau (H_q,) fp32 on the index device.  Returns (out_dense, CompactResult|None).
    With `scan_key` (n_heads, D) in the index dtype and `scan_out` (new_scan_slots), the parents are
    also scored against that key for the `append_scanned` that follows."""
    lib = L.load()
    hq = q.shape[0]
    tp = tp or tile_parents(st)
    if want_compact and compact is None:
        compact = alloc_compact(st, hq, tp)
    if scan_out is not None:
        if q2kv is not None:
            raise ValueError("the fused parent scan needs the default head grouping")
        assert scan_key.dtype == st.dtype and scan_key.shape[0] == st.n_heads and scan_key.stride(-1) == 1
        rc = lib.hira_search_scan(st.struct, L.ptr(q), L.ptr(tau), L.ptr(scaling), L.ptr(qnorm), hq, flags, tp,
                                  L.ptr(out_dense), L.ptr(compact.idx) if compact else None,
                                  L.ptr(compact.score) if compact else None, L.ptr(compact.count) if compact else None,
                                  L.ptr(stats), L.ptr(scan_key), scan_key.stride(0), L.ptr(scan_out),
                                  L.current_stream(st.device))
        L.check(rc, "hira_search_scan")
        if compact is not None:
            compact.n_tiles_active = None if (st.active_parents == 0 or out_dense is not None) \
                else -(-st.active_parents // tp)
        return out_dense, compact
    rc = lib.hira_search(st.struct, L.ptr(q), L.ptr(tau), L.ptr(scaling), L.ptr(qnorm), L.ptr(q2kv), hq,
                         max_group, flags, tp, L.ptr(out_dense),
                         L.ptr(compact.idx) if compact else None, L.ptr(compact.score) if compact else None,
                         L.ptr(compact.count) if compact else None, L.ptr(stats), L.current_stream(st.device))
    L.check(rc, "hira_search")
    if compact is not None:
        compact.n_tiles_active = None if (st.active_parents == 0 or out_dense is not None) \
            else -(-st.active_parents // tp)
    return out_dense, compact


def q8_fallback_count(device=None) -> int:
    """CTAs of the int8 pre-filter search on `device` (default: current) that took their exact fallback
    because a bounded wait ran out, since the library was loaded (hira_q8_fallback_count; synchronises)."""
    import ctypes as C
    v = C.c_uint32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        L.check(L.load().hira_q8_fallback_count(C.byref(v)), "hira_q8_fallback_count")
    return int(v.value)


def new_stats(hq: int, device) -> torch.Tensor:
    """Zeroed traffic counters for `search(..., stats=)`: (H_q, HIRA_SEARCH_STATS) int32."""
    return torch.zeros((hq, L.SEARCH_STATS), dtype=torch.int32, device=device)


def alloc_compact(st: IndexState, hq: int, tp: Optional[int] = None) -> CompactResult:
    tp = tp or tile_parents(st)
    dev = st.device
    return CompactResult(
        idx=torch.empty((hq, st.cap_children), dtype=torch.int32, device=dev),
        score=torch.empty((hq, st.cap_children), dtype=torch.float32, device=dev),
        count=torch.zeros((hq, n_tiles(st, tp)), dtype=torch.int32, device=dev),
        tile_parents=tp, tile_rows=tp * st.bf)


def attn_splits(st: IndexState, hq: int, tp: Optional[int] = None) -> int:
    tp = tp or tile_parents(st)
    tiles = n_tiles(st, tp) if st.active_parents == 0 else -(-st.active_parents // tp)
    return int(L.load().hira_attn_default_splits(hq, tiles))


def sparse_attn(st: IndexState, q, scaling, compact: CompactResult, *, q2kv=None, queued_k=None, queued_v=None,
                n_splits: Optional[int] = None, workspace=None, out=None, out_ml=None):
    """`out` / `out_ml` may be strided views (rows of a packed (H_q, 2 + V) message): only the
    last dimension has to be contiguous."""
    lib = L.load()
    hq = q.shape[0]
    n_splits = n_splits or attn_splits(st, hq, compact.tile_parents)
    dev = st.device
    if workspace is None:
        workspace = torch.empty((hq * n_splits * (st.vdim + 2),), dtype=torch.float32, device=dev)
    if out is None:
        out = torch.empty((hq, st.vdim), dtype=torch.float32, device=dev)
    n_queued, qstride = 0, 0
    if queued_k is not None and queued_k.shape[-2] > 0:
        assert queued_k.is_contiguous() and queued_v.is_contiguous()
        assert queued_k.dtype == st.dtype and queued_v.dtype == st.vdtype
        n_queued = queued_k.shape[-2]
        qstride = n_queued * st.dim
        if st.vdim != st.dim:
            raise ValueError("queued keys/values with vdim != dim are not supported")
    rc = lib.hira_sparse_attn(st.struct, L.ptr(q), L.ptr(scaling), L.ptr(q2kv), hq, compact.tile_parents,
                              L.ptr(compact.idx), L.ptr(compact.score), L.ptr(compact.count),
                              L.ptr(queued_k) if n_queued else None, L.ptr(queued_v) if n_queued else None,
                              n_queued, qstride, n_splits, L.ptr(workspace), L.ptr(out), L.ptr(out_ml),
                              out.stride(0), out_ml.stride(0) if out_ml is not None else 0, L.current_stream(dev))
    L.check(rc, "hira_sparse_attn")
    return out


def merge_partials(part_o, part_ml, out=None, out_ml=None):
    """part_o (n_parts, H_q, V), part_ml (n_parts, H_q, 2): any strides with a contiguous last
    dimension (e.g. two views of one gathered (n_parts, H_q, 2 + V) buffer)."""
    lib = L.load()
    n_parts, hq, vdim = part_o.shape
    assert part_o.stride(2) == 1 and part_ml.stride(2) == 1
    if out is None:
        out = torch.empty((hq, vdim), dtype=torch.float32, device=part_o.device)
    rc = lib.hira_merge_partials(L.ptr(part_o), L.ptr(part_ml), n_parts, hq, vdim, part_o.stride(0), part_o.stride(1),
                                 part_ml.stride(0), part_ml.stride(1), L.ptr(out), L.ptr(out_ml),
                                 L.current_stream(part_o.device))
    L.check(rc, "hira_merge_partials")
    return out


def append(st: IndexState, new_k: torch.Tensor, new_v: Optional[torch.Tensor], token_base: int = -1,
           use_workspace: bool = True):
    """new_k (n_heads, M, D), new_v (n_heads, M, V) contiguous, index dtypes."""
    lib = L.load()
    assert new_k.is_contiguous() and new_k.dtype == st.dtype
    m = new_k.shape[1]
    if new_v is not None:
        assert new_v.is_contiguous() and new_v.dtype == st.vdtype
    ws, nbytes = None, 0
    if use_workspace:
        nbytes = int(lib.hira_append_workspace_bytes(st.struct, m))
        if nbytes:
            ws = getattr(st, "_append_ws", None)
            if ws is None or ws.numel() < nbytes:
                ws = st._append_ws = torch.empty((nbytes,), dtype=torch.uint8, device=st.device)
    rc = lib.hira_append(st.struct, L.ptr(new_k), L.ptr(new_v), m, m * st.dim,
                         m * st.vdim if new_v is not None else 0, token_base, L.ptr(st.status),
                         L.ptr(ws), nbytes, L.current_stream(st.device))
    L.check(rc, "hira_append")


def new_scan_slots(st: IndexState) -> torch.Tensor:
    """The (n_heads,) buffer `search(..., scan_out=)` fills and `append_scanned` consumes."""
    return torch.full((st.n_heads,), -1, dtype=torch.int64, device=st.device)


def append_scanned(st: IndexState, new_k: torch.Tensor, new_v: Optional[torch.Tensor], scan: torch.Tensor,
                   token_base: int = -1):
    """One key per head, new_k (n_heads, 1, D) / new_v (n_heads, 1, V) in the index dtypes, whose
    nearest parent the preceding `search(..., scan_key=new_k[:, 0], scan_out=scan)` found."""
    lib = L.load()
    assert new_k.dtype == st.dtype and new_k.shape[1] == 1 and new_k.stride(-1) == 1
    if new_v is not None:
        assert new_v.dtype == st.vdtype and new_v.stride(-1) == 1
    rc = lib.hira_append_scanned(st.struct, L.ptr(new_k), L.ptr(new_v), new_k.stride(0),
                                 new_v.stride(0) if new_v is not None else 0, token_base, L.ptr(st.status),
                                 L.ptr(scan), L.current_stream(st.device))
    L.check(rc, "hira_append_scanned")


def threshold(samples: torch.Tensor, q: torch.Tensor, method: int, k: int = 1, q2kv=None, out=None):
    """samples (H_kv, S, D) contiguous fp32/bf16, q (H_q, D) fp32 -> tau (H_q,)."""
    lib = L.load()
    hkv, s, d = samples.shape
    hq = q.shape[0]
    if out is None:
        out = torch.empty((hq,), dtype=torch.float32, device=q.device)
    rc = lib.hira_threshold(L.ptr(samples), L.dtype_code(samples.dtype), hkv, s, d, s * d, L.ptr(q), L.ptr(q2kv),
                            hq, method, k, L.ptr(out), L.current_stream(q.device))
    L.check(rc, "hira_threshold")
    return out


def prepare_query(q: torch.Tensor, sm_scale: float, q_hat=None, logit_scale=None):
    """q (H_q, D) fp32/bf16 contiguous -> (q_hat (H_q, D) fp32, logit_scale (H_q,) fp32)."""
    lib = L.load()
    hq, d = q.shape
    if q_hat is None:
        q_hat = torch.empty((hq, d), dtype=torch.float32, device=q.device)
    if logit_scale is None:
        logit_scale = torch.empty((hq,), dtype=torch.float32, device=q.device)
    rc = lib.hira_prepare_query(L.ptr(q), L.dtype_code(q.dtype), hq, d, float(sm_scale), L.ptr(q_hat),
                                L.ptr(logit_scale), L.current_stream(q.device))
    L.check(rc, "hira_prepare_query")
    return q_hat, logit_scale


def decode_attention(st: IndexState, q: torch.Tensor, sm_scale: float, tau: torch.Tensor, compact: CompactResult,
                     q_hat: torch.Tensor, logit_scale: torch.Tensor, *, q2kv=None, max_group: int = 0, flags: int = 0,
                     queued_k=None, queued_v=None, n_splits: int, workspace: torch.Tensor, out: torch.Tensor,
                     out_ml=None, scan_key=None, scan_out=None, searched_event=None):
    """prepare_query + search (compact) + sparse_attn in one library call.  q (H_q, D) fp32/bf16
    contiguous; everything else preallocated by the caller."""
    lib = L.load()
    hq = q.shape[0]
    n_queued, qstride = 0, 0
    if queued_k is not None and queued_k.shape[-2] > 0:
        assert queued_k.is_contiguous() and queued_v.is_contiguous()
        assert queued_k.dtype == st.dtype and queued_v.dtype == st.vdtype
        n_queued = queued_k.shape[-2]
        qstride = n_queued * st.dim
        if st.vdim != st.dim:
            raise ValueError("queued keys/values with vdim != dim are not supported")
    rc = lib.hira_decode_attention(st.struct, L.ptr(q), L.dtype_code(q.dtype), float(sm_scale), L.ptr(tau), L.ptr(q2kv),
                                   hq, max_group, flags, compact.tile_parents, L.ptr(q_hat), L.ptr(logit_scale),
                                   L.ptr(compact.idx), L.ptr(compact.score), L.ptr(compact.count),
                                   L.ptr(queued_k) if n_queued else None, L.ptr(queued_v) if n_queued else None,
                                   n_queued, qstride, n_splits, L.ptr(workspace), L.ptr(out), L.ptr(out_ml),
                                   out.stride(0), out_ml.stride(0) if out_ml is not None else 0,
                                   L.ptr(scan_key) if scan_out is not None else None,
                                   scan_key.stride(0) if scan_out is not None else 0, L.ptr(scan_out),
                                   searched_event, L.current_stream(st.device))
    L.check(rc, "hira_decode_attention")
    compact.n_tiles_active = None if st.active_parents == 0 else -(-st.active_parents // compact.tile_parents)
    return out


def kth_score(st: IndexState, compact: CompactResult, k: torch.Tensor, out=None):
    lib = L.load()
    hq = compact.idx.shape[0]
    if out is None:
        out = torch.empty((hq,), dtype=torch.float32, device=st.device)
    rc = lib.hira_kth_score(st.struct, hq, compact.tile_parents, L.ptr(compact.score), L.ptr(compact.count),
                            L.ptr(k), L.ptr(out), L.current_stream(st.device))
    L.check(rc, "hira_kth_score")
    return out


def build(st: IndexState, keys: torch.Tensor, values: Optional[torch.Tensor], *, cent_idx1=None, cent_idx2=None,
          n_iters: int = 1, balance_rounds: int = 0, use_tensor_cores: bool = True, token_base: int = 0):
    """keys (n_heads, n, D), values (n_heads, n, V) contiguous, index dtypes."""
    lib = L.load()
    assert keys.is_contiguous() and keys.dtype == st.dtype
    n = keys.shape[1]
    if values is not None:
        assert values.is_contiguous() and values.dtype == st.vdtype
    st.status.zero_()
    nbytes = int(lib.hira_build_workspace_bytes(st.struct, n))
    ws = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=st.device)
    rc = lib.hira_build(st.struct, L.ptr(keys), L.ptr(values), n, n * st.dim,
                        n * st.vdim if values is not None else 0, token_base, L.ptr(cent_idx1), L.ptr(cent_idx2),
                        n_iters, int(balance_rounds), 1 if use_tensor_cores else 0, L.ptr(st.status), L.ptr(ws), nbytes,
                        L.current_stream(st.device))
    L.check(rc, "hira_build")


def recompute_radii(st: IndexState):
    L.check(L.load().hira_recompute_radii(st.struct, L.current_stream(st.device)), "hira_recompute_radii")


def export(st: IndexState, n_out: int, token_base: int = 0):
    lib = L.load()
    out_k = torch.zeros((st.n_heads, n_out, st.dim), dtype=st.dtype, device=st.device)
    out_v = torch.zeros((st.n_heads, n_out, st.vdim), dtype=st.vdtype, device=st.device) if st.values is not None else None
    rc = lib.hira_export(st.struct, token_base, n_out, L.ptr(out_k), L.ptr(out_v), L.current_stream(st.device))
    L.check(rc, "hira_export")
    return out_k, out_v


def assign(points: torch.Tensor, cents: torch.Tensor, use_tensor_cores: bool = False):
    """points (H, n, D), cents (H, k, D) -> (idx (H, n) int32, dist2 (H, n) fp32)."""
    lib = L.load()
    h, n, d = points.shape
    k = cents.shape[1]
    dev = points.device
    idx = torch.empty((h, n), dtype=torch.int32, device=dev)
    d2 = torch.empty((h, n), dtype=torch.float32, device=dev)
    csq = torch.empty((h, k), dtype=torch.float32, device=dev)
    rc = lib.hira_assign(L.ptr(points.contiguous()), L.ptr(cents.contiguous()), L.dtype_code(points.dtype), h, n, k, d,
                         1 if use_tensor_cores else 0, L.ptr(csq), L.ptr(idx), L.ptr(d2), L.current_stream(dev))
    L.check(rc, "hira_assign")
    return idx, d2


class DecodeStep:
    """Device scratch and events of `hira_decode_step` for one index: the whole decode step of a
    layer (query copy, threshold, search, sparse attention, output copy and, beside them on a
    second stream, the 1-key append) behind one library call with host buffers in and out."""

    def __init__(self, st: IndexState, n_qheads: int, q_dtype: torch.dtype = torch.float32, *, flags: int,
                 fused_scan: bool = False, tau_samples: Optional[torch.Tensor] = None,
                 tau_method: int = L.HIRA_TAU_SAMPLE_MEAN_TOPK, tau_k: int = 16):
        lib = L.load()
        dev = st.device
        self.st, self.n_qheads, self.q_dtype = st, n_qheads, q_dtype
        tp = tile_parents(st)
        self.compact = alloc_compact(st, n_qheads, tp)
        # splits sized for the whole capacity: the bound on the slots in use moves from step to step
        self.n_splits = int(lib.hira_attn_default_splits(n_qheads, n_tiles(st, tp)))
        f32 = dict(dtype=torch.float32, device=dev)
        self.q_dev = torch.empty((n_qheads, st.dim), dtype=q_dtype, device=dev)
        self.k_dev = torch.empty((st.n_heads, st.dim), dtype=st.dtype, device=dev)
        self.v_dev = torch.empty((st.n_heads, max(st.vdim, 1)), dtype=st.vdtype, device=dev)
        self.q_hat = torch.empty((n_qheads, st.dim), **f32)
        self.logit_scale = torch.empty((n_qheads,), **f32)
        self.tau = torch.empty((n_qheads,), **f32)
        self.workspace = torch.empty((n_qheads * self.n_splits * (st.vdim + 2),), **f32)
        self.out_dev = torch.empty((n_qheads, st.vdim), **f32)
        self.scan = new_scan_slots(st) if fused_scan else None
        nbytes = int(lib.hira_append_workspace_bytes(st.struct, 1))
        self.append_ws = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=dev) if nbytes else None
        self.tau_samples = tau_samples
        s = L.HiraStepStruct()
        for name in ("q_dev", "k_dev", "v_dev", "q_hat", "logit_scale", "tau", "workspace", "out_dev", "scan",
                     "append_ws", "tau_samples"):
            setattr(s, name, L.ptr(getattr(self, name)))
        s.idx, s.score, s.count = L.ptr(self.compact.idx), L.ptr(self.compact.score), L.ptr(self.compact.count)
        s.status = L.ptr(st.status)
        s.append_ws_bytes = nbytes
        if tau_samples is not None:
            assert tau_samples.dtype == st.dtype and tau_samples.is_contiguous() and tau_samples.shape[0] == st.n_heads
            s.n_samples, s.samples_head_stride = tau_samples.shape[1], tau_samples.stride(0)
        s.tau_method, s.tau_k = tau_method, tau_k
        s.n_splits, s.tile_parents, s.flags = self.n_splits, tp, flags
        self._struct = s
        L.check(lib.hira_step_events_create(C.byref(s)), "hira_step_events_create")

    def __del__(self):
        try:
            L.load().hira_step_events_destroy(C.byref(self._struct))
        except Exception:
            pass

    def run(self, q_host: torch.Tensor, out_host: torch.Tensor, *, sm_scale: float, tau: Optional[torch.Tensor] = None,
            k_host: Optional[torch.Tensor] = None, v_host: Optional[torch.Tensor] = None, side_stream=None):
        """q_host (H_q, D), k_host (H_kv, D), v_host (H_kv, V), out_host (H_q, V) fp32: contiguous
        (pinned) host tensors.  `tau` (H_q,) on the device, or None to find it from the samples."""
        st = self.st
        assert q_host.dtype == self.q_dtype and q_host.is_contiguous() and out_host.is_contiguous()
        rc = L.load().hira_decode_step(st.struct, C.byref(self._struct), q_host.data_ptr(), L.dtype_code(self.q_dtype),
                                       float(sm_scale), self.n_qheads, L.ptr(tau),
                                       None if k_host is None else k_host.data_ptr(),
                                       None if v_host is None else v_host.data_ptr(), out_host.data_ptr(),
                                       L.current_stream(st.device),
                                       None if side_stream is None else side_stream.cuda_stream)
        L.check(rc, "hira_decode_step")
