"""CUDAIndexer: the reference's blocked 2/3-level index (indexer/cuda.py:16-1302) with
the same constructor, `build` / `update` entry points and tensor attributes, backed by
the CUDA library instead of torch op chains and Triton kernels.

Attribute parity (indexer/cuda.py:40-54): `children (H, P*bf, D)`, `values (1, H, P*bf, V)`,
`parents (H, P, D)`, `parent_radii (H, P)`, `grand_parents (H, G, D)`, `grand_parent_radii
(H, G)`, `_child_counts`, `_parent_valid`, `_gp_child_counts`, `branching_factor`, `depth`,
`pad_value`, `dim`, `num_heads`.  They are views over the memory the kernels use.

Differences by design:
  * children keep the dtype of the keys given to `build` (the reference always casts to
    float32, indexer/cuda.py:365-368), so a bf16 cache is searched as bf16;
  * validity is explicit state (`_child_counts`, `_gp_child_counts`, `used`), not "row is
    all pad_value";
  * `max_context` pre-allocates room for that many keys per head so that `update` never
    reallocates and never synchronises with the host; without it the arrays are sized
    exactly as the reference sizes them and grow (by reallocation) when needed;
  * a batch larger than 1 is folded into the head axis (the reference is batch-1,
    indexer/cuda.py:61).
"""
from __future__ import annotations

from enum import Enum
from typing import Optional

import torch

from .. import index_state as S
from .base import BaseIndexer

DEFAULT_PAD_VALUE = 0.0


class CUDAIndexer(BaseIndexer):

    class DEPTH(Enum):
        TWO_LEVELS = 2
        THREE_LEVELS = 3

    def __init__(self, num_levels, max_iterations: int, branching_factor: int, verbose: bool = False,
                 pad_value: float = DEFAULT_PAD_VALUE, *, max_context: Optional[int] = None,
                 reserve_worst_case: bool = False, use_tensor_cores: bool = True, seed: int = 1234,
                 balance_rounds: int = 0):
        # More than three levels (HiraConfig.num_levels defaults to 5, the CPU indexer's depth) are
        # served by a three-level index: balls enclose all their descendants, so the keys selected
        # under a leaf-tested rule do not depend on the depth; further levels would only skip whole
        # grandparent blocks earlier.  The reference's CUDAIndexer rejects such depths (indexer/cuda.py:18-21).
        self.requested_levels = num_levels.value if isinstance(num_levels, CUDAIndexer.DEPTH) else int(num_levels)
        if not isinstance(num_levels, CUDAIndexer.DEPTH):
            num_levels = min(int(num_levels), 3)
        self.depth = num_levels if isinstance(num_levels, CUDAIndexer.DEPTH) else CUDAIndexer.DEPTH(num_levels)
        self.max_iterations = max_iterations
        self.branching_factor = int(branching_factor)
        self.verbose = verbose
        self.pad_value = pad_value
        self.max_context = max_context
        self.reserve_worst_case = reserve_worst_case
        self.balance_rounds = int(balance_rounds)   # capacity-aware assignment rounds of the build (0: reference rule)
        self.use_tensor_cores = use_tensor_cores
        self.seed = seed
        self.dim: int = 0
        self.num_heads: int = 0
        self.state: Optional[S.IndexState] = None
        self._parents_bound = 0   # host-side upper bounds on used parent / grandparent slots
        self._gp_bound = 0
        self._snapshot = None     # (pinned copy of `used`, event, keys appended when it was taken)
        self._scan_slots = None   # nearest-parent results of a search that scanned for the next update
        self._scan_pending = False
        self._searched = None     # event recorded right after the latest search of a decode step
        self._searched_fresh = False
        self._pending_append = None   # event of an update that ran on a caller's side stream
        self._pinned = None
        self._appended = 0        # keys appended since the build
        self._n_keys = 0

    # ---- reference attribute names as views ---------------------------------
    @property
    def children(self):
        return None if self.state is None else self.state.children

    @property
    def values(self):
        return None if self.state is None or self.state.values is None else self.state.values.unsqueeze(0)

    @property
    def parents(self):
        return None if self.state is None else self.state.parents

    @property
    def parent_radii(self):
        return None if self.state is None else self.state.parent_radii

    @property
    def grand_parents(self):
        return None if self.state is None else self.state.grand_parents

    @property
    def grand_parent_radii(self):
        return None if self.state is None else self.state.gp_radii

    @property
    def _child_counts(self):
        return None if self.state is None else self.state.child_counts

    @property
    def _gp_child_counts(self):
        return None if self.state is None else self.state.gp_counts

    @property
    def _parent_valid(self):
        st = self.state
        if st is None:
            return None
        p = torch.arange(st.cap_parents, device=st.device)
        if st.depth == 3:
            g = p // st.bf
            ok = (g[None, :] < st.used[:, 1:2]) & ((p % st.bf)[None, :] < st.gp_counts.gather(1, g[None, :].expand(st.n_heads, -1).long()))
        else:
            ok = p[None, :] < st.used[:, 0:1]
        return ok

    @property
    def slot2token(self):
        return None if self.state is None else self.state.slot2token

    # ---- build --------------------------------------------------------------
    @staticmethod
    def _fold(t: torch.Tensor) -> torch.Tensor:
        if t.ndim != 4:
            raise ValueError(f"expected a (B, H, L, D) tensor, got {tuple(t.shape)}")
        b, h, l, d = t.shape
        return t.reshape(b * h, l, d).contiguous()

    @staticmethod
    def _stratified(h: int, n: int, k: int, g: torch.Generator, device) -> torch.Tensor:
        lo = (torch.arange(k + 1, device=device, dtype=torch.int64) * n) // k        # stride boundaries
        width = (lo[1:] - lo[:-1]).to(torch.float32)
        jitter = (torch.rand((h, k), generator=g, device=device) * width).to(torch.int64)
        return (lo[:-1] + torch.minimum(jitter, (lo[1:] - lo[:-1] - 1).clamp_min(0))).to(torch.int32).contiguous()

    def _capacity_parents(self, n_keys: int) -> int:
        bf = self.branching_factor
        k1 = max(1, -(-n_keys // bf))
        if self.max_context is None:
            return k1
        # Room for max_context keys.  Worst case of the append rule: every appended key finds
        # its nearest parent full and opens a new parent -- and, with three levels, finds its
        # nearest grandparent full too and opens a whole new grandparent block (bf^2 child
        # slots: 512 KiB of bf16 keys and values at bf = 32, D = 128, per key and head).
        # `reserve_worst_case` pre-allocates exactly that, so that `update` never reallocates;
        # otherwise the reserve is what the appended keys need when they pack (one parent per bf
        # keys, one grandparent per bf parents) plus a few blocks, and `_ensure_capacity` grows
        # the arrays by half when the device counters show it running short.
        extra = max(self.max_context, n_keys) - n_keys
        if self.depth == CUDAIndexer.DEPTH.THREE_LEVELS:
            spare = extra if self.reserve_worst_case else min(extra, -(-extra // (bf * bf)) + 8)
            return (-(-k1 // bf) + spare) * bf
        spare = extra if self.reserve_worst_case else min(extra, -(-extra // bf) + 8 * bf)
        return k1 + spare

    @torch.no_grad()
    def build(self, keys: torch.Tensor, values: Optional[torch.Tensor] = None):
        """keys (B, H, L, D); values optional (B, H, L, V)."""
        return self._build(keys, values, reuse=None)

    def _build(self, keys, values, reuse: Optional[S.IndexState]):
        """`reuse`: a state of this indexer whose arrays are taken over when they are large enough
        (a rebuild): nothing is allocated and only the slots that were in use are cleared."""
        if not torch.cuda.is_available():
            raise RuntimeError("CUDAIndexer needs a CUDA device (there is no CPU fallback)")
        keys = self._fold(keys.to("cuda"))
        h, n, d = keys.shape
        if values is not None:
            values = self._fold(values.to("cuda"))
            if values.shape[:2] != keys.shape[:2]:
                raise ValueError("values must have the same (B, H, L) as keys")
        self.num_heads, self.dim = h, d
        bf = self.branching_factor
        cap_p = self._capacity_parents(n)
        vdim = values.shape[-1] if values is not None else 0
        st = reuse
        if st is not None and not (st.n_heads == h and st.dim == d and st.vdim == vdim and st.bf == bf
                                   and st.depth == self.depth.value and st.dtype == keys.dtype
                                   and (values is None or st.vdtype == values.dtype)
                                   and st.cap_parents >= (-(-cap_p // bf) * bf if st.depth == 3 else cap_p)):
            st = None
        if st is None:
            st = S.IndexState(n_heads=h, dim=d, vdim=vdim, bf=bf, depth=self.depth.value, cap_parents=cap_p,
                              dtype=keys.dtype, vdtype=values.dtype if values is not None else None, device=keys.device,
                              with_values=values is not None)
        else:
            st.active_parents = self.active_parents     # the build clears only what was in use
        k1 = -(-n // bf) if n else 0
        k2 = -(-k1 // bf) if k1 else 0
        g = torch.Generator(device=keys.device)
        g.manual_seed(self.seed)
        cent1 = cent2 = None
        if n:
            # distinct random points as initial centres (indexer/cuda.py:229-237): one uniformly drawn
            # point out of each of k equal strides of the sequence (O(k), no sort)
            cent1 = self._stratified(h, n, k1, g, keys.device)
            if st.depth == 3:
                cent2 = self._stratified(h, k1, k2, g, keys.device)
        S.build(st, keys, values, cent_idx1=cent1, cent_idx2=cent2, n_iters=max(1, int(self.max_iterations)),
                balance_rounds=self.balance_rounds, use_tensor_cores=self.use_tensor_cores)
        self.state = st
        self._n_keys = n
        self._parents_bound = k2 * bf if st.depth == 3 else k1
        self._gp_bound = k2
        self._snapshot = None
        self._scan_slots, self._scan_pending = None, False
        self._appended = 0
        st.active_parents = 0
        return self

    # ---- update -------------------------------------------------------------
    def _ensure_capacity(self, m: int):
        st = self.state
        need_p = self._parents_bound + m
        need_g = self._gp_bound + m
        short = (need_g > st.cap_gp) if st.depth == 3 else (need_p > st.cap_parents)
        if not short:
            return
        # tighten the bounds from the device state before paying for a reallocation
        used = st.used.max(dim=0).values.tolist()
        self._parents_bound, self._gp_bound = int(used[0]), int(used[1])
        self._snapshot = None
        need_p, need_g = self._parents_bound + m, self._gp_bound + m
        if st.depth == 3:
            if need_g <= st.cap_gp:
                return
            new_cap = max(need_g, st.cap_gp + max(1, st.cap_gp // 2)) * st.bf
        else:
            if need_p <= st.cap_parents:
                return
            new_cap = max(need_p, st.cap_parents + max(1, st.cap_parents // 2))
        self.state = st.grown(new_cap)

    # ---- updates beside the attention, on a second stream ---------------------
    def searched_event(self) -> int:
        """Handle (cudaEvent_t) of the event a decode step records right after its search; an
        `update(..., stream=side)` that follows starts once that event has fired."""
        if self._searched is None:
            self._searched = torch.cuda.Event()
            self._searched.record(torch.cuda.current_stream(self.state.device))   # creates the CUDA event
        self._searched_fresh = True
        return self._searched.cuda_event

    def wait_pending_update(self):
        """Makes the current stream wait for an update that is still running on a side stream.
        The searcher and the decode step call this before they touch the index."""
        if self._pending_append is not None:
            torch.cuda.current_stream(self.state.device).wait_event(self._pending_append)
            self._pending_append = None

    @torch.no_grad()
    def begin_scanned_update(self, key: torch.Tensor):
        """For the search that precedes `update(key, value, scanned=True)`: the key folded to
        (B*H, D) in the index dtype and the per-head slots the search leaves its nearest-parent
        result in."""
        st = self.state
        if st is None:
            raise ValueError("Indexer is not built")
        if key.ndim != 4 or key.shape[2] != 1:
            raise ValueError(f"append_key must be (B, H, 1, D), got {tuple(key.shape)}")
        k = self._fold(key.to(st.device)).to(st.dtype)[:, 0].contiguous()
        if k.shape != (self.num_heads, self.dim):
            raise ValueError(f"append_key has (heads, dim)={tuple(k.shape)}, index has ({self.num_heads}, {self.dim})")
        if self._scan_slots is None or self._scan_slots.device != st.device or self._scan_slots.numel() != st.n_heads:
            self._scan_slots = S.new_scan_slots(st)
        elif self._scan_pending:
            self._scan_slots.fill_(-1)        # an earlier scan was never consumed
        self._scan_pending = True
        return k, self._scan_slots

    @torch.no_grad()
    def update(self, new_keys: torch.Tensor, new_values: Optional[torch.Tensor] = None, scanned: bool = False,
               stream: Optional["torch.cuda.Stream"] = None):
        """new_keys (B, H, M, D), new_values optional (B, H, M, V) -- appended one after another.
        `scanned=True` (M == 1): the search that ran just before was given this key
        (`hira_decode_attention(..., append_key=new_keys)`) and already found its nearest parent.
        `stream`: run the append on this stream, beside the attention of the decode step that was
        enqueued just before on the current stream: it starts when that step's search has finished
        (the attention reads nothing the append writes).  `new_keys` / `new_values` must be ready
        on `stream`; whoever touches the index next waits for the append (`wait_pending_update`)."""
        if self.state is None:
            raise ValueError("Indexer is not built")
        if stream is not None:
            cur = torch.cuda.current_stream(self.state.device)
            if stream != cur:
                if self._pending_append is not None:
                    stream.wait_event(self._pending_append)
                if self._searched is not None and self._searched_fresh:
                    stream.wait_event(self._searched)
                else:
                    stream.wait_stream(cur)     # no decode step to hook on: after everything enqueued so far
                self._searched_fresh = False
                for t in (new_keys, new_values):      # allocated on another stream, consumed on this one
                    if t is not None and t.is_cuda:
                        t.record_stream(stream)
                with torch.cuda.stream(stream):
                    self.update(new_keys, new_values, scanned=scanned)
                    done = torch.cuda.Event()
                    done.record(stream)
                self._pending_append = done
                return self
        self.wait_pending_update()
        assert new_values is None or new_keys.shape[:3] == new_values.shape[:3]
        if new_keys.ndim != 4:
            raise ValueError(f"new_keys must be (B, H, M, D), got {tuple(new_keys.shape)}")
        k = self._fold(new_keys.to(self.state.device))
        h, m, d = k.shape
        if h != self.num_heads or d != self.dim:
            raise ValueError(f"new_keys has (heads, dim)=({h}, {d}), index has ({self.num_heads}, {self.dim})")
        has_values = self.state.values is not None
        v = None
        if has_values:
            if new_values is None:
                raise ValueError("the index stores values: new_values is required")
            v = self._fold(new_values.to(self.state.device)).to(self.state.vdtype)
        if m == 0:
            return self
        self._ensure_capacity(m)
        if scanned:
            if m != 1 or not self._scan_pending:
                raise ValueError("update(scanned=True) needs one key per head and a search that scanned for it")
            S.append_scanned(self.state, k.to(self.state.dtype), v, self._scan_slots)
        else:
            if self._scan_pending:
                self._scan_slots.fill_(-1)    # the index changes: that scan is void
            S.append(self.state, k.to(self.state.dtype), v)
        self._scan_pending = False
        self._parents_bound += m
        self._gp_bound += m
        self._n_keys += m
        self._appended += m
        if self._snapshot is not None or self._appended % self.BOUND_REFRESH_EVERY < m:
            self._tighten_bounds()
        return self

    BOUND_REFRESH_EVERY = 8   # appended keys between two read-backs of the device counters

    def _tighten_bounds(self):
        """The bounds grow by the worst case (one new parent and one new grandparent per key);
        the counts the device actually reached come back through a small asynchronous copy, read
        one or more appends later without ever blocking on the stream."""
        st = self.state
        if st.device.type != "cuda":
            return
        snap = self._snapshot
        if snap is not None:
            host, event, appended_then = snap
            if not event.query():
                return
            used = host.max(dim=0).values.tolist()
            since = self._appended - appended_then
            self._parents_bound = min(self._parents_bound, int(used[0]) + since)
            self._gp_bound = min(self._gp_bound, int(used[1]) + since)
            self._snapshot = None
            return
        if self._pinned is None or self._pinned[0].shape != st.used.shape:
            self._pinned = [torch.empty(tuple(st.used.shape), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._pinned.reverse()
        host = self._pinned[0]
        host.copy_(st.used, non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(st.device))
        self._snapshot = (host, event, self._appended)

    @property
    def active_parents(self) -> int:
        """Upper bound on the parent slots that can hold keys (for depth 3 whole grandparent
        blocks): what the searcher passes down so that empty capacity is not visited."""
        st = self.state
        if st is None:
            return 0
        n = self._gp_bound * st.bf if st.depth == 3 else self._parents_bound
        return min(int(n), st.cap_parents)

    def check_status(self):
        """Raises if an append ran out of pre-allocated slots (reads one word from the device)."""
        self.wait_pending_update() if self.state is not None else None
        code = int(self.state.status.item())
        if code & 4:
            raise RuntimeError("the tensor-core assignment of the build gave up on a bounded wait for some points "
                               "(status bit HIRA_STATUS_ASSIGN_FAILED); rebuild with use_tensor_cores=False")
        if code:
            raise RuntimeError(f"index capacity exhausted during update (status {code}); raise max_context")

    @torch.no_grad()
    def rebuild(self):
        """Full rebuild over the keys currently stored (token order), e.g. every N decode steps.  The
        arrays are reused when they have room for `max_context` again: no allocation, and only the
        slots that were in use are cleared."""
        self.wait_pending_update() if self.state is not None else None
        st = self.state
        n = self._n_keys
        st.active_parents = self.active_parents     # the export visits only the slots that can hold keys
        keys, values = S.export(st, n)
        self._build(keys.unsqueeze(0), None if values is None else values.unsqueeze(0), reuse=st)
        return self

    # ---- checkpoint ---------------------------------------------------------
    def state_dict(self) -> dict:
        self.wait_pending_update() if self.state is not None else None
        d = self.state.state_dict()
        d["meta"].update(n_keys=self._n_keys, parents_bound=self._parents_bound, gp_bound=self._gp_bound)
        return d

    @classmethod
    def from_state_dict(cls, sd: dict, device="cuda", **kw) -> "CUDAIndexer":
        m = sd["meta"]
        dt = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16}
        self = cls(m["depth"], kw.pop("max_iterations", 1), m["bf"], **kw)
        st = S.IndexState(n_heads=m["n_heads"], dim=m["dim"], vdim=m["vdim"], bf=m["bf"], depth=m["depth"],
                          cap_parents=m["cap_parents"], dtype=dt[m["dtype"]], vdtype=dt[m["vdtype"]], device=device,
                          with_values=sd.get("values") is not None)
        st.load_arrays(sd)
        self.state, self.num_heads, self.dim = st, m["n_heads"], m["dim"]
        self._n_keys = m.get("n_keys", 0)
        self._parents_bound = m.get("parents_bound", st.cap_parents)
        self._gp_bound = m.get("gp_bound", st.cap_gp)
        return self
