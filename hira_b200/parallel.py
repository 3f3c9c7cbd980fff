"""Multi-GPU plumbing for the decode path (one process per GPU, torch.distributed).

Two ways to spread the path over the GPUs of a node, neither present in the reference
(which is single-device):
  * by KV head: the (batch, kv_head) groups are independent from index build to attention
    output, so each rank owns whole heads and nothing is exchanged (`shard_heads`);
  * by sequence shard (million-token contexts): each rank indexes a contiguous slice of the
    sequence, all ranks search with the same threshold, and the per-shard softmax partials
    (m, l, normalised o) are exchanged and merged with the log-sum-exp arithmetic: by ONE
    kernel per step that stores this rank's rows into every peer's buffer over NVLink peer
    memory, waits for the peers' rows and merges them (`PeerPartialsExchange`), or by an NCCL
    all-gather followed by the merge kernel (`PartialsExchange`, or the allocation-per-call
    `gather_partials` + `merge_gathered`).  The append goes to the last shard only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def shard_heads(n_kv_heads: int, world_size: int, rank: int) -> range:
    """KV heads owned by `rank`: contiguous, as even as possible (8 heads over 8 GPUs -> 1 each)."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n_kv_heads, world_size)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def shard_sequence(n_tokens: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the contiguous sequence shard of `rank`."""
    per = -(-n_tokens // world_size)
    lo = min(n_tokens, rank * per)
    return lo, min(n_tokens, lo + per)


class PartialsExchange:
    """The one exchange of sequence-sharded decode: every rank's (m, l, normalised out) rows, one
    message of H_q x (2 + V) floats per rank, all-gathered into a buffer that is allocated once.
    The attention kernel writes this rank's rows straight into its slice (`local_out`,
    `local_ml` are strided views of it), the all-gather is in place, and the merge kernel reads
    the gathered buffer through strides -- no concatenation and no copy on either side."""

    def __init__(self, n_qheads: int, vdim: int, device, group=None):
        import torch.distributed as dist
        self.group = group
        ok = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if ok else 1
        self.rank = dist.get_rank(group) if ok else 0
        self.n_qheads, self.vdim = n_qheads, vdim
        self.buf = torch.zeros((self.world, n_qheads, vdim + 2), dtype=torch.float32, device=device)
        mine = self.buf[self.rank]
        self.local_ml = mine[:, :2]
        self.local_out = mine[:, 2:]

    @property
    def message_bytes(self) -> int:
        return self.n_qheads * (self.vdim + 2) * 4

    def all_gather(self):
        """Enqueues the all-gather on the current stream (rank r's rows land in buf[r])."""
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.buf.view(self.world * self.n_qheads, self.vdim + 2), self.buf[self.rank],
                                        group=self.group)
        return self.buf

    def merge(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Log-sum-exp merge of the gathered partials on the device (hira_merge_partials)."""
        from . import index_state as S
        return S.merge_partials(self.buf[:, :, 2:], self.buf[:, :, :2], out=out)


class PeerPartialsExchange:
    """The exchange of sequence-sharded decode over NVLink peer memory, fused with the merge
    (hira_exchange_merge): every rank owns a buffer its peers map through CUDA IPC; one kernel per
    step stores this rank's (m, l, normalised out) rows into every rank's buffer with plain peer
    stores, flags them with the step number, waits (bounded) for the peers' rows of the same step and
    merges.  No library collective is on the data path; torch.distributed only carries the 64-byte
    handles at set-up.  Same surface as PartialsExchange: the attention kernel writes `local_out` /
    `local_ml`, `all_gather()` is a no-op, `merge(out=)` runs the fused step.

    peers=... (a list of already mapped buffer addresses with this rank's own at [rank]) skips the
    IPC set-up: several emulated ranks of one process on one GPU, driven with `phases`.

    The step number is an argument of the launch: a step recorded into a CUDA graph carries its number
    with it, so such a graph can be replayed once per recording, not over and over (the peers' flags would
    already hold that number)."""

    def __init__(self, n_qheads: int, vdim: int, device, group=None, *, rank: Optional[int] = None,
                 world: Optional[int] = None, peers=None, wait_seconds: float = 2.0):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib as L
        self._L, self._C = L, C
        self.lib = L.load()
        self.group = group
        ok = dist.is_available() and dist.is_initialized()
        self.world = world if world is not None else (dist.get_world_size(group) if ok else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if ok else 0)
        if not 1 <= self.world <= L.MAX_PEERS:
            raise ValueError(f"PeerPartialsExchange serves up to {L.MAX_PEERS} ranks, got {self.world}")
        self.n_qheads, self.vdim, self.device = n_qheads, vdim, torch.device(device)
        self.wait_seconds = float(wait_seconds)
        self.local = torch.zeros((n_qheads, vdim + 2), dtype=torch.float32, device=device)
        self.local_ml = self.local[:, :2]
        self.local_out = self.local[:, 2:]
        self.status = torch.zeros((1,), dtype=torch.int32, device=device)
        self.seq = 0
        self._own = None
        self._opened = []
        if peers is not None:
            addrs = [int(a) for a in peers]
        else:
            nbytes = int(self.lib.hira_exchange_bytes(self.world, n_qheads, vdim))
            own = C.c_void_p()
            handle = C.create_string_buffer(L.PEER_HANDLE_BYTES)
            with torch.cuda.device(self.device):
                L.check(self.lib.hira_peer_alloc(nbytes, C.byref(own), handle), "hira_peer_alloc")
            self._own = own.value
            addrs = [None] * self.world
            addrs[self.rank] = own.value
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                with torch.cuda.device(self.device):
                    for r, hb in enumerate(handles):
                        if r == self.rank:
                            continue
                        p = C.c_void_p()
                        L.check(self.lib.hira_peer_open(hb, C.byref(p)), f"hira_peer_open(rank {r})")
                        addrs[r] = p.value
                        self._opened.append(p.value)
        self.peer_addrs = addrs
        self._peers = (C.c_void_p * self.world)(*addrs)

    @property
    def message_bytes(self) -> int:
        return self.n_qheads * (self.vdim + 2) * 4

    def all_gather(self):
        """Nothing to enqueue: the rows travel inside `merge`."""
        return None

    def merge(self, out: Optional[torch.Tensor] = None, out_ml: Optional[torch.Tensor] = None, *, phases: int = 3,
              seq: Optional[int] = None) -> torch.Tensor:
        """One step: push, wait, merge (phases=3) on the current stream; `check()` reads the status."""
        L = self._L
        if out is None:
            out = torch.empty((self.n_qheads, self.vdim), dtype=torch.float32, device=self.device)
        if seq is None:
            self.seq += 1
            seq = self.seq
        rc = self.lib.hira_exchange_merge(L.ptr(self.local), self._peers, self.world, self.rank, self.n_qheads, self.vdim,
                                          seq, phases, self.wait_seconds, L.ptr(out), L.ptr(out_ml), L.ptr(self.status),
                                          L.current_stream(self.device))
        L.check(rc, "hira_exchange_merge")
        return out

    def check(self):
        """Synchronises and raises if a wait for a peer's rows ran out in any step since the last check."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("hira_exchange_merge: a peer's partials did not arrive within "
                               f"{self.wait_seconds} s (rank {self.rank} of {self.world})")

    def close(self):
        """Unmaps the peers' buffers; call on every rank, then a host barrier, then `free()`."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened:
                self.lib.hira_peer_close(p)
        self._opened = []

    def free(self):
        if self._own is not None:
            with torch.cuda.device(self.device):
                self.lib.hira_peer_free(self._own)
            self._own = None


def gather_partials(out: torch.Tensor, ml: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gathers the per-shard attention partials.  out (H_q, V) normalised fp32, ml (H_q, 2) =
    (running max, denominator).  Returns (parts_o (world, H_q, V), parts_ml (world, H_q, 2))."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    payload = torch.cat([out, ml], dim=1).contiguous()            # one message per rank: H_q x (V + 2) floats
    hq = payload.shape[0]
    flat = torch.empty((world * hq, payload.shape[1]), dtype=payload.dtype, device=payload.device)
    dist.all_gather_into_tensor(flat, payload, group=group)     # rank r's rows land at [r*hq, (r+1)*hq)
    gathered = flat.view(world, hq, payload.shape[1])
    v = out.shape[1]
    return gathered[..., :v].contiguous(), gathered[..., v:].contiguous()


def merge_gathered(parts_o: torch.Tensor, parts_ml: torch.Tensor, out: Optional[torch.Tensor] = None):
    """Log-sum-exp merge of gathered partials on the device (hira_merge_partials)."""
    from . import index_state as S
    return S.merge_partials(parts_o, parts_ml, out=out)
