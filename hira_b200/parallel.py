"""Multi-GPU plumbing for the decode path (one process per GPU, torch.distributed).

Two ways to spread the path over the GPUs of a node, neither present in the reference
(which is single-device):
  * by KV head: the (batch, kv_head) groups are independent from index build to attention
    output, so each rank owns whole heads and nothing is exchanged (`shard_heads`);
  * by sequence shard (million-token contexts): each rank indexes a contiguous slice of the
    sequence, all ranks search with the same threshold, and the per-shard softmax partials
    (m, l, normalised o) are all-gathered and merged with the log-sum-exp kernel
    (`PartialsExchange`, or the allocation-per-call `gather_partials` + `merge_gathered`).
    The append goes to the last shard only.
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
