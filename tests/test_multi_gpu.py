"""Two-GPU checks (skipped on a single GPU): sequence-sharded decode -- every rank indexes its
slice of the sequence, all ranks search with the same threshold, the per-shard softmax
partials are all-gathered over NCCL and merged on the device -- against attention over the
whole sequence; the one-kernel exchange over NVLink peer memory against that; and KV-head sharding
against the unsharded result."""
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200.parallel import gather_partials, merge_gathered, shard_heads, shard_sequence

    h, g, n, d, bf = 2, 4, 8192, 128, 32
    gen = torch.Generator().manual_seed(5)
    keys = torch.randn((h, n, d), generator=gen).to(torch.bfloat16)
    vals = torch.randn((h, n, d), generator=gen).to(torch.bfloat16)
    q = torch.randn((h * g, d), generator=gen)
    q = (q / q.norm(dim=-1, keepdim=True)).cuda()
    scores = torch.einsum("hgd,hnd->hgn", q.cpu().view(h, g, d), keys.float()).reshape(h * g, n)
    srt = torch.sort(scores, dim=-1).values
    kth = n - n // 20
    tau = (0.5 * (srt[:, kth - 1] + srt[:, kth])).cuda()              # midpoint: no key on the boundary
    scaling = torch.full((h * g,), 4.0, device="cuda")
    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE

    def attend(k_part, v_part, heads):
        st = S.IndexState(n_heads=k_part.shape[0], dim=d, vdim=d, bf=bf, depth=3, cap_parents=-(-k_part.shape[1] // bf),
                          dtype=torch.bfloat16, vdtype=torch.bfloat16, device="cuda")
        S.build(st, k_part.cuda().contiguous(), v_part.cuda().contiguous())
        qs = torch.cat([q[hh * g:(hh + 1) * g] for hh in heads]).contiguous()
        ts = torch.cat([tau[hh * g:(hh + 1) * g] for hh in heads]).contiguous()
        sc = scaling[: qs.shape[0]].contiguous()
        _, compact = S.search(st, qs, ts, scaling=sc, flags=flags, want_compact=True)
        ml = torch.empty((qs.shape[0], 2), device="cuda")
        out = S.sparse_attn(st, qs, sc, compact, out_ml=ml)
        return out, ml

    # reference: softmax over the selected keys of the whole sequence (fp32, rank 0's copy)
    mask = scores >= tau.cpu()[:, None]
    logits = torch.where(mask, scores * 4.0, torch.full_like(scores, float("-inf")))
    w = torch.softmax(logits, dim=-1)
    want = torch.einsum("hgn,hnd->hgd", w.view(h, g, n), vals.float()).reshape(h * g, d)

    # (1) sequence shards + NCCL all-gather + merge
    lo, hi = shard_sequence(n, world, rank)
    out, ml = attend(keys[:, lo:hi], vals[:, lo:hi], range(h))
    parts_o, parts_ml = gather_partials(out, ml)
    merged = merge_gathered(parts_o, parts_ml)
    torch.cuda.synchronize()
    err_seq = float((merged.cpu() - want).abs().max() / want.abs().max())

    # (1b) the same exchange as ONE kernel over NVLink peer memory (push, wait, merge): bit-identical
    # to the all-gather + merge, step after step on both buffer parities
    from hira_b200.parallel import PeerPartialsExchange
    ex = PeerPartialsExchange(h * g, d, "cuda")
    same = True
    for step in range(4):
        f = 1.0 + 0.25 * step                                    # different rows every step
        ex.local_out.copy_(out * f)
        ex.local_ml.copy_(ml)
        po, pml = gather_partials(out * f, ml)
        want_step = merge_gathered(po, pml)
        got = ex.merge()
        ex.check()
        same = same and torch.equal(got, want_step)
    dist.barrier()
    ex.close()
    dist.barrier()
    ex.free()

    # (2) KV-head shards: no exchange on the data path, only the comparison gathers
    mine = list(shard_heads(h, world, rank))
    out_h, _ = attend(keys[mine], vals[mine], mine)
    gathered = [torch.empty_like(out_h) for _ in range(world)]
    dist.all_gather(gathered, out_h)
    torch.cuda.synchronize()
    err_head = float((torch.cat(gathered).cpu() - want).abs().max() / want.abs().max())
    ret[rank] = (err_seq, err_head, same)
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_and_head_sharding_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 1000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert len(ret) == 2
        for err_seq, err_head, same in ret.values():
            assert err_seq < 2e-3 and err_head < 2e-3, (err_seq, err_head)
            assert same, "the peer-memory exchange differs from all-gather + merge"
