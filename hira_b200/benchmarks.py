"""Secondary workloads of the decode path (the headline one lives in bench.py):

    python -m hira_b200.benchmarks streaming          # prefix 65,536 keys/head, 4,096 single-key appends,
                                                      # full rebuild every 1,024: append us, rebuild ms
    python -m hira_b200.benchmarks longctx            # 131,072 tokens per GPU, 64 q / 8 kv heads, bf 64:
    torchrun --nproc-per-node N -m hira_b200.benchmarks longctx   # sequence shards, NCCL all-gather merge

Synthetic data, seeded; one JSON line per run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from . import _lib as L
from . import index_state as S
from .indexer import CUDAIndexer
from .parallel import gather_partials, merge_gathered

DIM = 128
ROPE_BASE = 500000.0


def _rope(x, pos):
    d = x.shape[-1]
    inv = 1.0 / (ROPE_BASE ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    c, s = ang.cos(), ang.sin()
    a, b = x[..., : d // 2].clone(), x[..., d // 2:].clone()
    x[..., : d // 2] = a * c - b * s
    x[..., d // 2:] = b * c + a * s
    return x


def keys_rope(h, n, seed, dev, first=0):
    """N(0,1) with RoPE by position and 4 outlier channels x8 (bf16)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    out = torch.empty((h, n, DIM), dtype=torch.bfloat16, device=dev)
    pos = torch.arange(first, first + n, device=dev)
    for i in range(h):
        k = _rope(torch.randn((n, DIM), generator=g, device=dev), pos)
        k[:, [7, 42, 71, 110]] *= 8.0
        out[i] = k.to(torch.bfloat16)
    return out


def keys_aniso(h, n, seed, dev):
    """N(0,1) scaled per channel by exp(N(0, 0.5)) (bf16)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    scale = torch.exp(torch.randn((DIM,), generator=g, device=dev) * 0.5)
    out = torch.empty((h, n, DIM), dtype=torch.bfloat16, device=dev)
    for i in range(h):
        out[i] = (torch.randn((n, DIM), generator=g, device=dev) * scale).to(torch.bfloat16)
    return out


def streaming(args):
    dev = torch.device("cuda", 0)
    h, prefix, steps, every, bf = 8, args.prefix, args.steps, args.rebuild_every, 32
    keys = keys_rope(h, prefix + steps, 1, dev)
    vals = torch.randn((h, prefix + steps, DIM), device=dev).to(torch.bfloat16)
    ix = CUDAIndexer(3, 1, bf, max_context=prefix + every + 8)   # room until the next rebuild
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ix.build(keys[None, :, :prefix], vals[None, :, :prefix])
    e1.record()
    torch.cuda.synchronize()
    build_ms = e0.elapsed_time(e1)
    append_us, rebuild_ms = [], []
    pos = prefix
    while pos < prefix + steps:
        n = min(every, prefix + steps - pos)
        e0.record()
        for i in range(n):
            S.append(ix.state, keys[:, pos + i:pos + i + 1].contiguous(), vals[:, pos + i:pos + i + 1].contiguous())
        e1.record()
        torch.cuda.synchronize()
        append_us.append(e0.elapsed_time(e1) * 1e3 / n)
        pos += n
        ix._n_keys = pos
        ix.check_status()
        if pos < prefix + steps or args.final_rebuild:
            ix.max_context = pos + every + 8
            e0.record()
            ix.rebuild()
            e1.record()
            torch.cuda.synchronize()
            rebuild_ms.append(e0.elapsed_time(e1))
    print(json.dumps({"workload": "streaming_update", "heads": h, "prefix": prefix, "appends": steps,
                      "rebuild_every": every, "levels": 3, "branching": bf, "dtype": "bf16",
                      "append_us_per_step": statistics.mean(append_us), "append_us_by_window": append_us,
                      "rebuild_ms": statistics.mean(rebuild_ms) if rebuild_ms else None, "rebuilds": len(rebuild_ms),
                      "initial_build_ms": build_ms}))


def longctx(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    hkv, hq, shard, bf = 8, 64, args.shard, 64
    keys = keys_aniso(hkv, shard, 100 + rank, dev)
    vals = torch.randn((hkv, shard, DIM), device=dev).to(torch.bfloat16)
    k1 = -(-shard // bf)
    k2 = -(-k1 // bf)
    spare = args.steps + args.warmup + 8
    st = S.IndexState(n_heads=hkv, dim=DIM, vdim=DIM, bf=bf, depth=3, cap_parents=(k2 + spare) * bf,
                      dtype=torch.bfloat16, vdtype=torch.bfloat16, device=dev)
    S.build(st, keys, vals)
    g = torch.Generator(device=dev).manual_seed(7)            # the same query on every rank
    q = torch.randn((hq, DIM), generator=g, device=dev)
    q_hat, lscale = S.prepare_query(q, DIM ** -0.5)
    # one threshold for all shards: 2% of this shard's keys (the shards are identically distributed)
    tp = S.tile_parents(st)
    compact = S.alloc_compact(st, hq, tp)
    S.search(st, q_hat, torch.full((hq,), float("-inf"), device=dev), flags=0, compact=compact, tp=tp)
    tau = S.kth_score(st, compact, torch.full((hq,), max(1, shard // 50), dtype=torch.int32, device=dev))
    if dist is not None:
        dist.broadcast(tau, 0)
    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
    n_splits = S.attn_splits(st, hq, tp)
    ws = torch.empty((hq * n_splits * (DIM + 2),), device=dev)
    out, ml = torch.empty((hq, DIM), device=dev), torch.empty((hq, 2), device=dev)
    new_k = keys_aniso(hkv, args.steps + args.warmup, 900, dev)
    new_v = torch.randn_like(new_k.float()).to(torch.bfloat16)
    merged = torch.empty((hq, DIM), device=dev)

    def step(i):
        S.search(st, q_hat, tau, scaling=lscale, flags=flags, compact=compact, tp=tp)
        S.sparse_attn(st, q_hat, lscale, compact, n_splits=n_splits, workspace=ws, out=out, out_ml=ml)
        if dist is not None:
            po, pml = gather_partials(out, ml)
            merge_gathered(po, pml, out=merged)
        if rank == world - 1:                                 # the newest token belongs to the last shard
            S.append(st, new_k[:, i:i + 1].contiguous(), new_v[:, i:i + 1].contiguous())

    for i in range(args.warmup):
        step(i)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        bytes_search = hkv * shard * DIM * 2
        print(json.dumps({"workload": "long_context_sequence_shards", "n_gpus": world, "tokens_per_gpu": shard,
                          "context": shard * world, "q_heads": hq, "kv_heads": hkv, "branching": bf, "levels": 3,
                          "dtype": "bf16", "step_us": float(t.item()) * 1e3,
                          "key_bytes_per_gpu": bytes_search,
                          "exchange_bytes_per_gpu": hq * (DIM + 2) * 4}))
    if dist is not None:
        dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m hira_b200.benchmarks")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("streaming")
    a.add_argument("--prefix", type=int, default=65536)
    a.add_argument("--steps", type=int, default=4096)
    a.add_argument("--rebuild-every", type=int, default=1024)
    a.add_argument("--final-rebuild", action="store_true")
    b = sub.add_parser("longctx")
    b.add_argument("--shard", type=int, default=131072)
    b.add_argument("--steps", type=int, default=20)
    b.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("these benchmarks need a CUDA device")
    (streaming if args.cmd == "streaming" else longctx)(args)


if __name__ == "__main__":
    main(sys.argv[1:])
