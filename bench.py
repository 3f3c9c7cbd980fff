"""Decode-step benchmark: search + sparse attention + 1-key append per head at 128k context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("cfg2_b16_ctx131072"): Llama-3-8B-shaped GQA decode, batch 16, 32 query heads /
8 KV heads, D = 128, bf16, context 131,072; keys/values N(0,1) with RoPE (base 500000)
applied to the keys by position and 4 outlier channels x8; index 3 levels, branching 32;
tau set per query head so that 2% of the keys survive (exact k-th largest score, computed
once at set-up).  The (batch, kv_head) groups are independent and are partitioned across
the N ranks (no collective on the data path); the timed value is the step time, max over
ranks, so scaling is strong (the job is fixed).

One JSON line on stdout from rank 0: `value` = device-timed step, `e2e` = the same step through
the public classes with host buffers, `roofline` = the search kernel's algorithmic bytes over its
CUDA-event time against the measured copy bandwidth, `cpu_baseline` = the CPU path on a sample.
`--impl reference` times the reference's CPU path (its fused_tree_search_v3 kernel built
from the reference sources into oracle/_ref, else the oracle port) on the host cores on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np
import torch

WORKLOAD = "cfg2_b16_ctx131072"
BATCH, H_KV, H_Q, DIM, CTX, BF, DEPTH = 16, 8, 32, 128, 131072, 32, 3
KEEP_FRAC = 0.02
ROPE_BASE = 500000.0
OUTLIER_CHANNELS = (7, 42, 71, 110)
N_QUERY_SETS = 4
# DRAM bytes (read + write) of one search_kernel launch per (batch, kv head) group of 131,072 keys, from
# an ncu capture of this bench at --batch 2 (16 groups: dram__bytes_read.sum 559.07 MB,
# dram__bytes_write.sum 7.25 MB); traffic grows in proportion to the groups a launch covers.
SEARCH_DRAM_BYTES_PER_GROUP_AT_CTX = (559.073280e6 + 7.247872e6) / 16


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------------
# synthetic data
# ----------------------------------------------------------------------------------
def rope_(x: torch.Tensor, positions: torch.Tensor):
    """Llama half-rotation RoPE, in place on (..., L, D) with positions (L,)."""
    d = x.shape[-1]
    inv = 1.0 / (ROPE_BASE ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    r1 = x1 * cos - x2 * sin
    r2 = x2 * cos + x1 * sin
    x[..., : d // 2] = r1.to(x.dtype)
    x[..., d // 2:] = r2.to(x.dtype)
    return x


def make_kv(n_groups: int, n: int, seed: int, device, first_pos: int = 0):
    """keys, values (n_groups, n, D) bf16 on `device`, generated group by group."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    keys = torch.empty((n_groups, n, DIM), dtype=torch.bfloat16, device=device)
    vals = torch.empty((n_groups, n, DIM), dtype=torch.bfloat16, device=device)
    pos = torch.arange(first_pos, first_pos + n, device=device)
    for i in range(n_groups):
        k = torch.randn((n, DIM), generator=g, device=device, dtype=torch.float32)
        rope_(k, pos)
        k[:, list(OUTLIER_CHANNELS)] *= 8.0
        keys[i] = k.to(torch.bfloat16)
        vals[i] = torch.randn((n, DIM), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    return keys, vals


def make_queries(n_qheads: int, seed: int, device, pos: int):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    q = torch.randn((n_qheads, 1, DIM), generator=g, device=device, dtype=torch.float32)
    rope_(q, torch.tensor([pos], device=device))
    return q[:, 0, :].contiguous()


# ----------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU from a thread while the timed region
    runs (NVML, read-only queries, ~1 ms period; `nvidia-smi -lms` is too coarse for a region
    of a few tens of milliseconds)."""

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples, self.times, self.reasons = [], [], set()
        self.max_mhz = None
        self._stop = False
        self.paused = False
        self._thread = None
        self._nvml = None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu_index
            if vis:
                try:
                    idx = int(vis.split(",")[self.gpu_index])
                except ValueError:
                    idx = self.gpu_index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nvml
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop:
            if self.paused:
                time.sleep(0.002)
                continue
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.times.append(time.time())
                if get_reasons:
                    r = int(get_reasons(self._h))
                    for k, bit in names.items():
                        if r & bit:
                            self.reasons.add(k)
            except Exception:
                break
            time.sleep(0.001)

    def stop(self, timed=None) -> dict:
        """`timed` = (t0, t1) host times of the timed region: the number of samples that fell
        inside it is reported beside the total (the rest were taken while the same step kept
        running right after it)."""
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0, "reasons": ["no samples (NVML unavailable)"]}
        out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
               "reasons": sorted(self.reasons)}
        if timed is not None:
            out["samples_in_timed_region"] = sum(1 for t in self.times if timed[0] <= t <= timed[1])
        return out


# ----------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------
def run_ours(args):
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200 import CUDAIndexer, CUDASearcher, hira_decode_attention
    from hira_b200.cache import CacheOutput

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (the CUDA library is the only compute path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    L.load()

    batch, ctx = args.batch, args.ctx
    total_groups = batch * H_KV
    # kv heads are dealt to ranks (8 heads -> 1 per GPU at 8); every rank keeps all batch items
    if H_KV % world != 0:
        raise SystemExit(f"--gpus {world} must divide the {H_KV} KV heads")
    kv_per_rank = H_KV // world
    n_groups = batch * kv_per_rank
    group = H_Q // H_KV
    n_qheads = n_groups * group
    steps_total = args.steps + args.warmup
    spare_gp = 2 * steps_total + 16   # worst case every appended key opens a new grandparent block

    t_setup = time.time()
    keys, vals = make_kv(n_groups, ctx, seed=1000 + rank, device=dev)
    k1 = ctx // BF
    k2 = -(-k1 // BF)
    st = S.IndexState(n_heads=n_groups, dim=DIM, vdim=DIM, bf=BF, depth=DEPTH, cap_parents=(k2 + spare_gp) * BF,
                      dtype=torch.bfloat16, vdtype=torch.bfloat16, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(7 + rank)
    cent1 = torch.rand((n_groups, ctx), generator=g, device=dev).topk(k1, dim=1).indices.to(torch.int32).contiguous()
    cent2 = torch.rand((n_groups, k1), generator=g, device=dev).topk(k2, dim=1).indices.to(torch.int32).contiguous()
    torch.cuda.synchronize()
    t0 = time.time()
    S.build(st, keys, vals, cent_idx1=cent1, cent_idx2=cent2, n_iters=1, use_tensor_cores=not args.no_tc)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    del keys, vals, cent1, cent2
    torch.cuda.empty_cache()

    tp = S.tile_parents(st)
    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
    compact = S.alloc_compact(st, n_qheads, tp)
    n_splits = S.attn_splits(st, n_qheads, tp)
    ws = torch.empty((n_qheads * n_splits * (DIM + 2),), dtype=torch.float32, device=dev)
    out = torch.empty((n_qheads, DIM), dtype=torch.float32, device=dev)

    # query sets with their exact 2% thresholds (set-up, not timed)
    sm_scale = DIM ** -0.5
    qsets = []
    kk = torch.full((n_qheads,), max(1, int(round(KEEP_FRAC * ctx))), dtype=torch.int32, device=dev)
    neg_inf = torch.full((n_qheads,), float("-inf"), device=dev)
    for i in range(N_QUERY_SETS):
        q = make_queries(n_qheads, seed=50 + 13 * i + 1000 * rank, device=dev, pos=ctx + i)
        qn = q.norm(dim=-1)
        q_hat = (q / qn[:, None]).contiguous()
        S.search(st, q_hat, neg_inf, flags=L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES, compact=compact, tp=tp)
        tau = S.kth_score(st, compact, kk)
        qsets.append((q_hat, tau.clone(), (qn * sm_scale).contiguous(), q))
    new_k, new_v = make_kv(n_groups, steps_total, seed=9000 + rank, device=dev, first_pos=ctx)
    new_k = new_k.transpose(0, 1).contiguous()   # (steps, groups, D)
    new_v = new_v.transpose(0, 1).contiguous()

    # traffic counters of one search (for the roofline numerator)
    stats = torch.zeros((n_qheads, 8), dtype=torch.int32, device=dev)
    S.search(st, qsets[0][0], qsets[0][1], scaling=qsets[0][2], flags=flags, compact=compact, stats=stats, tp=tp)
    torch.cuda.synchronize()
    s = stats.to(torch.int64).sum(dim=0).tolist()
    rows_read, parents_read, emitted = s[6], s[7], s[5]
    n_gp_rows = n_groups * k2
    e = 2
    search_bytes = n_gp_rows * (DIM * e + 4) + parents_read * (DIM * e + 4 + 4) + rows_read * DIM * e
    attn_bytes = emitted * (DIM * e + 8) + n_qheads * DIM * 4
    append_bytes = n_groups * ((k1 + k2) * (DIM * e + 4) + 2 * DIM * e)
    scanned_frac = rows_read / float(n_groups * ctx)
    setup_s = time.time() - t_setup

    # fused: the search scores the parent rows it reads against the key appended right after, so
    # the append needs no parent scan of its own.  With the append running beside the attention
    # (below) the separate scan is mostly hidden anyway: at batch 16 both ways take the same time,
    # at the per-GPU share of an 8-GPU run the fused one is 4 % faster (--unfused switches back).
    fused = not args.unfused
    scan = S.new_scan_slots(st)

    def search_step(i, q_hat, tau, lscale):
        if fused:
            S.search(st, q_hat, tau, scaling=lscale, flags=flags, compact=compact, tp=tp, scan_key=new_k[i], scan_out=scan)
        else:
            S.search(st, q_hat, tau, scaling=lscale, flags=flags, compact=compact, tp=tp)

    def append_step(i):
        if fused:
            S.append_scanned(st, new_k[i].unsqueeze(1), new_v[i].unsqueeze(1), scan)
        else:
            S.append(st, new_k[i].unsqueeze(1), new_v[i].unsqueeze(1))

    # The append touches neither the compacted lists nor the value rows the attention reads, so
    # it runs beside the attention on a second stream; the next search waits for both.
    side = None if args.serial else torch.cuda.Stream(device=dev)

    def step(i: int, ev=None):
        q_hat, tau, lscale, _ = qsets[i % N_QUERY_SETS]
        main = torch.cuda.current_stream()
        if ev:
            ev[0].record()
        search_step(i, q_hat, tau, lscale)
        if ev:
            ev[1].record()
        if side is None:
            S.sparse_attn(st, q_hat, lscale, compact, n_splits=n_splits, workspace=ws, out=out)
            if ev:
                ev[2].record()
                ev[3].record()
            append_step(i)
            if ev:
                ev[4].record()
            return
        searched = torch.cuda.Event()
        searched.record(main)
        with torch.cuda.stream(side):
            side.wait_event(searched)
            if ev:
                ev[3].record(side)
            append_step(i)
            if ev:
                ev[4].record(side)
            appended = torch.cuda.Event()
            appended.record(side)
        S.sparse_attn(st, q_hat, lscale, compact, n_splits=n_splits, workspace=ws, out=out)
        if ev:
            ev[2].record()
        main.wait_event(appended)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    host_t0 = time.time()
    t_start.record()
    for j in range(args.steps):
        step(args.warmup + j, ev[j])
    t_end.record()
    barrier()
    host_t1 = time.time()
    total_ms = t_start.elapsed_time(t_end)
    search_ms = statistics.mean(ev[j][0].elapsed_time(ev[j][1]) for j in range(args.steps))
    attn_ms = statistics.mean(ev[j][1].elapsed_time(ev[j][2]) for j in range(args.steps))
    append_ms = statistics.mean(ev[j][3].elapsed_time(ev[j][4]) for j in range(args.steps))
    status = int(st.status.item())
    if status:
        raise RuntimeError(f"index capacity exhausted during the bench (status {status})")

    # dense attention over the full cache on the same shapes (torch SDPA), for context
    dense_ms = None
    if args.dense and rank == 0:
        dense_ms = time_dense(st, n_groups, group, ctx, dev)

    # ---- end to end through the public API with host buffers ----------------------------
    sampler.paused = True        # the end-to-end loop is host-latency sensitive: no sampling thread beside it
    e2e = run_e2e(args, st, qsets, n_groups, group, k2, dev, CUDAIndexer, CUDASearcher, CacheOutput,
                  hira_decode_attention, barrier, new_k, new_v)
    sampler.paused = False
    if rank == 0:
        # an NVML query takes milliseconds, the timed region a few tens: run the step's search and
        # attention again (untimed; no appends, so the index does not grow) until the sampler has
        # seen the load for a quarter of a second.  Done last so that the heat it makes reaches no
        # timed loop.
        t_more = time.time()
        while time.time() - t_more < 0.25:
            for i in range(8):
                q_hat, tau, lscale, _ = qsets[i % N_QUERY_SETS]
                S.search(st, q_hat, tau, scaling=lscale, flags=flags, compact=compact, tp=tp)
                S.sparse_attn(st, q_hat, lscale, compact, n_splits=n_splits, workspace=ws, out=out)
            torch.cuda.synchronize()
    clocks = sampler.stop((host_t0, host_t1)) if rank == 0 else None
    barrier()

    t = torch.tensor([total_ms, search_ms, attn_ms, append_ms, e2e["ms_per_step"]], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, search_ms, attn_ms, append_ms, e2e_ms = t.tolist()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    ms_per_step = total_ms / args.steps
    peak, peak_src = peaks()
    achieved = search_bytes / (search_ms * 1e-3) / 1e9
    step_bytes = search_bytes + attn_bytes + append_bytes
    cpu = cpu_baseline_sample(args) if (world == 1 or rank == 0) and not args.no_cpu else None
    line = {
        "metric": "decode_step_us", "value": ms_per_step * 1e3, "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD if (batch, ctx) == (BATCH, CTX) else f"b{batch}_ctx{ctx}",
                   "batch": batch, "kv_heads": H_KV, "q_heads": H_Q, "dim": DIM, "context": ctx, "levels": DEPTH,
                   "branching": BF, "keep_frac": KEEP_FRAC, "tau": "exact k-th largest score per query head, set up front",
                   "sharding": f"kv_head x{world}", "l2": "inputs>L2 (keys per GPU >> 126 MB)",
                   "gate": "ge", "leaf": "ge",
                   "step": ("search with the append's parent scan folded in" if fused else "search") + ", then sparse attention "
                           + ("followed by" if side is None else "and, beside it on a second stream,") + " the 1-key append"},
        "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": args.steps * (1 + (1 if n_splits == 1 else 2) + (1 if fused else 2)),   # search, sparse_attn[, merge][, append_scan], append
        "roofline": {"bound": "hbm", "kernel": "search_kernel", "achieved": achieved, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (SEARCH_DRAM_BYTES_PER_GROUP_AT_CTX * n_groups if ctx == CTX else None),
                     "algorithmic_bytes_per_launch": search_bytes},
        "breakdown_us": {"search": search_ms * 1e3, "sparse_attn": attn_ms * 1e3, "append": append_ms * 1e3},
        "step_hbm": {"bytes": step_bytes, "achieved_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                     "frac_of_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak},
        "scanned_fraction": scanned_frac, "selected_per_qhead": emitted / n_qheads,
        "dense_attention_us": None if dense_ms is None else dense_ms * 1e3,
        "build_s": build_s, "setup_s": setup_s, "clocks": clocks, "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def time_dense(st, n_groups, group, ctx, dev):
    """torch SDPA over the whole bf16 cache (dense decode attention), same shapes."""
    k = st.children[:, :ctx].unsqueeze(0)            # (1, groups, ctx, D) -- slot order is irrelevant for timing
    v = st.values[:, :ctx].unsqueeze(0)
    q = torch.randn((1, n_groups * group, 1, DIM), device=dev, dtype=torch.bfloat16)
    f = torch.nn.functional.scaled_dot_product_attention
    for _ in range(3):
        f(q, k, v, enable_gqa=True)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        f(q, k, v, enable_gqa=True)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / 5


def run_e2e(args, st, qsets, n_groups, group, k2, dev, CUDAIndexer, CUDASearcher, CacheOutput,
            hira_decode_attention, barrier, new_k, new_v):
    """The same step through the public classes, with host buffers: per step the query and
    the new key/value rows come from pinned host memory and the attention output goes back."""
    idx = CUDAIndexer(DEPTH, 1, BF)
    idx.state, idx.num_heads, idx.dim = st, n_groups, DIM
    used = st.used.max(dim=0).values.tolist()        # capacity was pre-allocated: start the host bounds here
    idx._parents_bound, idx._gp_bound = int(used[0]), int(used[1])
    searcher = CUDASearcher(BF)
    n_q = n_groups * group
    steps = args.steps
    nset = len(qsets)
    h_q = [qs[3].reshape(1, n_q, 1, DIM).cpu().pin_memory() for qs in qsets]       # fp32 queries
    h_k = new_k[: 4].reshape(4, 1, n_groups, 1, DIM).cpu().pin_memory()
    h_v = new_v[: 4].reshape(4, 1, n_groups, 1, DIM).cpu().pin_memory()
    h_out = torch.empty((1, n_q, 1, DIM), dtype=torch.float32).pin_memory()
    empty = torch.empty((1, n_groups, 0, DIM), dtype=torch.bfloat16, device=dev)
    co = CacheOutput(queued_keys=empty, queued_values=empty, prefill_keys=None, prefill_values=None, indexer=idx,
                     searcher=searcher)
    taus = [qs[1] for qs in qsets]

    side = None if args.serial else torch.cuda.Stream(device=dev)

    def one(i):
        q = h_q[i % nset].to(dev, non_blocking=True)
        if side is not None:
            # the new key / value rows are copied and appended on a second stream, beside the
            # attention; the append starts when the step's search has finished
            o = hira_decode_attention(q, co, threshold=taus[i % nset])
            with torch.cuda.stream(side):
                k = h_k[i % 4].to(dev, non_blocking=True)
                v = h_v[i % 4].to(dev, non_blocking=True)
            idx.update(k, v, stream=side)
            h_out.copy_(o, non_blocking=True)
            idx.wait_pending_update()                   # the step ends when the append has landed too
            return
        # (the scan folded into the search, `append_key=` / `update(scanned=True)`, would put the
        # key's copy in front of the search: through host buffers the plain order is faster)
        o = hira_decode_attention(q, co, threshold=taus[i % nset])
        k = h_k[i % 4].to(dev, non_blocking=True)       # queued behind the attention: not on its critical path
        v = h_v[i % 4].to(dev, non_blocking=True)
        idx.update(k, v)
        h_out.copy_(o, non_blocking=True)

    for i in range(max(3, args.warmup)):
        one(i)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        one(i)
        torch.cuda.current_stream().synchronize()   # the caller reads the result before the next token
    b.record()
    barrier()
    if idx.state is not st:
        raise RuntimeError("the index was reallocated during the end-to-end loop: capacity was mis-sized")
    h2d = h_q[0].numel() * 4 + h_k[0].numel() * 2 + h_v[0].numel() * 2
    return {"ms_per_step": a.elapsed_time(b) / steps, "h2d": h2d, "d2h": h_out.numel() * 4}


# ----------------------------------------------------------------------------------
# CPU side: the reference's kernel (oracle/_ref) or the oracle port, on a bounded sample
# ----------------------------------------------------------------------------------
def load_ref_ext():
    so = ROOT / "oracle" / "_ref" / "hira_torch_ext_v3.so"
    if not so.exists():
        return None
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location("hira_torch_ext_v3", str(so))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        return m
    except Exception:
        return None


def cpu_sample_index(n_kv: int, ctx: int, seed: int):
    """CPU-format index (the reference CPUIndexer's levels, indexer/cpu.py:48-122) for `n_kv`
    heads of the workload: level sizes ctx, ctx/bf, ctx/bf^2; one Lloyd pass from random
    centres stands in for faiss.Kmeans (not installed); radii by the triangle inequality
    (indexer/cpu.py:263-311).  numpy/BLAS, set-up only."""
    g = torch.Generator().manual_seed(seed)
    pos = torch.arange(ctx)
    keys = torch.randn((n_kv, ctx, DIM), generator=g)
    for h in range(n_kv):
        rope_(keys[h], pos)
    keys[..., list(OUTLIER_CHANNELS)] *= 8.0
    keys = keys.to(torch.bfloat16).float()
    vals = torch.randn((n_kv, ctx, DIM), generator=g).to(torch.bfloat16).float()
    centers, radii, c2p, sizes = [keys], [torch.zeros((n_kv, ctx))], [], [ctx]
    size = ctx
    for _ in range(DEPTH - 1):
        size = size // BF
        child = centers[-1]
        n_child = child.shape[1]
        cent = torch.empty((n_kv, size, DIM))
        assign = torch.empty((n_kv, n_child), dtype=torch.long)
        for h in range(n_kv):
            init = child[h][torch.randperm(n_child, generator=g)[:size]]
            a = torch.cdist(child[h], init).argmin(dim=1)
            sums = torch.zeros((size, DIM)).index_add_(0, a, child[h])
            cnt = torch.bincount(a, minlength=size).clamp_min(1).float()[:, None]
            c = torch.where(torch.bincount(a, minlength=size)[:, None] > 0, sums / cnt, init)
            cent[h] = c
            assign[h] = torch.cdist(child[h], c).argmin(dim=1)
        parent_for_child = cent.gather(1, assign.unsqueeze(-1).expand(-1, -1, DIM))
        contrib = (child - parent_for_child).norm(dim=-1) + radii[-1]
        r = torch.full((n_kv, size), float("-inf")).scatter_reduce_(1, assign, contrib, reduce="amax", include_self=True)
        centers.append(cent)
        radii.append(r)
        c2p.append(assign)
        sizes.append(size)
    # CSR adjacency as CPUSearcher builds it (searcher/cpu.py:345-363)
    offsets, children = [], []
    for l in range(DEPTH - 1):
        P = sizes[l + 1]
        off = torch.empty((n_kv, P + 1), dtype=torch.long)
        ch = torch.empty((n_kv, sizes[l]), dtype=torch.long)
        for h in range(n_kv):
            order = torch.argsort(c2p[l][h])
            off[h, 0] = 0
            off[h, 1:] = torch.bincount(c2p[l][h], minlength=P).cumsum(0)
            ch[h] = order
        offsets.append(off)
        children.append(ch)
    offsets.append(torch.empty(0, dtype=torch.long))
    children.append(torch.empty(0, dtype=torch.long))
    c2p.append(torch.empty(0, dtype=torch.long))
    return dict(keys=keys, vals=vals, centers=centers, radii=radii, c2p=c2p, sizes=sizes, offsets=offsets,
                children=children)


def cpu_step_timer(n_kv: int, ctx: int, reps: int, warm: int):
    """Times one decode step (search + attention over survivors + 1-key append) of the CPU
    path for `n_kv` KV heads x (H_Q/H_KV) query heads each.  Returns (seconds per step, kind, cores)."""
    from oracle import oracle as O
    ext = load_ref_ext()
    torch.set_num_threads(os.cpu_count() or 1)
    ix = cpu_sample_index(n_kv, ctx, seed=4242)
    group = H_Q // H_KV
    hq = n_kv * group
    g = torch.Generator().manual_seed(99)
    q = torch.randn((hq, DIM), generator=g)
    qn = q.norm(dim=-1)
    q_hat = (q / qn[:, None]).contiguous()
    keys = ix["keys"]
    sc = torch.einsum("hgd,hnd->hgn", q_hat.view(n_kv, group, DIM), keys).reshape(hq, ctx)
    kth = max(1, int(round(KEEP_FRAC * ctx)))
    tau = sc.kthvalue(ctx - kth + 1, dim=1).values.contiguous()
    scaling = (qn * DIM ** -0.5).contiguous()
    q2kv = torch.arange(hq) // group
    vals = ix["vals"]
    new_k = torch.randn((n_kv, 1, DIM), generator=g)
    state = {"keys": keys, "vals": vals}

    def search():
        if ext is not None:
            return ext.fused_tree_search_v3(state["keys"], q_hat, tau, ix["centers"],
                                            ix["radii"], ix["c2p"], ix["sizes"], ix["offsets"], ix["children"],
                                            q2kv, scaling)
        out, _ = O.search_csr([c.numpy() for c in ix["centers"]], [r.numpy() for r in ix["radii"]],
                              [o.numpy() if o.numel() else None for o in ix["offsets"]],
                              [c.numpy() if c.numel() else None for c in ix["children"]], ix["sizes"],
                              q_hat.numpy(), tau.numpy(), scaling=scaling.numpy(), q2kv=q2kv.numpy())
        return torch.from_numpy(out)

    def one():
        dense = search()                                   # (hq, ctx) logits, 0 where not selected
        outs = []
        for qh in range(hq):                               # attention over the survivors (the reference has none)
            sel = dense[qh].nonzero().squeeze(1)
            w = torch.softmax(dense[qh, sel], dim=0)
            outs.append(w @ state["vals"][qh // group, sel])
        # append as CPUIndexer.update does for one key: concatenate onto every level (indexer/cpu.py:158-181)
        k_cat = torch.cat([state["keys"], new_k], dim=1)
        v_cat = torch.cat([state["vals"], new_k], dim=1)
        del k_cat, v_cat                                   # not kept: the next step searches the same index
        return outs

    for _ in range(warm):
        one()
    t0 = time.perf_counter()
    for _ in range(reps):
        one()
    dt = (time.perf_counter() - t0) / reps
    cores = min(hq, os.cpu_count() or 1) if ext is not None else min(hq, O.num_threads())
    return dt, ("reference" if ext is not None else "port"), cores


def cpu_baseline_sample(args):
    """Bounded CPU sample: 1 of the batch items (8 KV heads x full context); scaled to the batch."""
    try:
        dt, kind, cores = cpu_step_timer(H_KV, args.ctx, reps=3, warm=1)
    except Exception as ex:  # the baseline is reported, never required
        return {"value": None, "unit": "us", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
    return {"value": dt * args.batch * 1e6, "unit": "us", "cores": cores, "kind": kind,
            "sample": f"1 of {args.batch} batch items ({H_KV} kv heads x {args.ctx} keys, {H_Q} query heads) timed "
                      f"{dt * 1e3:.1f} ms/step, x{args.batch}; index = numpy Lloyd stand-in for faiss k-means; "
                      "search = reference fused_tree_search_v3" + ("" if kind == "reference" else " (oracle port)")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    reps = max(1, args.steps)
    warm = max(1, min(args.warmup, 2))
    reps = min(reps, 5)
    dt, kind, cores = cpu_step_timer(H_KV, args.ctx, reps=reps, warm=warm)
    value = dt * args.batch * 1e6
    sample = (f"each step = 1 of {args.batch} batch items ({H_KV} kv heads x {args.ctx} keys) on the host cores, "
              f"x{args.batch}; {reps} steps timed")
    line = {
        "impl": "reference", "metric": "decode_step_us", "value": value, "unit": "us", "n_gpus": world,
        "steps": reps, "warmup": warm, "ms_per_step": value / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD if (args.batch, args.ctx) == (BATCH, CTX) else f"b{args.batch}_ctx{args.ctx}",
                   "batch": args.batch, "kv_heads": H_KV, "q_heads": H_Q, "dim": DIM, "context": args.ctx,
                   "levels": DEPTH, "branching": BF, "keep_frac": KEEP_FRAC},
        "cpu_baseline": {"value": value, "unit": "us", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-tc", action="store_true", help="build the index with the CUDA-core assignment")
    ap.add_argument("--dense", action="store_true", help="also time torch SDPA over the full cache")
    ap.add_argument("--serial", action="store_true", help="append after the attention on one stream instead of beside it")
    ap.add_argument("--unfused", action="store_true",
                    help="separate parent scan in the append instead of the scan folded into the search")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
