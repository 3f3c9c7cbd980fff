"""Decode-step benchmark: search + sparse attention + 1-key append per head at 128k context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload ("cfg2_b16_ctx131072", hira_b200/workloads.py): Llama-3-8B-shaped GQA decode,
batch 16, 32 query / 8 KV heads, D = 128, bf16, context 131,072; keys/values N(0,1) with RoPE
(base 500000) by position on the keys and 4 outlier channels x8; index 3 levels, branching 32;
tau per query head = the exact 2 % score, set up front.  The (batch, kv_head) groups are
independent and are dealt to the N ranks (no collective on the data path); the timed value is the
step time, max over ranks, so scaling is strong (the job is fixed).

One JSON line on stdout from rank 0:
  value       device-timed step (CUDA events, inputs resident in HBM): the K steps launched kernel by
              kernel from the host, or the same K steps each captured once into a CUDA graph and
              replayed, whichever is faster (config.launch says which; variants has both);
  e2e         the same step through the one-call host-buffer entry (HiraDecodeStep ->
              hira_decode_step): query and new key/value rows from pinned host memory, output
              back to the host, every step; median of 5 repeats of the K-step loop;
  roofline    the search kernel: algorithmic bytes (from the kernel's own counters) over its
              CUDA-event time, against the measured copy bandwidth;
  variants    the step with the threshold found on the device inside it (hira_threshold), the
              search with and without the append's parent scan folded in;
  dense_attention_us  torch SDPA over the same bf16 cache on the same GPU;
  secondary   the other configurations: cfg1 (batch 1, 32k: latency regime), cfg3 (streaming
              appends + rebuilds), cfg4 (sequence shards of 131,072 keys per GPU, the softmax
              partials exchanged and merged by one kernel over NVLink peer memory, checked against
              a one-rank recomputation);
  cpu_baseline  the reference's CPU path on a bounded sample, on this box's host cores.
`--impl reference` times the reference's CPU path: its fused_tree_search_v3 kernel (built from
the reference sources into oracle/_ref; else the oracle port) driven exactly as its CPUSearcher
drives it, on an index laid out as its CPUIndexer lays it out and updated as its `update` does
(oracle/cpu_index.py restates both; the reference's Python sources do not travel to the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch

from hira_b200 import workloads as W

DIM = W.DIM
N_QUERY_SETS = 4
E2E_REPEATS = 5
# DRAM bytes (read + write) of one search_kernel launch per (batch, kv head) group of 131,072 keys,
# from an ncu capture of this bench at --batch 2 (16 groups); traffic grows in proportion to the
# groups a launch covers.  Keyed by kernel variant; None = not captured.
SEARCH_DRAM_BYTES_PER_GROUP = {"search_kernel": (559.073280e6 + 7.247872e6) / 16,
                               "search_q8_kernel": (323.377408e6 + 4.551936e6) / 16}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
# one decode workload on this rank
# ----------------------------------------------------------------------------------
class DecodeBench:
    """Index, buffers and device loop of one decode workload on one GPU: `n_groups`
    (batch, kv head) groups of `ctx` keys each, `group` query heads per group."""

    def __init__(self, w: W.Workload, n_groups: int, ctx: int, appends: int, dev, seed_offset: int = 0,
                 use_tc: bool = True, exchange=None, int8_copy: bool = True, n_iters: int = 1, balance_rounds: int = 0):
        from hira_b200 import _lib as L
        from hira_b200 import index_state as S
        self.L, self.S, self.w, self.dev = L, S, w, dev
        self.n_groups, self.ctx, self.bf, self.group = n_groups, ctx, w.branching, w.group
        self.n_qheads = n_groups * w.group
        bf = w.branching
        t0 = time.time()
        keys, vals = W.make_kv(n_groups, ctx, 1000 + w.seed + seed_offset, dev, dist=w.dist, dtype=w.dtype)
        self.k1 = ctx // bf
        self.k2 = -(-self.k1 // bf)
        spare_gp = appends + 16   # worst case every appended key opens a new grandparent block
        self.st = st = S.IndexState(n_heads=n_groups, dim=DIM, vdim=DIM, bf=bf, depth=w.levels,
                                    cap_parents=(self.k2 + spare_gp) * bf, dtype=w.dtype, vdtype=w.dtype, device=dev,
                                    int8_copy=int8_copy)
        cent1 = W.random_centres(n_groups, ctx, self.k1, 7 + seed_offset, dev)
        cent2 = W.random_centres(n_groups, self.k1, self.k2, 8 + seed_offset, dev)
        torch.cuda.synchronize()
        t1 = time.time()
        S.build(st, keys, vals, cent_idx1=cent1, cent_idx2=cent2, n_iters=n_iters, balance_rounds=balance_rounds,
                use_tensor_cores=use_tc)
        torch.cuda.synchronize()
        self.build_s = time.time() - t1
        # threshold samples: 1000 stored key rows per head (filled slots are the first ctx of a fresh build)
        g = torch.Generator(device=dev)
        g.manual_seed(99 + seed_offset)
        pick = torch.randint(0, ctx, (1000,), generator=g, device=dev)
        self.samples = keys[:, pick].contiguous()
        del keys, vals, cent1, cent2
        torch.cuda.empty_cache()
        self.tp = S.tile_parents(st)
        self.flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
        self.compact = S.alloc_compact(st, self.n_qheads, self.tp)
        self.appended = 0
        self._bound()
        self.n_splits = S.attn_splits(st, self.n_qheads, self.tp)
        self.ws = torch.empty((self.n_qheads * self.n_splits * (DIM + 2),), dtype=torch.float32, device=dev)
        self.exchange = exchange
        if exchange is not None:
            self.out, self.out_ml = exchange.local_out, exchange.local_ml
        else:
            self.out, self.out_ml = torch.empty((self.n_qheads, DIM), dtype=torch.float32, device=dev), None
        self.sm_scale = DIM ** -0.5
        self.scan = S.new_scan_slots(st)
        self.setup_s = time.time() - t0
        self.qsets = []
        self.new_k = self.new_v = None

    def _bound(self):
        # the host's bound on the parent slots in use: every append may open one grandparent block
        self.st.active_parents = (self.k2 + self.appended) * self.bf

    def make_queries(self, n_sets: int, seed: int, tau=None):
        """Query sets (unit query, tau, logit scale, raw query); tau = exact w.keep score unless given."""
        S, L = self.S, self.L
        kk = torch.full((self.n_qheads,), max(1, int(round(self.w.keep * self.ctx))), dtype=torch.int32, device=self.dev)
        neg_inf = torch.full((self.n_qheads,), float("-inf"), device=self.dev)
        for i in range(n_sets):
            q = W.make_queries(self.n_qheads, seed + 13 * i, self.dev, pos=self.ctx + i)
            qn = q.norm(dim=-1)
            q_hat = (q / qn[:, None]).contiguous()
            if tau is None:
                S.search(self.st, q_hat, neg_inf, flags=L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES, compact=self.compact, tp=self.tp)
                t = S.kth_score(self.st, self.compact, kk).clone()
            else:
                t = tau
            self.qsets.append((q_hat, t, (qn * self.sm_scale).contiguous(), q))

    def make_new_keys(self, n: int, seed: int):
        k, v = W.make_kv(self.n_groups, n, seed, self.dev, dist=self.w.dist, dtype=self.w.dtype, first_pos=self.ctx)
        self.new_k, self.new_v = k.transpose(0, 1).contiguous(), v.transpose(0, 1).contiguous()   # (steps, groups, D)

    def counters(self):
        """Traffic counters of one search of query set 0 -> algorithmic bytes of the step."""
        S = self.S
        q_hat, tau, lscale, _ = self.qsets[0]
        stats = S.new_stats(self.n_qheads, self.dev)
        S.search(self.st, q_hat, tau, scaling=lscale, flags=self.flags, compact=self.compact, stats=stats, tp=self.tp)
        torch.cuda.synchronize()
        s = stats.to(torch.int64).sum(dim=0).tolist()
        rows_read, parents_read, emitted, reread, rows8 = s[6], s[7], s[5], s[8], s[9]
        e = 2 if self.w.dtype == torch.bfloat16 else 4
        # child rows: in the index dtype, or -- through the int8 side copy -- 128 B + 8 B of (step, error)
        # per scored row plus the candidates re-read in the index dtype
        child_bytes = rows8 * (DIM + 8) + reread * DIM * e if rows8 else rows_read * DIM * e
        self.search_kernel = "search_q8_kernel" if rows8 else "search_kernel"
        self.reread_fraction = reread / float(rows8) if rows8 else None
        search_bytes = self.n_groups * self.k2 * (DIM * e + 4) + parents_read * (DIM * e + 8) + child_bytes
        attn_bytes = emitted * (DIM * e + 8) + self.n_qheads * DIM * 4
        append_bytes = self.n_groups * ((self.k1 + self.k2) * (DIM * e + 4) + 2 * DIM * e)
        return dict(search_bytes=search_bytes, attn_bytes=attn_bytes, append_bytes=append_bytes,
                    scanned_fraction=rows_read / float(self.n_groups * self.ctx * -(-self.group // 4)),
                    selected_per_qhead=emitted / self.n_qheads)

    # ---- the step ---------------------------------------------------------------------
    def step(self, i: int, ev=None, *, fused=True, side=None, tau_in_step=False, append=True, nccl_ev=None):
        S, L, st = self.S, self.L, self.st
        q_hat, tau, lscale, _ = self.qsets[i % len(self.qsets)]
        main = torch.cuda.current_stream()
        self._bound()
        if ev:
            ev[0].record()
        if tau_in_step:
            tau = S.threshold(self.samples, q_hat, L.HIRA_TAU_SAMPLE_MEAN_TOPK, 16, out=self.tau_buf)
        j = i % self.new_k.shape[0] if self.new_k is not None else 0
        if fused and append:
            S.search(st, q_hat, tau, scaling=lscale, flags=self.flags, compact=self.compact, tp=self.tp,
                     scan_key=self.new_k[j], scan_out=self.scan)
        else:
            S.search(st, q_hat, tau, scaling=lscale, flags=self.flags, compact=self.compact, tp=self.tp)
        if ev:
            ev[1].record()

        def do_append():
            if fused:
                S.append_scanned(st, self.new_k[j].unsqueeze(1), self.new_v[j].unsqueeze(1), self.scan)
            else:
                S.append(st, self.new_k[j].unsqueeze(1), self.new_v[j].unsqueeze(1))
            self.appended += 1

        def attend():
            S.sparse_attn(st, q_hat, lscale, self.compact, n_splits=self.n_splits, workspace=self.ws, out=self.out,
                          out_ml=self.out_ml)
            if self.exchange is not None:
                if nccl_ev:
                    nccl_ev[0].record()
                self.exchange.all_gather()
                self.exchange.merge(out=self.merged)
                if nccl_ev:
                    nccl_ev[1].record()

        if not append:
            attend()
            if ev:
                ev[2].record()
            return
        if side is None:
            attend()
            if ev:
                ev[2].record()
                ev[3].record()
            do_append()
            if ev:
                ev[4].record()
            return
        # The append touches neither the compacted lists nor the value rows the attention reads, so
        # it runs beside the attention on a second stream; the next search waits for both.
        self._searched.record(main)
        with torch.cuda.stream(side):
            side.wait_event(self._searched)
            if ev:
                ev[3].record(side)
            do_append()
            if ev:
                ev[4].record(side)
            self._appended_ev.record(side)
        attend()
        if ev:
            ev[2].record()
        main.wait_event(self._appended_ev)

    def timed_loop(self, steps: int, warmup: int, barrier, first: int = 0, **kw):
        """W warm-up steps, then K timed steps between barriers; returns ms totals (this rank)."""
        self._searched, self._appended_ev = torch.cuda.Event(), torch.cuda.Event()
        self.tau_buf = torch.empty((self.n_qheads,), dtype=torch.float32, device=self.dev)
        if self.exchange is not None:
            self.merged = torch.empty((self.n_qheads, DIM), dtype=torch.float32, device=self.dev)
        for i in range(warmup):
            self.step(first + i, **kw)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
        nccl = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(steps)] if self.exchange is not None else None
        barrier()
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        host_t0 = time.time()
        t_start.record()
        for j in range(steps):
            self.step(first + warmup + j, ev[j], nccl_ev=nccl[j] if nccl else None, **kw)
        t_end.record()
        barrier()
        host_t1 = time.time()
        has_append = kw.get("append", True)
        res = dict(total_ms=t_start.elapsed_time(t_end), host=(host_t0, host_t1),
                   search_ms=statistics.mean(ev[j][0].elapsed_time(ev[j][1]) for j in range(steps)),
                   attn_ms=statistics.mean(ev[j][1].elapsed_time(ev[j][2]) for j in range(steps)),
                   append_ms=statistics.mean(ev[j][3].elapsed_time(ev[j][4]) for j in range(steps)) if has_append else 0.0)
        # every step on its own (start of step j to start of step j + 1): a single stall of the host or of a
        # peer shows up here instead of hiding in the mean
        res["step_ms_each"] = [ev[j][0].elapsed_time(ev[j + 1][0] if j + 1 < steps else t_end) for j in range(steps)]
        if nccl:
            res["exchange_ms"] = statistics.mean(nccl[j][0].elapsed_time(nccl[j][1]) for j in range(steps))
            res["exchange_ms_median"] = statistics.median(nccl[j][0].elapsed_time(nccl[j][1]) for j in range(steps))
        status = int(self.st.status.item())
        if status:
            raise RuntimeError(f"index capacity exhausted during the bench (status {status})")
        return res

    def graph_loop(self, steps: int, warmup: int, barrier, first: int = 0, **kw):
        """The same W + K steps, each captured once into a CUDA graph (its own query set and its own
        new key, the side-stream append forked and joined inside the graph) and then replayed: what a
        serving loop does when the launches, not the kernels, bound a small step.  The host's bound on
        the slots in use is set to its value after the last step before capturing (grids are frozen in
        a graph), so early steps visit a few tiles that are still empty.  Returns ms for the K steps."""
        n = warmup + steps
        self._searched, self._appended_ev = torch.cuda.Event(), torch.cuda.Event()
        saved = self.appended
        self.appended = saved + n
        self._bound()
        bound_fn, self._bound = self._bound, (lambda: None)
        graphs = []
        try:
            for i in range(n):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.step(first + i, None, **kw)
                graphs.append(g)
        finally:
            self._bound = bound_fn
        self.appended = saved                 # capturing ran nothing
        for g in graphs[:warmup]:
            g.replay()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for g in graphs[warmup:]:
            g.replay()
        t1.record()
        barrier()
        self.appended = saved + n
        self._bound()
        status = int(self.st.status.item())
        if status:
            raise RuntimeError(f"index capacity exhausted during the graph loop (status {status})")
        return t0.elapsed_time(t1)

    def time_search_only(self, reps: int, fused: bool):
        """Mean search time in us over `reps` launches (no append follows; the scan slot is reset)."""
        S = self.S
        q_hat, tau, lscale, _ = self.qsets[0]
        self._bound()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tot = 0.0
        for r in range(reps + 2):
            a.record()
            if fused:
                S.search(self.st, q_hat, tau, scaling=lscale, flags=self.flags, compact=self.compact, tp=self.tp,
                         scan_key=self.new_k[0], scan_out=self.scan)
            else:
                S.search(self.st, q_hat, tau, scaling=lscale, flags=self.flags, compact=self.compact, tp=self.tp)
            b.record()
            if fused:
                self.scan.fill_(-1)
            torch.cuda.synchronize()
            if r >= 2:
                tot += a.elapsed_time(b)
        return tot / reps * 1e3

    def time_dense(self, reps: int = 5):
        """torch SDPA over the whole cache of this rank (dense decode attention), same shapes, in ms."""
        st = self.st
        k = st.children[:, : self.ctx].unsqueeze(0)     # (1, groups, ctx, D) -- slot order is irrelevant for timing
        v = st.values[:, : self.ctx].unsqueeze(0)
        q = torch.randn((1, self.n_qheads, 1, DIM), device=self.dev, dtype=self.w.dtype)
        f = torch.nn.functional.scaled_dot_product_attention
        for _ in range(3):
            f(q, k, v, enable_gqa=True)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            f(q, k, v, enable_gqa=True)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    def snapshot(self):
        st = self.st
        names = ("parents", "parent_radii", "parent_sqnorm", "child_counts", "grand_parents", "gp_radii", "gp_sqnorm",
                 "gp_counts", "used")
        return {n: getattr(st, n).clone() for n in names if getattr(st, n) is not None}, self.appended

    def restore(self, snap):
        arrays, appended = snap
        for n, t in arrays.items():
            getattr(self.st, n).copy_(t)
        self.appended = appended


def run_e2e(b: DecodeBench, steps: int, warmup: int, barrier, serial: bool, graph: bool = False):
    """The step through the public host-buffer entry (HiraDecodeStep -> hira_decode_step): per step
    the query and the new key/value rows come from pinned host memory and the attention output
    goes back; the caller reads the result before the next token (stream synchronize per step).
    Repeated E2E_REPEATS times from the same index state; returns the per-repeat ms per step.
    graph=True: HiraDecodeStep(graph_steps=...) -- the call recorded into a CUDA graph per set of host
    buffers during the warm-up steps and replayed in the timed ones."""
    from hira_b200 import CUDAIndexer, HiraDecodeStep
    st = b.st
    idx = CUDAIndexer(b.w.levels, 1, b.bf)
    idx.state, idx.num_heads, idx.dim = st, b.n_groups, DIM
    snap = b.snapshot()
    used = st.used.max(dim=0).values.tolist()
    n_q = b.n_qheads
    side = None if serial else torch.cuda.Stream(device=b.dev)
    n_warm = max(3, warmup)
    if graph:
        n_warm = max(n_warm, len(b.qsets), 4)          # every set of host buffers is recorded before the timed steps
    step = HiraDecodeStep(idx, n_q, q_dtype=torch.float32, threshold_method="none", side_stream=side,
                          graph_steps=(steps + n_warm + 1) if graph else 0)
    if serial:
        step.side = None
    nset = len(b.qsets)
    h_q = [qs[3].cpu().pin_memory() for qs in b.qsets]                  # (n_q, D) fp32 raw queries
    h_k = b.new_k[:4].cpu().pin_memory()                                 # (4, groups, D)
    h_v = b.new_v[:4].cpu().pin_memory()
    h_out = torch.empty((n_q, DIM), dtype=torch.float32).pin_memory()
    taus = [qs[1] for qs in b.qsets]
    cur = torch.cuda.current_stream()

    def one(i):
        step(h_q[i % nset], h_out, threshold=taus[i % nset], k_host=h_k[i % 4], v_host=h_v[i % 4])
        cur.synchronize()        # the caller reads the result before the next token

    per_repeat = []
    for _ in range(E2E_REPEATS):
        b.restore(snap)
        idx._parents_bound, idx._gp_bound = int(used[0]), int(used[1])
        idx._snapshot, idx._appended = None, 0
        step._graph_left = 0                            # graph mode: record anew from this index state
        for i in range(n_warm):
            one(i)
        barrier()
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            one(i)
        e.record()
        barrier()
        per_repeat.append(a.elapsed_time(e) / steps)
    if idx.state is not st:
        raise RuntimeError("the index was reallocated during the end-to-end loop: capacity was mis-sized")
    b.restore(snap)
    h2d = h_q[0].numel() * 4 + h_k[0].numel() * 2 + h_v[0].numel() * 2
    return {"per_repeat_ms": per_repeat, "h2d": h2d, "d2h": h_out.numel() * 4}


# ----------------------------------------------------------------------------------
# secondary workloads
# ----------------------------------------------------------------------------------
def small_config_loops(args, b, steps, warm, barrier_local, snap, side):
    """The timed steps launched kernel by kernel from the host, then (from the same index state) replayed
    from CUDA graphs: below a batch of about 8 per GPU the host's launch rate, not the kernels, bounds the
    first form.  Returns (per-phase result of the first loop, its us per step, the replay's us per step or None)."""
    r = b.timed_loop(steps, warm, barrier_local, fused=True, side=side)   # small launch: the separate scan would not hide
    stream_us = r["total_ms"] / steps * 1e3
    graph_us = None
    if not args.no_graph:
        out_plain = b.out.clone()
        b.restore(snap)
        try:
            g_ms = b.graph_loop(steps, warm, barrier_local, fused=True, side=side)
            if torch.allclose(out_plain.float(), b.out.float(), rtol=1e-4, atol=1e-5):
                graph_us = g_ms / steps * 1e3
        except Exception:   # noqa: BLE001 - the stream-launch number stands
            torch.cuda.synchronize()
    return r, stream_us, graph_us


def secondary_cfg1(args, dev, barrier_local, peak):
    """Configuration 1: batch 1, 8 KV / 32 query heads, 32,768 keys: the latency regime."""
    w = W.CFG1
    steps, warm = args.steps, args.warmup
    b = DecodeBench(w, w.kv_heads, w.context, steps + warm + 8, dev, seed_offset=500, use_tc=not args.no_tc)
    b.make_queries(N_QUERY_SETS, 250)
    b.make_new_keys(steps + warm, 9100)
    c = b.counters()
    side = None if args.serial else torch.cuda.Stream(device=dev)
    snap = b.snapshot()
    r, stream_us, graph_us = small_config_loops(args, b, steps, warm, barrier_local, snap, side)
    dense_ms = b.time_dense()
    step_us = min(stream_us, graph_us) if graph_us is not None else stream_us
    ach = c["search_bytes"] / (r["search_ms"] * 1e-3) / 1e9
    # the same step behind ONE library call with host buffers (no interpreter between the launches):
    # at this size the device loop above is partly a measure of the host's launch rate
    b.restore(snap)
    e = run_e2e(b, steps, warm, barrier_local, args.serial)
    e2e_graph_us = None
    if not args.no_graph:
        try:
            b.restore(snap)
            e2e_graph_us = statistics.median(run_e2e(b, steps, warm, barrier_local, args.serial, graph=True)["per_repeat_ms"]) * 1e3
        except Exception:   # noqa: BLE001 - the plain call's number stands
            torch.cuda.synchronize()
    return {"workload": w.name, "step_us": step_us, "step_stream_launch_us": stream_us, "step_graph_replay_us": graph_us,
            "e2e_us": statistics.median(e["per_repeat_ms"]) * 1e3, "e2e_graph_replay_us": e2e_graph_us,
            "search_us": r["search_ms"] * 1e3, "sparse_attn_us": r["attn_ms"] * 1e3,
            "append_us": r["append_ms"] * 1e3, "algorithmic_bytes": c["search_bytes"] + c["attn_bytes"] + c["append_bytes"],
            "search_bytes": c["search_bytes"], "search_gbs": ach, "frac": ach / peak,
            "scanned_fraction": c["scanned_fraction"], "dense_attention_us": dense_ms * 1e3, "build_ms": b.build_s * 1e3}


def secondary_clustered(args, dev, barrier_local, peak):
    """Control: configuration 1's shape on clustered keys (1,024 tight clusters per head), index built
    with 4 Lloyd iterations and 4 capacity-aware rounds -- data on which the ball gates do prune, to
    show the step when the hierarchy has something to skip."""
    w = W.CLUSTERED
    steps, warm = args.steps, args.warmup
    b = DecodeBench(w, w.kv_heads, w.context, steps + warm + 8, dev, seed_offset=900, use_tc=not args.no_tc,
                    n_iters=4, balance_rounds=4)
    b.make_queries(N_QUERY_SETS, 350)
    b.make_new_keys(steps + warm, 9300)
    c = b.counters()
    side = None if args.serial else torch.cuda.Stream(device=dev)
    r, stream_us, graph_us = small_config_loops(args, b, steps, warm, barrier_local, b.snapshot(), side)
    ach = c["search_bytes"] / (r["search_ms"] * 1e-3) / 1e9
    return {"workload": w.name, "note": "control, not a BASELINE configuration: clustered keys, 4 Lloyd iterations, 4 balanced rounds",
            "step_us": min(stream_us, graph_us) if graph_us is not None else stream_us,
            "step_stream_launch_us": stream_us, "step_graph_replay_us": graph_us, "search_us": r["search_ms"] * 1e3, "sparse_attn_us": r["attn_ms"] * 1e3,
            "scanned_fraction": c["scanned_fraction"], "selected_per_qhead": c["selected_per_qhead"],
            "search_bytes": c["search_bytes"], "search_gbs": ach, "build_ms": b.build_s * 1e3}


def secondary_cfg3(args, dev):
    """Configuration 3: streaming index update.  Prefix 65,536 keys per head, 8 KV heads, 4,096
    single-key appends (incremental nearest-leaf assign + radius widen), full rebuild every 1,024."""
    from hira_b200 import CUDAIndexer
    from hira_b200 import index_state as S
    w = W.CFG3
    h, prefix, steps, every, bf = w.kv_heads, w.context, args.stream_steps, 1024, w.branching
    keys, vals = W.make_kv(h, prefix + steps, 1300, dev, dist=w.dist, dtype=w.dtype)
    # room for the whole stream is reserved once (as a server that knows its maximum context does), so that the
    # rebuilds reuse the index arrays instead of growing them
    ix = CUDAIndexer(3, 1, bf, max_context=prefix + steps + every + 8, reserve_worst_case=True,
                     use_tensor_cores=not args.no_tc)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ix.build(keys[None, :, :prefix], vals[None, :, :prefix])         # warm: allocations, first launches
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
        ix._n_keys = pos                      # the library was called directly: keep the indexer's host-side
        ix._parents_bound += n                # key count and worst-case bounds on the slots in use by hand
        ix._gp_bound += n
        ix.check_status()
        if pos < prefix + steps:
            e0.record()
            ix.rebuild()
            e1.record()
            torch.cuda.synchronize()
            rebuild_ms.append(e0.elapsed_time(e1))
    e = 2
    k1 = prefix // bf
    append_bytes = h * ((k1 + k1 // bf) * (DIM * e + 4) + 2 * DIM * e)
    return {"workload": w.name, "heads": h, "prefix": prefix, "appends": steps, "rebuild_every": every,
            "append_us_per_step": statistics.mean(append_us), "append_us_by_window": append_us,
            "append_algorithmic_bytes": append_bytes, "rebuild_ms": statistics.median(rebuild_ms) if rebuild_ms else None, "rebuild_ms_each": rebuild_ms,
            "rebuilds": len(rebuild_ms), "initial_build_ms": build_ms,
            "note": "append step = 8 heads, launch-latency bound (one small kernel pair per step)"}


def secondary_cfg4(args, dev, rank, world, dist, barrier, peak):
    """Configuration 4: sequence shards of 131,072 keys per GPU (context = N x 131,072), 64 query /
    8 KV heads, branching 64; every rank searches its shard with the same threshold, the softmax
    partials (m, l, out) are all-gathered over NCCL into a preallocated buffer and merged on the
    device; the append goes to the last shard.  Rank 0 then recomputes all shards alone."""
    from hira_b200 import index_state as S
    from hira_b200.parallel import PartialsExchange, PeerPartialsExchange
    w = W.CFG4
    steps, warm = args.steps, args.warmup
    # the exchange: one kernel per step over NVLink peer memory; the NCCL all-gather + merge kernel only
    # if the peers' buffers cannot be mapped on this node (every rank takes the same branch)
    ex, why = None, ""
    try:
        ex = PeerPartialsExchange(w.q_heads, DIM, dev, wait_seconds=1.0)
    except Exception as e:   # noqa: BLE001 - reported in the result line
        why = f"{type(e).__name__}: {e}"[:160]
    if dist is not None:
        okf = torch.tensor([1 if ex is not None else 0], device=dev)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if int(okf.item()) == 0 and ex is not None:
            ex.close()
            ex.free()
            ex, why = None, "a peer rank could not map the buffers"
    if ex is not None:
        exchange_kind = "one kernel per step: peer stores of the (m, l, out) rows over NVLink + flags + merge (hira_exchange_merge)"
    else:
        ex = PartialsExchange(w.q_heads, DIM, dev)
        exchange_kind = "NCCL all-gather of (m, l, out) rows into a preallocated buffer + merge kernel (peer mapping unavailable: " + why + ")"
    b = DecodeBench(w, w.kv_heads, w.context, steps + warm + 8, dev, seed_offset=700 + rank, use_tc=not args.no_tc,
                    exchange=ex)
    # the same query on every rank; one threshold for all shards: 2 % of shard 0 (identically distributed shards)
    b.make_queries(1, 333)
    tau = b.qsets[0][1]
    if dist is not None:
        dist.broadcast(tau, 0)
    b.make_new_keys(steps + warm, 9200)
    c = b.counters()
    # check step: no append, merged output kept for the one-rank recomputation
    b._searched, b._appended_ev = torch.cuda.Event(), torch.cuda.Event()
    b.merged = torch.empty((w.q_heads, DIM), dtype=torch.float32, device=dev)
    barrier()                        # the ranks enter their first exchange together (its wait is bounded)
    b.step(0, append=False)
    torch.cuda.synchronize()

    def exchange_flagged() -> bool:
        """True on every rank if on any rank a wait for a peer's rows ran out."""
        if not isinstance(b.exchange, PeerPartialsExchange):
            return False
        f = b.exchange.status.clone()
        if dist is not None:
            dist.all_reduce(f, op=dist.ReduceOp.MAX)
        return int(f.item()) != 0

    if exchange_flagged():
        # the peer route does not work on this node: every rank falls back to all-gather + merge
        barrier()
        ex.close()
        barrier()
        ex.free()
        ex = PartialsExchange(w.q_heads, DIM, dev)
        exchange_kind = ("NCCL all-gather of (m, l, out) rows into a preallocated buffer + merge kernel "
                         "(a peer's rows did not arrive within 1 s in the first step)")
        b.exchange, b.out, b.out_ml = ex, ex.local_out, ex.local_ml
        barrier()
        b.step(0, append=False)
        torch.cuda.synchronize()
    merged_dist = b.merged.clone()
    last = rank == world - 1
    fb0 = S.q8_fallback_count(dev)
    # the last shard's append runs beside its attention and exchange on a second stream
    r = b.timed_loop(steps, warm, barrier, fused=False, side=torch.cuda.Stream(dev) if last else None, append=last)
    each = r["step_ms_each"]
    t = torch.tensor([r["total_ms"], r["search_ms"], r["attn_ms"], r.get("exchange_ms", 0.0), r["append_ms"],
                      statistics.median(each), max(each), r.get("exchange_ms_median", 0.0),
                      float(S.q8_fallback_count(dev) - fb0)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, search_ms, attn_ms, exch_ms, append_ms, step_median_ms, step_max_ms, exch_median_ms, fallbacks = t.tolist()
    exchange_error = None
    if isinstance(ex, PeerPartialsExchange):
        if exchange_flagged():           # reported, never fatal for the headline
            exchange_error = "a wait for a peer's rows ran out during the timed loop: the step time is not valid"
        if dist is not None:
            dist.barrier()
        ex.close()
        if dist is not None:
            dist.barrier()
        ex.free()
    check = None
    if rank == 0:
        # one-rank recomputation: every shard's index rebuilt here in turn, same kernels, one merge
        buf = torch.zeros((world, w.q_heads, DIM + 2), dtype=torch.float32, device=dev)
        q_hat, _, lscale, _ = b.qsets[0]
        del b.st, b.compact
        torch.cuda.empty_cache()
        for r_ in range(world):
            bb = DecodeBench(w, w.kv_heads, w.context, 8, dev, seed_offset=700 + r_, use_tc=not args.no_tc)
            S.search(bb.st, q_hat, tau, scaling=lscale, flags=bb.flags, compact=bb.compact, tp=bb.tp)
            S.sparse_attn(bb.st, q_hat, lscale, bb.compact, n_splits=bb.n_splits, workspace=bb.ws,
                          out=buf[r_][:, 2:], out_ml=buf[r_][:, :2])
            torch.cuda.synchronize()
            del bb
            torch.cuda.empty_cache()
        alone = S.merge_partials(buf[:, :, 2:], buf[:, :, :2])
        check = float((alone - merged_dist).abs().max() / alone.abs().max())
    ach = c["search_bytes"] / (search_ms * 1e-3) / 1e9
    return {"workload": w.name, "n_gpus": world, "context": w.context * world, "tokens_per_gpu": w.context,
            "step_us": total_ms / steps * 1e3, "step_us_median": step_median_ms * 1e3, "step_us_max": step_max_ms * 1e3,
            "search_ctas_that_fell_back": int(fallbacks),
            "search_us": search_ms * 1e3, "sparse_attn_and_exchange_us": attn_ms * 1e3,
            "exchange_us": exch_ms * 1e3, "exchange_us_median": exch_median_ms * 1e3, "exchange_note": "max over ranks; includes waiting for the slowest rank's rows",
            "append_us_last_shard": append_ms * 1e3,
            "exchange": exchange_kind,
            "exchange_bytes_per_gpu": ex.message_bytes, "algorithmic_bytes_per_gpu": c["search_bytes"] + c["attn_bytes"],
            "search_gbs_per_gpu": ach, "frac": ach / peak, "scanned_fraction": c["scanned_fraction"],
            "merged_vs_one_rank_max_rel_err": check, **({"exchange_error": exchange_error} if exchange_error else {})}


def phase_profile(args):
    """`--phase-profile`: per-CTA phase times of the int8 pre-filter search kernel at the headline
    shape, from the profiling build of the library (`python -m hira_b200.build --profile`), whose
    kernel stamps %globaltimer at its phase boundaries.  One JSON line."""
    import ctypes as C
    import numpy as np
    from hira_b200 import _lib as L
    from hira_b200.build import PROFILE_LIB_PATH
    if not PROFILE_LIB_PATH.exists():
        raise SystemExit("build the profiling library first: python -m hira_b200.build --profile")
    L.LIB_PATH = PROFILE_LIB_PATH
    from hira_b200 import index_state as S
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    b = DecodeBench(W.CFG2, args.batch * W.CFG2.kv_heads, args.ctx, 32, dev)
    b.make_queries(1, 50)
    q_hat, tau, lscale, _ = b.qsets[0]
    for _ in range(3):
        S.search(b.st, q_hat, tau, scaling=lscale, flags=b.flags, compact=b.compact, tp=b.tp)
    torch.cuda.synchronize()
    a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    S.search(b.st, q_hat, tau, scaling=lscale, flags=b.flags, compact=b.compact, tp=b.tp)
    e.record()
    torch.cuda.synchronize()
    lib = L.load()
    buf = np.zeros((16384, 16), np.uint64)
    lib.hira_q8_profile_read.argtypes = [C.c_void_p]
    if lib.hira_q8_profile_read(buf.ctypes.data) != 0:
        raise SystemExit("reading the stamps failed")
    t = buf.astype(np.int64)
    t = t[(t[:, 0] > 0) & (t[:, 7] > 0)]
    mid = t[(t[:, 0] > np.percentile(t[:, 0], 20)) & (t[:, 0] < np.percentile(t[:, 0], 80))]   # CTAs of the steady state
    us = lambda x, y: float(((mid[:, x] - mid[:, y]) / 1e3).mean())
    out = {"workload": f"b{args.batch}_ctx{args.ctx}", "search_us": a.elapsed_time(e) * 1e3, "ctas_stamped": int(len(t)),
           "per_cta_us": {"init": us(1, 0), "gates": us(2, 1), "wait_query_terms": us(3, 2), "scores_until_last_stage": us(4, 3),
                          "candidate_list": us(5, 4), "exact_pass": us(6, 5), "compaction": us(7, 6), "total": us(7, 0)},
           "producer_us": {"start_to_first_request": us(8, 0), "first_request_to_first_stage": us(9, 8),
                           "first_to_fourth_stage": us(11, 9), "first_stage_to_last_mma": us(10, 9)}}
    print(json.dumps(out), flush=True)


def pruning_table(args):
    """Index quality against pruning power (`--pruning-table`): for the two data distributions
    (cfg0: per-channel scaled Gaussian, fp32, 4,096 keys; cfg1: RoPE + outlier channels, bf16, 32,768
    keys; 8 KV heads, one query head each, 3 levels, tau = the exact 2 % score), branching factors,
    Lloyd iterations and capacity-aware assignment rounds: the share of leaf rows the gates let
    through (from the search kernel's own counters), the mean leaf-ball radius against the
    threshold, and the search time.  One JSON line per setting."""
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rows = []
    for w in (W.CFG0, W.CFG1, W.CLUSTERED):
        keys, vals, q = W.make_inputs(w, dev)
        h, n, d = keys.shape
        q = q.view(h, w.group, d)[:, 0].contiguous()          # one query head per KV head
        q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
        sc = torch.einsum("hd,hnd->hn", q_hat, keys.float())
        tau = torch.sort(sc, dim=-1, descending=True).values[:, max(1, n // 50) - 1].contiguous()
        for bf in (8, 16, 32, 64):
            k1 = -(-n // bf)
            k2 = -(-k1 // bf)
            for iters in (1, 4, 10):
                for rounds in (0, 4):
                    st = S.IndexState(n_heads=h, dim=d, vdim=d, bf=bf, depth=3, cap_parents=k2 * bf, dtype=w.dtype,
                                      vdtype=w.dtype, device=dev)
                    S.build(st, keys, vals, cent_idx1=W.random_centres(h, n, k1, 7, dev),
                            cent_idx2=W.random_centres(h, k1, k2, 8, dev), n_iters=iters, balance_rounds=rounds,
                            use_tensor_cores=False)
                    stats = S.new_stats(h, dev)
                    flags = L.HIRA_GATE_GE | L.HIRA_LEAF_GE
                    _, compact = S.search(st, q_hat, tau, flags=flags, want_compact=True, stats=stats)
                    a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    for _ in range(3):
                        S.search(st, q_hat, tau, flags=flags, compact=compact)
                    a.record()
                    for _ in range(10):
                        S.search(st, q_hat, tau, flags=flags, compact=compact)
                    e.record()
                    torch.cuda.synchronize()
                    s = stats.to(torch.int64).sum(dim=0).tolist()
                    filled = st.child_counts > 0
                    rows.append({"data": w.name.split("_")[0], "keys": n, "bf": bf, "lloyd_iterations": iters,
                                 "balance_rounds": rounds, "scanned_fraction": s[6] / float(h * n),
                                 "parents_kept_fraction": s[3] / float(max(1, s[2])),
                                 "gp_kept_fraction": s[1] / float(max(1, s[0])),
                                 "mean_leaf_radius": float(st.parent_radii[filled].mean()),
                                 "mean_gp_radius": float(st.gp_radii[:, :k2].mean()),
                                 "tau_mean": float(tau.mean()), "selected": s[5] / float(h),
                                 "search_us": a.elapsed_time(e) * 100.0})
                    print(json.dumps(rows[-1]), flush=True)
                    del st
    return rows


# ----------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------
def run_ours(args):
    from hira_b200 import _lib as L
    w = W.CFG2
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

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    batch, ctx = args.batch, args.ctx
    # kv heads are dealt to ranks (8 heads -> 1 per GPU at 8); every rank keeps all batch items
    if w.kv_heads % world != 0:
        raise SystemExit(f"--gpus {world} must divide the {w.kv_heads} KV heads")
    n_groups = batch * (w.kv_heads // world)
    steps, warm = args.steps, args.warmup
    tau_steps, tau_warm = min(steps, 10), 3
    appends = (steps + warm) + (tau_steps + tau_warm) + 8
    b = DecodeBench(w, n_groups, ctx, appends, dev, seed_offset=rank, use_tc=not args.no_tc, int8_copy=not args.no_int8)
    b.make_queries(N_QUERY_SETS, 50 + 1000 * rank)
    b.make_new_keys(steps + warm, 9000 + rank)
    c = b.counters()
    kernel_name, reread_fraction = b.search_kernel, b.reread_fraction
    # The append's parent scan folded into the search pays with the streaming kernel (the parent rows
    # are in registers anyway); with the int8 pre-filter the gates sit on each CTA's critical path and
    # the separate scan hides beside the attention on the second stream, so it stays separate there.
    fused = args.fused if args.fused is not None else (kernel_name == "search_kernel")
    side = None if args.serial else torch.cuda.Stream(device=dev)

    snap = b.snapshot()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    r = b.timed_loop(steps, warm, barrier, fused=fused, side=side)
    # the same steps replayed from CUDA graphs (no host work between the launches)
    graph_ms, graph_err = None, None
    if not args.no_graph:
        out_plain = b.out.clone()
        b.restore(snap)
        try:
            graph_ms = b.graph_loop(steps, warm, barrier, fused=fused, side=side)
            # same selected keys; the attention's split boundaries follow the (larger, frozen) bound on the
            # tiles in use, so the partials may be summed in another order
            if not torch.allclose(out_plain.float(), b.out.float(), rtol=1e-4, atol=1e-5):
                graph_err, graph_ms = "the replayed steps' last output differs from the plain loop's", None
        except Exception as ex:   # noqa: BLE001 - reported; the plain loop's number stands
            graph_err = repr(ex)[:200]
            torch.cuda.synchronize()
    sampler.paused = True
    # the step with the threshold found on the device inside it (sample_mean_topk over 1000 stored keys)
    rt = b.timed_loop(tau_steps, tau_warm, barrier, first=steps + warm, fused=fused, side=side, tau_in_step=True)
    stats = b.S.new_stats(b.n_qheads, dev)
    b.S.search(b.st, b.qsets[0][0], b.tau_buf, scaling=b.qsets[0][2], flags=b.flags, compact=b.compact, stats=stats, tp=b.tp)
    sel_tau = float(stats[:, 5].sum().item()) / b.n_qheads
    b.restore(snap)
    search_plain_us = b.time_search_only(5, fused=False)
    search_scan_us = b.time_search_only(5, fused=True)
    dense_ms = b.time_dense() if not args.no_dense else None

    # ---- end to end through the host-buffer entry ------------------------------------------------
    e2e = run_e2e(b, steps, warm, barrier, args.serial)
    e2e_graph_ms = float("inf")           # the same entry replayed from CUDA graphs (HiraDecodeStep(graph_steps=))
    if not args.no_graph:
        try:
            e2e_graph_ms = statistics.median(run_e2e(b, steps, warm, barrier, args.serial, graph=True)["per_repeat_ms"])
        except Exception as ex:   # noqa: BLE001 - reported; the plain entry's number stands
            graph_err = (graph_err or "") + " e2e: " + repr(ex)[:160]
            torch.cuda.synchronize()
    sampler.paused = False
    if rank == 0:
        # an NVML query takes milliseconds, the timed region a few tens: run the step's search and
        # attention again (untimed; no appends) until the sampler has seen the load for a quarter of
        # a second.  Done after the timed loops so that the heat it makes reaches none of them.
        t_more = time.time()
        while time.time() - t_more < 0.25:
            for i in range(8):
                b.step(i, append=False)
            torch.cuda.synchronize()
    clocks = sampler.stop(r["host"]) if rank == 0 else None
    barrier()

    e2e_ms = statistics.median(e2e["per_repeat_ms"])
    t = torch.tensor([r["total_ms"], r["search_ms"], r["attn_ms"], r["append_ms"], e2e_ms, rt["total_ms"],
                      min(e2e["per_repeat_ms"]), max(e2e["per_repeat_ms"]), search_plain_us, search_scan_us,
                      dense_ms or 0.0, graph_ms if graph_ms is not None else float("inf"), e2e_graph_ms],
                     device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    (total_ms, search_ms, attn_ms, append_ms, e2e_ms, tau_total_ms, e2e_min, e2e_max, search_plain_us, search_scan_us,
     dense_max, graph_total_ms, e2e_graph_ms) = t.tolist()
    e2e_plain_ms = e2e_ms
    e2e_use_graph = e2e_graph_ms < e2e_ms
    if e2e_use_graph:
        e2e_ms = e2e_graph_ms
    stream_total_ms = total_ms
    use_graph = graph_total_ms != float("inf") and graph_total_ms < total_ms   # on every rank, max over ranks
    if use_graph:
        total_ms = graph_total_ms
    peak, peak_src = peaks()

    # ---- secondary workloads -------------------------------------------------------------------
    secondary = {}
    if not args.no_secondary and (batch, ctx) == (w.batch, w.context):
        del b.st, b.compact, b.ws
        b = None
        torch.cuda.empty_cache()
        if rank == 0:
            try:
                secondary["cfg1"] = secondary_cfg1(args, dev, torch.cuda.synchronize, peak)
            except Exception as ex:  # reported, never fatal for the headline
                secondary["cfg1"] = {"error": repr(ex)}
            torch.cuda.empty_cache()
            try:
                secondary["clustered"] = secondary_clustered(args, dev, torch.cuda.synchronize, peak)
            except Exception as ex:
                secondary["clustered"] = {"error": repr(ex)}
            torch.cuda.empty_cache()
            try:
                secondary["cfg3"] = secondary_cfg3(args, dev)
            except Exception as ex:
                secondary["cfg3"] = {"error": repr(ex)}
            torch.cuda.empty_cache()
        barrier()
        secondary["cfg4"] = secondary_cfg4(args, dev, rank, world, dist, barrier, peak)
        barrier()

    from hira_b200 import index_state as S_
    q8_fallbacks = S_.q8_fallback_count(dev)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    ms_per_step = total_ms / steps
    achieved = c["search_bytes"] / (search_ms * 1e-3) / 1e9
    step_bytes = c["search_bytes"] + c["attn_bytes"] + c["append_bytes"]
    cpu = cpu_baseline_sample(args) if not args.no_cpu else None
    traffic = SEARCH_DRAM_BYTES_PER_GROUP.get(args.traffic_key or kernel_name)
    line = {
        "metric": "decode_step_us", "value": ms_per_step * 1e3, "unit": "us", "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w.name if (batch, ctx) == (w.batch, w.context) else f"b{batch}_ctx{ctx}",
                   "batch": batch, "kv_heads": w.kv_heads, "q_heads": w.q_heads, "dim": DIM, "context": ctx,
                   "levels": w.levels, "branching": w.branching, "keep_frac": w.keep,
                   "tau": "exact k-th largest score per query head, set up front (variants.tau_in_step: found in the step)",
                   "sharding": f"kv_head x{world}", "l2": "inputs>L2 (keys per GPU >> 126 MB)", "gate": "ge", "leaf": "ge",
                   "step": ("search with the append's parent scan folded in" if fused else "search") + ", then sparse attention "
                           + ("followed by" if side is None else "and, beside it on a second stream,") + " the 1-key append",
                   "launch": ("each step captured once into a CUDA graph and replayed (variants.step_stream_launch_us: the "
                              "same steps launched kernel by kernel from the host; breakdown_us and roofline are from that loop)")
                             if use_graph else "kernel by kernel from the host"},
        "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "repeats": E2E_REPEATS, "min_us": e2e_min * 1e3, "max_us": e2e_max * 1e3,
                "entry": "HiraDecodeStep -> hira_decode_step (one C call per step, host buffers)"
                         + (", recorded into a CUDA graph per set of host buffers and replayed (graph_steps)" if e2e_use_graph else ""),
                "plain_call_us": e2e_plain_ms * 1e3,
                "graph_replay_us": None if e2e_graph_ms == float("inf") else e2e_graph_ms * 1e3},
        # [query terms,] search, sparse_attn (one split: no merge), [append_scan,] append
        "gpu_launches": steps * ((2 if kernel_name == "search_q8_kernel" else 1) + 1 + (1 if fused else 2)),
        "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (traffic * n_groups if (traffic and ctx == w.context) else None),
                     "algorithmic_bytes_per_launch": c["search_bytes"]},
        "breakdown_us": {"search": search_ms * 1e3, "sparse_attn": attn_ms * 1e3, "append": append_ms * 1e3},
        "variants": {"tau_in_step": {"step_us": tau_total_ms / tau_steps * 1e3, "method": "sample_mean_topk, 1000 samples, top 16",
                                     "selected_per_qhead": sel_tau, "steps": tau_steps},
                     "search_plain_us": search_plain_us, "search_with_parent_scan_us": search_scan_us,
                     "step_stream_launch_us": stream_total_ms / steps * 1e3,
                     "step_graph_replay_us": None if graph_total_ms == float("inf") else graph_total_ms / steps * 1e3,
                     **({"graph_error": graph_err} if graph_err else {})},
        "step_hbm": {"bytes": step_bytes, "achieved_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                     "frac_of_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak},
        "scanned_fraction": c["scanned_fraction"], "selected_per_qhead": c["selected_per_qhead"],
        "int8_prefilter": None if reread_fraction is None else {
            "rows_reread_in_index_dtype_fraction": reread_fraction,
            "bytes_per_child_row": (DIM + 8) + reread_fraction * DIM * 2, "extra_memory": "136 B per child slot"},
        "dense_attention_us": None if dense_ms is None else dense_max * 1e3,
        "vs_dense": None if dense_ms is None else dense_max / ms_per_step,
        "secondary": secondary, "clocks": clocks, "cpu_baseline": cpu,
        # CTAs of the pre-filter search (rank 0, whole run) whose bounded wait ran out and that took the exact fallback
        "search_ctas_that_fell_back": q8_fallbacks,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------
# CPU side: the reference's kernel (oracle/_ref) or the oracle port, on a bounded sample
# ----------------------------------------------------------------------------------
class CpuDecode:
    """One batch item of the workload on the host cores, the way the reference's CPU classes run it:
    CPUIndexer.build (k-means stand-in, see oracle/cpu_index.py), then per step
    CPUSearcher(search_strategy="fused_v3").search -- which rebuilds its level tensors and CSR
    adjacency whenever the number of keys changed, i.e. every step here (searcher/cpu.py:280-343) --
    attention over the survivors (the reference ships none: fp32 torch softmax), and
    CPUIndexer.update with the token's key (indexer/cpu.py:124-190)."""

    def __init__(self, w: W.Workload, ctx: int):
        from oracle import cpu_index as CI
        from oracle import oracle as O
        self.CI, self.O, self.w = CI, O, w
        self.ext = CI.load_reference_kernel(ROOT)
        torch.set_num_threads(os.cpu_count() or 1)
        keys, vals = W.make_kv(w.kv_heads, ctx, 4242, "cpu", dist=w.dist, dtype=w.dtype)
        self.vals = vals.float()
        self.levels = CI.build_levels(keys.float().numpy(), w.levels, w.branching, 1)
        self.group = w.group
        hq = w.kv_heads * w.group
        q = W.make_queries(hq, 99, "cpu", pos=ctx)
        qn = q.norm(dim=-1)
        self.q_hat = (q / qn[:, None]).contiguous()
        sc = torch.einsum("hgd,hnd->hgn", self.q_hat.view(w.kv_heads, w.group, DIM), keys.float()).reshape(hq, ctx)
        kth = max(1, int(round(w.keep * ctx)))
        self.tau = sc.kthvalue(ctx - kth + 1, dim=1).values.contiguous()
        self.scaling = (qn * DIM ** -0.5).contiguous()
        nk, nv = W.make_kv(w.kv_heads, 64, 4343, "cpu", dist=w.dist, dtype=w.dtype, first_pos=ctx)
        self.new_k, self.new_v = nk.float(), nv.float()
        self.i = 0
        self.kind = "reference" if self.ext is not None else "port"
        self.cores = min(hq, os.cpu_count() or 1) if self.ext is not None else min(hq, O.num_threads())

    def search(self):
        CI, O = self.CI, self.O
        prepared = CI.searcher_inputs(self.levels)          # recomputed: num_keys changed since the last step
        if self.ext is not None:
            return CI.reference_search(self.ext, self.levels, self.q_hat, self.tau, self.scaling, prepared=prepared)
        cs, rs, c2ps, sizes, offs, chs = prepared
        hq = self.q_hat.shape[0]
        q2kv = (torch.arange(hq) // self.group).numpy()
        out, _ = O.search_csr([c.numpy() for c in cs], [r.numpy() for r in rs],
                              [o.numpy() if o.numel() else None for o in offs],
                              [c.numpy() if c.numel() else None for c in chs], sizes, self.q_hat.numpy(),
                              self.tau.numpy(), scaling=self.scaling.numpy(), q2kv=q2kv)
        return torch.from_numpy(out)

    def step(self):
        dense = self.search()                                   # (hq, n) logits, 0 where not selected
        outs = []
        for qh in range(dense.shape[0]):
            sel = dense[qh].nonzero().squeeze(1)
            wgt = torch.softmax(dense[qh, sel], dim=0)
            outs.append(wgt @ self.vals[qh // self.group, sel])
        j = self.i % self.new_k.shape[1]
        self.CI.update_levels(self.levels, self.new_k[:, j:j + 1].numpy(), self.w.branching, 1)
        self.vals = torch.cat([self.vals, self.new_v[:, j:j + 1]], dim=1)
        self.i += 1
        return outs


def cpu_time_steps(args, reps: int, warm: int):
    cd = CpuDecode(W.CFG2, args.ctx)
    for _ in range(warm):
        cd.step()
    t0 = time.perf_counter()
    for _ in range(reps):
        cd.step()
    return (time.perf_counter() - t0) / reps, cd.kind, cd.cores


def cpu_baseline_sample(args):
    """Bounded CPU sample: 1 of the batch items (8 KV heads x full context); scaled to the batch."""
    w = W.CFG2
    try:
        dt, kind, cores = cpu_time_steps(args, reps=3, warm=1)
    except Exception as ex:  # the baseline is reported, never required
        return {"value": None, "unit": "us", "cores": 0, "kind": "port", "sample": f"failed: {ex!r}"}
    return {"value": dt * args.batch * 1e6, "unit": "us", "cores": cores, "kind": kind,
            "sample": f"1 of {args.batch} batch items ({w.kv_heads} kv heads x {args.ctx} keys, {w.q_heads} query heads) timed "
                      f"{dt * 1e3:.1f} ms/step over 3 steps, x{args.batch}; index and per-step update as the reference "
                      "CPUIndexer lays them out (k-means: numpy Lloyd stand-in for faiss); search = reference "
                      "fused_tree_search_v3" + ("" if kind == "reference" else " (oracle port)") +
                      " driven as its CPUSearcher drives it"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    w = W.CFG2
    reps, warm = max(1, args.steps), max(1, args.warmup)
    dt, kind, cores = cpu_time_steps(args, reps=reps, warm=warm)
    value = dt * args.batch * 1e6
    sample = (f"each step = 1 of {args.batch} batch items ({w.kv_heads} kv heads x {args.ctx} keys) on the host cores, "
              f"x{args.batch}; {reps} steps timed after {warm} warm-up steps")
    line = {
        "impl": "reference", "metric": "decode_step_us", "value": value, "unit": "us", "n_gpus": world,
        "steps": reps, "warmup": warm, "ms_per_step": value / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name if (args.batch, args.ctx) == (w.batch, w.context) else f"b{args.batch}_ctx{args.ctx}",
                   "batch": args.batch, "kv_heads": w.kv_heads, "q_heads": w.q_heads, "dim": DIM, "context": args.ctx,
                   "levels": w.levels, "branching": w.branching, "keep_frac": w.keep},
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
    ap.add_argument("--batch", type=int, default=W.CFG2.batch)
    ap.add_argument("--ctx", type=int, default=W.CFG2.context)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-tc", action="store_true", help="build the index with the CUDA-core assignment")
    ap.add_argument("--no-dense", action="store_true", help="skip timing torch SDPA over the full cache")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay of the timed steps")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (cfg1, cfg3, cfg4)")
    ap.add_argument("--stream-steps", type=int, default=4096, help="appends of the streaming workload (cfg3)")
    ap.add_argument("--serial", action="store_true", help="append after the attention on one stream instead of beside it")
    ap.add_argument("--fused", dest="fused", action="store_true", default=None,
                    help="fold the append's parent scan into the search (default with the streaming kernel)")
    ap.add_argument("--unfused", dest="fused", action="store_false",
                    help="separate parent scan in the append (default with the int8 pre-filter)")
    ap.add_argument("--no-int8", action="store_true", help="search without the int8 side copy (plain streaming kernel)")
    ap.add_argument("--phase-profile", action="store_true",
                    help="per-CTA phase times of the pre-filter search kernel (needs the profiling build), then exit")
    ap.add_argument("--pruning-table", action="store_true",
                    help="print scanned fraction against branching factor, Lloyd iterations and balanced rounds, then exit")
    ap.add_argument("--traffic-key", default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.phase_profile:
        phase_profile(args)
    elif args.pruning_table:
        pruning_table(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
