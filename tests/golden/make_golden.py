"""Generates tests/golden/*.npz from the REFERENCE's own code, run on CPU.

Run where the reference checkout exists (it is not needed to run the tests):

    cd /tmp && python -O /path/to/repo/tests/golden/make_golden.py [--ref /path/to/reference]

What runs, and how it runs without a GPU and without faiss:
  * `python -O` strips the `assert x.is_cuda` lines of indexer/cuda.py, so CUDAIndexer's
    radius routines and its `update` run on CPU tensors;
  * TRITON_INTERPRET=1 makes the reference's Triton kernels (search filters, nearest-L2,
    slot fill, radius max) run in the Triton interpreter on CPU tensors;
  * the reference's fused_tree_search_v3 is the binary built from its source by
    oracle/Makefile (`make ref`); the JIT loader module is replaced by a stub holding it;
  * `faiss` is a numpy Lloyd stand-in (only CPUIndexer uses it; the k-means arithmetic
    is therefore not the reference's, the index it yields is simply "an index").
Inputs are seeded; the initial blocked indexes are laid out by the oracle's build (any
valid blocked index would do: the reference routines only see tensors).
"""
import argparse
import importlib.util
import os
import sys
import tempfile
import types
from pathlib import Path

if "--gpu" not in sys.argv:
    os.environ["TRITON_INTERPRET"] = "1"

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]

# `faiss` for the reference's CPUIndexer: the Lloyd stand-in of oracle/cpu_index.py, so that the
# restatement of CPUIndexer there can be pinned against the reference running the same k-means
FAISS_SHIM = "from oracle.cpu_index import LloydKmeans as Kmeans\n"


def setup_reference(ref: Path):
    if __debug__:
        raise SystemExit("run with `python -O` (the reference asserts .is_cuda on its tensors)")
    tmp = Path(tempfile.mkdtemp(prefix="hira_ref_"))
    (tmp / "shim").mkdir()
    (tmp / "shim" / "faiss.py").write_text(FAISS_SHIM)
    os.symlink(ref, tmp / "hira")
    sys.path[:0] = [str(tmp / "shim"), str(tmp), str(ROOT)]
    so = ROOT / "oracle" / "_ref" / "hira_torch_ext_v3.so"
    if not so.exists():
        raise SystemExit("build the reference kernels first: make -C oracle ref")
    spec = importlib.util.spec_from_file_location("hira_torch_ext_v3", str(so))
    v3 = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(v3)
    stub = types.ModuleType("hira.kernels.cpp.torch_ext_loader")
    stub.hira_torch_ext = stub.hira_torch_ext_v2 = stub.hira_torch_ext_v4 = None
    stub.hira_torch_ext_v3 = v3
    sys.modules["hira.kernels.cpp.torch_ext_loader"] = stub


def unit(rng, shape):
    import numpy as np
    x = rng.standard_normal(shape).astype(np.float32)
    return x / np.linalg.norm(x, axis=-1, keepdims=True)


def ref_indexer_from(ox, depth, bf):
    """A reference CUDAIndexer holding the arrays of an oracle-built index (CPU tensors)."""
    import torch
    from hira.indexer.cuda import CUDAIndexer
    ref = CUDAIndexer(depth, 1, bf)
    ref.dim, ref.num_heads = ox.dim, ox.n_heads
    up, ug = int(ox.used[0, 0]), int(ox.used[0, 1])
    ref.parents = torch.from_numpy(ox.parents[:, :up].copy())
    ref.children = torch.from_numpy(ox.children[:, :up * bf].copy())
    ref.values = torch.from_numpy(ox.values[:, :up * bf].copy()).unsqueeze(0)
    ref.parent_radii = torch.from_numpy(ox.parent_radii[:, :up].copy())
    if depth == 3:
        ref.grand_parents = torch.from_numpy(ox.grand_parents[:, :ug].copy())
        ref.grand_parent_radii = torch.from_numpy(ox.gp_radii[:, :ug].copy())
    return ref


def initial_arrays(ox):
    return {f"ix_{k}": v for k, v in ox.arrays().items() if k != "meta" and v is not None}


def gen_append_and_radii(out: Path):
    import numpy as np
    import torch
    from oracle import oracle as O
    # depth 3 with one head: with several heads the reference pads every head to the same
    # number of grandparent blocks and its nearest-grandparent search then sees those
    # all-zero pad rows as candidates (indexer/cuda.py:918-920) -- an artefact of the batched
    # tensor shapes that this build does not reproduce (blocks are per head here).
    for seed, (name, H, n, D, bf, depth, m) in enumerate((("append_l2", 2, 96, 32, 4, 2, 8),
                                                          ("append_l3", 1, 160, 32, 4, 3, 10),
                                                          ("append_l2_free", 2, 90, 64, 8, 2, 8))):
        rng = np.random.default_rng(100 + seed)
        keys, vals = unit(rng, (H, n, D)), rng.standard_normal((H, n, D)).astype(np.float32)
        k1 = -(-n // bf)
        ox = O.OracleIndex(n_heads=H, dim=D, vdim=D, bf=bf, depth=depth, cap_parents=k1 + 64)
        O.build(ox, keys, vals)
        ref = ref_indexer_from(ox, depth, bf)
        rec = dict(initial_arrays(ox), H=H, n=n, D=D, bf=bf, depth=depth, cap_parents=ox.cap_parents)
        rec["radii_parent_from_layout"] = ref._compute_parent_radii_from_layout().numpy()
        if depth == 3:
            rec["radii_gp_from_layout"] = ref._compute_grandparent_radii_from_layout().numpy()
        ref._init_update_state()
        rec["init_child_counts"] = ref._child_counts.numpy().copy()
        new_k, new_v = unit(rng, (H, m, D)), rng.standard_normal((H, m, D)).astype(np.float32)
        for i in range(m):   # one key per call: the deterministic case of the reference's update
            ref.update(torch.from_numpy(new_k[:, i:i + 1]).unsqueeze(0), torch.from_numpy(new_v[:, i:i + 1]).unsqueeze(0))
        rec.update(new_k=new_k, new_v=new_v, after_children=ref.children.numpy(),
                   after_values=ref.values.squeeze(0).numpy(), after_parents=ref.parents.numpy(),
                   after_parent_radii=ref.parent_radii.numpy(), after_child_counts=ref._child_counts.numpy())
        if depth == 3:
            rec.update(after_gps=ref.grand_parents.numpy(), after_gp_radii=ref.grand_parent_radii.numpy(),
                       after_gp_counts=ref._gp_child_counts.numpy())
        np.savez_compressed(out / f"{name}.npz", **rec)
        print("wrote", name)


def gen_triton_search(out: Path):
    import numpy as np
    import torch
    from hira.kernels.triton_search_kernels import (three_level_filter_kernel_v1_batched,
                                                    two_level_filter_kernel_batched)
    from oracle import oracle as O
    for name, H, G, n, D, bf, depth in (("search_triton_l2", 2, 2, 256, 32, 8, 2), ("search_triton_l3", 2, 2, 512, 64, 8, 3)):
        rng = np.random.default_rng(7 + depth)
        keys, vals = unit(rng, (H, n, D)), rng.standard_normal((H, n, D)).astype(np.float32)
        k1 = n // bf
        ox = O.OracleIndex(n_heads=H, dim=D, vdim=D, bf=bf, depth=depth, cap_parents=k1)
        O.build(ox, keys, vals)
        hq = H * G
        q = unit(rng, (hq, D))
        q2kv = np.repeat(np.arange(H), G).astype(np.int64)
        # thresholds with a guard band: no gate value q.c + r within 1e-3 of tau
        gate_vals = []
        for qh in range(hq):
            h = q2kv[qh]
            gate_vals.append(np.concatenate([ox.parents[h] @ q[qh] + ox.parent_radii[h]] +
                                            ([ox.grand_parents[h] @ q[qh] + ox.gp_radii[h]] if depth == 3 else [])))
        tau = np.zeros(hq, np.float32)
        for qh in range(hq):
            gv = np.sort(gate_vals[qh])
            gaps = np.diff(gv)
            lo = len(gv) // 3
            j = lo + int(np.argmax(gaps[lo:2 * lo + 1]))          # a wide gap in the middle third: some nodes pruned
            tau[qh] = 0.5 * (gv[j] + gv[j + 1])
            assert gaps[j] > 2e-3, gaps[j]
        scaling = rng.uniform(0.5, 2.0, hq).astype(np.float32)
        K, P, R = torch.from_numpy(ox.children), torch.from_numpy(ox.parents), torch.from_numpy(ox.parent_radii)
        qt, tt, st = torch.from_numpy(q), torch.from_numpy(tau), torch.from_numpy(scaling)
        m = torch.from_numpy(q2kv)
        outt = torch.zeros((hq, n), dtype=torch.float32)
        if depth == 2:
            two_level_filter_kernel_batched[(k1, hq)](
                K_ptr=K, P_ptr=P, R_ptr=R, q_ptr=qt, q_head_to_kv_ptr=m, out_ptr=outt, t_ptr=tt, scaling_ptr=st,
                K_h_stride=K.stride(0), K_row_stride=K.stride(1), P_h_stride=P.stride(0), P_row_stride=P.stride(1),
                R_h_stride=R.stride(0), R_row_stride=R.stride(1), q_h_stride=qt.stride(0), q_d_stride=qt.stride(1),
                out_h_stride=outt.stride(0), out_row_stride=outt.stride(1), t_h_stride=tt.stride(0),
                scaling_h_stride=st.stride(0), q2kv_h_stride=m.stride(0), n_cols=D, BLOCK_C=bf, branching_factor=bf)
        else:
            P2, R2 = torch.from_numpy(ox.grand_parents), torch.from_numpy(ox.gp_radii)
            three_level_filter_kernel_v1_batched[(P2.shape[1], hq)](
                K_ptr=K, P1_ptr=P, R1_ptr=R, P2_ptr=P2, R2_ptr=R2, q_ptr=qt, q_head_to_kv_ptr=m, out_ptr=outt,
                t_ptr=tt, scaling_ptr=st, K_h_stride=K.stride(0), K_row_stride=K.stride(1), P1_h_stride=P.stride(0),
                P1_row_stride=P.stride(1), R1_h_stride=R.stride(0), R1_row_stride=R.stride(1),
                P2_h_stride=P2.stride(0), P2_row_stride=P2.stride(1), R2_h_stride=R2.stride(0),
                R2_row_stride=R2.stride(1), q_h_stride=qt.stride(0), q_d_stride=qt.stride(1),
                out_h_stride=outt.stride(0), out_row_stride=outt.stride(1), t_h_stride=tt.stride(0),
                scaling_h_stride=st.stride(0), q2kv_h_stride=m.stride(0), n_cols=D, branch=bf, BLOCK_C=bf)
        rec = dict(initial_arrays(ox), H=H, n=n, D=D, bf=bf, depth=depth, cap_parents=ox.cap_parents, q=q, tau=tau,
                   scaling=scaling, q2kv=q2kv.astype(np.int32), expected_dense=outt.numpy())
        np.savez_compressed(out / f"{name}.npz", **rec)
        print("wrote", name, "emitted", int((outt != 0).sum()), "of", outt.numel())


def gen_cpu_search(out: Path):
    import numpy as np
    import torch
    from hira.indexer.cpu import CPUIndexer
    from hira.searcher.cpu import CPUSearcher
    for name, H, G, n, D, bf, levels in (("search_cpu_v3_l2", 2, 2, 512, 64, 16, 2), ("search_cpu_v3_l3", 2, 1, 768, 32, 8, 3)):
        rng = np.random.default_rng(21 + levels)
        keys = torch.from_numpy(unit(rng, (1, H, n, D)))
        idx = CPUIndexer(num_levels=levels, branching_factor=bf, max_iterations=3).build(keys)
        hq = H * G
        q = unit(rng, (hq, D))
        sc = np.einsum("hgd,hnd->hgn", q.reshape(H, G, D), keys[0].numpy()).reshape(hq, n)
        s = np.sort(sc, axis=-1)
        k = n // 10
        tau = (0.5 * (s[:, n - k - 1] + s[:, n - k])).astype(np.float32)     # midpoint: no key on the boundary
        scaling = rng.uniform(0.5, 2.0, hq).astype(np.float32)
        searcher = CPUSearcher(search_strategy="fused_v3")
        outt = searcher.search(torch.from_numpy(q).view(1, hq, 1, D), torch.from_numpy(tau), idx,
                               scaling=torch.from_numpy(scaling))
        rec = dict(H=H, G=G, n=n, D=D, bf=bf, n_levels=len(idx.levels), q=q, tau=tau, scaling=scaling,
                   expected_dense=outt.numpy())
        for l, lev in enumerate(idx.levels):
            rec[f"centers_{l}"] = lev.ball_centers.numpy()
            rec[f"radii_{l}"] = lev.ball_radii.numpy()
            if lev.child2parent is not None:
                rec[f"c2p_{l}"] = lev.child2parent.numpy()
        np.savez_compressed(out / f"{name}.npz", **rec)
        print("wrote", name, "selected", int((outt != 0).sum()), "of", outt.numel())


def gen_cpu_indexer_levels(out: Path):
    """The reference CPUIndexer (build, then update) with the Lloyd stand-in as faiss: pins
    oracle/cpu_index.py's restatement of everything around the k-means call."""
    import numpy as np
    import torch
    from hira.indexer.cpu import CPUIndexer
    H, n, D, bf, levels, m = 2, 600, 32, 8, 3, 20
    rng = np.random.default_rng(77)
    keys = rng.standard_normal((1, H, n, D)).astype(np.float32)
    new_keys = rng.standard_normal((1, H, m, D)).astype(np.float32)
    idx = CPUIndexer(num_levels=levels, branching_factor=bf, max_iterations=3).build(torch.from_numpy(keys))
    rec = dict(H=H, n=n, D=D, bf=bf, num_levels=levels, max_iterations=3, keys=keys[0], new_keys=new_keys[0])

    def dump(tag):
        rec[f"{tag}_n_levels"] = len(idx.levels)
        for l, lev in enumerate(idx.levels):
            rec[f"{tag}_centers_{l}"] = lev.ball_centers.numpy().copy()
            rec[f"{tag}_radii_{l}"] = lev.ball_radii.numpy().copy()
            if lev.child2parent is not None:
                rec[f"{tag}_c2p_{l}"] = lev.child2parent.numpy().copy()
    dump("built")
    idx.update(torch.from_numpy(new_keys))
    dump("updated")
    np.savez_compressed(out / "cpu_indexer_levels.npz", **rec)
    print("wrote cpu_indexer_levels", [lev.size for lev in idx.levels])


def _gate_guard_banded_tau(ox, q, q2kv, depth, start_tau, band):
    """Per query head a threshold with no gate value q.c + r within `band` of it.  Even heads
    start from `start_tau` (the workload's threshold: on this data every gate passes); odd heads
    start from the median gate value of their parents, so that the gates do prune there."""
    import numpy as np
    tau = np.array(start_tau, np.float32).copy()
    for qh in range(q.shape[0]):
        h = int(q2kv[qh])
        up, ug = int(ox.used[h, 0]), int(ox.used[h, 1])
        from oracle import oracle as O
        par = O.as_f32(ox.parents[h, :up]) if ox.parents.dtype != np.float32 else ox.parents[h, :up]
        gv = [par @ q[qh] + ox.parent_radii[h, :up]]
        if depth == 3:
            gp = O.as_f32(ox.grand_parents[h, :ug]) if ox.grand_parents.dtype != np.float32 else ox.grand_parents[h, :ug]
            gv.append(gp @ q[qh] + ox.gp_radii[h, :ug])
        if qh % 2 == 1:
            tau[qh] = np.float32(np.median(gv[0]))
        gv = np.sort(np.concatenate(gv).astype(np.float64))
        t = float(tau[qh])
        while True:
            i = np.searchsorted(gv, t)
            near = [abs(gv[j] - t) for j in (i - 1, i) if 0 <= j < len(gv)]
            if not near or min(near) > band:
                break
            t += band
        tau[qh] = np.float32(t)
    return tau


def gen_triton_search_bf16(out: Path):
    """The reference's Triton filters (interpreter) on bf16 keys of the decode workload's
    distribution (RoPE + outlier channels, un-normalised), D = 128, branching 32."""
    import numpy as np
    import torch
    from hira.kernels.triton_search_kernels import (three_level_filter_kernel_v1_batched,
                                                    two_level_filter_kernel_batched)
    from hira_b200 import workloads as W
    from oracle import oracle as O
    D, bf = 128, 32
    for name, H, G, n, depth in (("search_triton_l2_bf16_d128_bf32", 1, 4, 2048, 2),
                                 ("search_triton_l3_bf16_d128_bf32", 1, 4, 4096, 3)):
        keys, vals = W.make_kv(H, n, 300 + depth, "cpu", dist="rope_outlier", dtype=torch.bfloat16)
        k1 = n // bf
        ox = O.OracleIndex(n_heads=H, dim=D, vdim=D, bf=bf, depth=depth, cap_parents=k1, dtype=O.HIRA_BF16,
                           vdtype=O.HIRA_BF16)
        c1 = W.random_centres(H, n, k1, 5, "cpu")
        c2 = W.random_centres(H, k1, k1 // bf, 6, "cpu") if depth == 3 else None
        O.build(ox, keys, vals, cent_idx1=c1, cent_idx2=c2)
        hq = H * G
        q = W.make_queries(hq, 9, "cpu", pos=n)
        q = (q / q.norm(dim=-1, keepdim=True)).numpy()
        q2kv = np.repeat(np.arange(H), G).astype(np.int64)
        kf = keys.float().numpy()
        sc = np.einsum("hgd,hnd->hgn", q.reshape(H, G, D), kf).reshape(hq, n)
        tau0 = np.sort(sc, axis=-1)[:, n - max(1, n // 50)]          # keeps about 2 %
        tau = _gate_guard_banded_tau(ox, q, q2kv, depth, tau0, 2e-3)
        scaling = np.random.default_rng(3).uniform(0.5, 2.0, hq).astype(np.float32)
        f32 = lambda a: torch.from_numpy(O.as_f32(a).copy())
        K, P, R = f32(ox.children), f32(ox.parents), torch.from_numpy(ox.parent_radii)
        qt, tt, st = torch.from_numpy(q), torch.from_numpy(tau), torch.from_numpy(scaling)
        m = torch.from_numpy(q2kv)
        outt = torch.zeros((hq, n), dtype=torch.float32)
        if depth == 2:
            two_level_filter_kernel_batched[(k1, hq)](
                K_ptr=K, P_ptr=P, R_ptr=R, q_ptr=qt, q_head_to_kv_ptr=m, out_ptr=outt, t_ptr=tt, scaling_ptr=st,
                K_h_stride=K.stride(0), K_row_stride=K.stride(1), P_h_stride=P.stride(0), P_row_stride=P.stride(1),
                R_h_stride=R.stride(0), R_row_stride=R.stride(1), q_h_stride=qt.stride(0), q_d_stride=qt.stride(1),
                out_h_stride=outt.stride(0), out_row_stride=outt.stride(1), t_h_stride=tt.stride(0),
                scaling_h_stride=st.stride(0), q2kv_h_stride=m.stride(0), n_cols=D, BLOCK_C=bf, branching_factor=bf)
        else:
            P2, R2 = f32(ox.grand_parents), torch.from_numpy(ox.gp_radii)
            three_level_filter_kernel_v1_batched[(P2.shape[1], hq)](
                K_ptr=K, P1_ptr=P, R1_ptr=R, P2_ptr=P2, R2_ptr=R2, q_ptr=qt, q_head_to_kv_ptr=m, out_ptr=outt,
                t_ptr=tt, scaling_ptr=st, K_h_stride=K.stride(0), K_row_stride=K.stride(1), P1_h_stride=P.stride(0),
                P1_row_stride=P.stride(1), R1_h_stride=R.stride(0), R1_row_stride=R.stride(1),
                P2_h_stride=P2.stride(0), P2_row_stride=P2.stride(1), R2_h_stride=R2.stride(0),
                R2_row_stride=R2.stride(1), q_h_stride=qt.stride(0), q_d_stride=qt.stride(1),
                out_h_stride=outt.stride(0), out_row_stride=outt.stride(1), t_h_stride=tt.stride(0),
                scaling_h_stride=st.stride(0), q2kv_h_stride=m.stride(0), n_cols=D, branch=bf, BLOCK_C=bf)
        rec = dict(H=H, n=n, D=D, bf=bf, depth=depth, cap_parents=ox.cap_parents, q=q, tau=tau, scaling=scaling,
                   q2kv=q2kv.astype(np.int32), keys_bf16=keys.view(torch.int16).numpy(),
                   cent_idx1=c1.numpy(), expected_mask=np.packbits(outt.numpy() != 0, axis=-1),
                   expected_sum=outt.numpy().sum(axis=-1))
        if depth == 3:
            rec["cent_idx2"] = c2.numpy()
        np.savez_compressed(out / f"{name}.npz", **rec)
        print("wrote", name, "emitted", int((outt != 0).sum()), "of", outt.numel())


def gen_gpu_reference_search(out: Path):
    """ON A CUDA DEVICE: the reference's own CUDASearcher (its Triton kernels, compiled for the
    GPU) on an index this library built from the cfg1 and cfg4 workloads -- 8 KV heads, bf16,
    D = 128; 32,768 keys / branching 32 / 32 query heads and 131,072 keys / branching 64 / 64
    query heads.  The reference searcher sees fp32 copies of the index arrays through an object
    with the attribute names of its CUDAIndexer.  The data is generated on the device from
    seeds; the fixture keeps checksums of it, the thresholds and the candidate bitmaps."""
    import hashlib
    import numpy as np
    import torch
    from hira.searcher.cuda import CUDASearcher as RefSearcher
    from hira.indexer.cuda import CUDAIndexer as RefIndexer
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200 import workloads as W
    from oracle import oracle as O
    dev = torch.device("cuda", 0)
    for tag, w in (("cfg1", W.CFG1), ("cfg4", W.CFG4)):
        H, n, D, bf, G = w.kv_heads, w.context, W.DIM, w.branching, w.group
        keys, vals, q = W.make_inputs(w, dev)
        k1, k2 = n // bf, n // bf // bf
        st = S.IndexState(n_heads=H, dim=D, vdim=D, bf=bf, depth=3, cap_parents=k1, dtype=torch.bfloat16,
                          vdtype=torch.bfloat16, device=dev)
        c1 = W.random_centres(H, n, k1, 7, dev)
        c2 = W.random_centres(H, k1, k2, 8, dev)
        S.build(st, keys, vals, cent_idx1=c1, cent_idx2=c2, n_iters=1, use_tensor_cores=False)
        torch.cuda.synchronize()
        hq = H * G
        q_hat = (q / q.norm(dim=-1, keepdim=True)).contiguous()
        ox = O.OracleIndex.from_arrays(st.state_dict())
        sc = torch.einsum("hgd,hnd->hgn", q_hat.view(H, G, D), keys.float()).reshape(hq, n)
        tau0 = torch.sort(sc, dim=-1).values[:, n - w.kth].cpu().numpy()
        q2kv = np.repeat(np.arange(H), G)
        tau = _gate_guard_banded_tau(ox, q_hat.cpu().numpy(), q2kv, 3, tau0, 2e-3)

        class View:
            pass
        v = View()
        v.children, v.parents = st.children.float(), st.parents.float()
        v.parent_radii, v.grand_parents = st.parent_radii, st.grand_parents.float()
        v.grand_parent_radii = st.gp_radii
        v.branching_factor, v.depth = bf, RefIndexer.DEPTH.THREE_LEVELS
        tt = torch.from_numpy(tau).to(dev)
        dense = RefSearcher(block_c=bf).search(q_hat.view(1, hq, 1, D), tt, v)
        torch.cuda.synchronize()
        ref_mask = (dense != 0).cpu().numpy()
        _, compact = S.search(st, q_hat, tt, flags=L.HIRA_GATE_GT | L.HIRA_LEAF_CANDIDATES, want_compact=True)
        ours = np.zeros_like(ref_mask)
        for qh, (slots, _) in enumerate(compact.to_lists()):
            ours[qh, slots.numpy()] = True
        sha = lambda t: hashlib.sha256(t.contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()
        rec = dict(H=H, n=n, D=D, bf=bf, G=G, tau=tau, keys_sha=sha(keys), children_sha=sha(st.children),
                   q_sha=sha(q_hat), expected_mask=np.packbits(ref_mask, axis=-1),
                   candidates=ref_mask.sum(axis=-1).astype(np.int64), equal_when_generated=bool((ours == ref_mask).all()))
        np.savez_compressed(out / f"search_triton_gpu_{tag}.npz", **rec)
        print("wrote", f"search_triton_gpu_{tag}", "candidates", int(ref_mask.sum()), "of", ref_mask.size,
              "ours == reference:", rec["equal_when_generated"], "differing:", int((ours != ref_mask).sum()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("HIRA_REFERENCE"), required="HIRA_REFERENCE" not in os.environ,
                    help="path of the reference checkout (or set HIRA_REFERENCE)")
    ap.add_argument("--out", default=str(HERE))
    ap.add_argument("--gpu", action="store_true",
                    help="run the reference's GPU searcher on a CUDA device (search_triton_gpu_*.npz only)")
    a = ap.parse_args()
    if a.gpu:
        os.environ.pop("TRITON_INTERPRET", None)
    setup_reference(Path(a.ref).resolve())
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    if a.gpu:
        gen_gpu_reference_search(out)
        return
    gen_append_and_radii(out)
    gen_triton_search(out)
    gen_triton_search_bf16(out)
    gen_cpu_search(out)
    gen_cpu_indexer_levels(out)


if __name__ == "__main__":
    main()
