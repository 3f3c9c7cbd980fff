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

os.environ["TRITON_INTERPRET"] = "1"

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]

FAISS_SHIM = '''
import numpy as np
class _Index:
    def __init__(self, c): self.c = c
    def search(self, x, k):
        d = (x * x).sum(1)[:, None] - 2.0 * x @ self.c.T + (self.c * self.c).sum(1)[None, :]
        i = d.argmin(1)
        return d[np.arange(len(x)), i][:, None], i[:, None]
class Kmeans:
    def __init__(self, d, k, niter=1, verbose=False, gpu=False, seed=0, min_points_per_centroid=1):
        self.d, self.k, self.niter, self.seed = d, k, niter, seed
    def train(self, x):
        rng = np.random.default_rng(self.seed)
        c = x[rng.choice(len(x), self.k, replace=False)].copy()
        for _ in range(self.niter):
            a = _Index(c).search(x, 1)[1][:, 0]
            for j in range(self.k):
                m = a == j
                if m.any(): c[j] = x[m].mean(0)
        self.centroids = c.astype(np.float32)
        self.index = _Index(self.centroids)
'''


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("HIRA_REFERENCE"), required="HIRA_REFERENCE" not in os.environ,
                    help="path of the reference checkout (or set HIRA_REFERENCE)")
    ap.add_argument("--out", default=str(HERE))
    a = ap.parse_args()
    setup_reference(Path(a.ref))
    out = Path(a.out)
    gen_append_and_radii(out)
    gen_triton_search(out)
    gen_cpu_search(out)


if __name__ == "__main__":
    main()
