"""ctypes/numpy front end of the CPU oracle (oracle/hira_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py -- never by the hira_b200 package.

An `OracleIndex` holds the arrays of one hira_index_t in host memory (numpy); bf16
arrays are kept as uint16 bit patterns.  `OracleIndex.from_arrays` accepts the dict that
`IndexState.state_dict()` produces (tensors are moved to the host), so an index can be
built on the device and searched by the oracle, or the other way round.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libhira_oracle.so"

HIRA_F32, HIRA_BF16 = 0, 1
GATE_GT, GATE_GE = 0, 1
LEAF_CANDIDATES, LEAF_GE, LEAF_GT = 0, 2, 4
TAU_SAMPLE_MAX, TAU_SAMPLE_MEAN_TOPK, TAU_SAMPLE_KTH = 0, 1, 2


class _IndexStruct(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("vdtype", C.c_int32), ("depth", C.c_int32), ("bf", C.c_int32),
        ("dim", C.c_int32), ("vdim", C.c_int32), ("n_heads", C.c_int32), ("cap_parents", C.c_int32),
        ("cap_gp", C.c_int32), ("active_parents", C.c_int32),
        ("children", C.c_void_p), ("values", C.c_void_p), ("slot2token", C.c_void_p),
        ("parents", C.c_void_p), ("parent_radii", C.c_void_p), ("parent_sqnorm", C.c_void_p),
        ("child_counts", C.c_void_p), ("grand_parents", C.c_void_p), ("gp_radii", C.c_void_p),
        ("gp_sqnorm", C.c_void_p), ("gp_counts", C.c_void_p), ("used", C.c_void_p),
        # the device-side int8 side copy of the children: always NULL here (the oracle has no use for it)
        ("children_q8", C.c_void_p), ("children_q8_meta", C.c_void_p), ("q8_chan_scale", C.c_void_p),
        ("q8_query_scratch", C.c_void_p),
    ]


def build_oracle(force: bool = False) -> Path:
    """Compiles libhira_oracle.so with the recipe in oracle/Makefile."""
    if force or not LIB.exists() or LIB.stat().st_mtime < (HERE / "hira_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "libhira_oracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build_oracle()
        _lib = C.CDLL(str(LIB))
        _lib.oracle_dot.restype = C.c_float
        _lib.oracle_dot.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def to_host(t):
    """torch tensor (any device, fp32/bf16/int) or ndarray -> contiguous ndarray; bf16 -> uint16 bits."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return np.ascontiguousarray(t)
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = u + 0x7FFF + ((u >> 16) & 1)
    return (r >> 16).astype(np.uint16)


def as_f32(a: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(a) if a.dtype == np.uint16 else a.astype(np.float32, copy=False)


class OracleIndex:
    ARRAYS = ("children", "values", "slot2token", "parents", "parent_radii", "parent_sqnorm", "child_counts",
              "grand_parents", "gp_radii", "gp_sqnorm", "gp_counts", "used")

    def __init__(self, *, n_heads, dim, vdim, bf, depth, cap_parents, dtype=HIRA_F32, vdtype=HIRA_F32,
                 with_values=True):
        self.n_heads, self.dim, self.bf, self.depth = n_heads, dim, bf, depth
        self.vdim = vdim if with_values else 0
        self.dtype, self.vdtype = dtype, vdtype
        if depth == 3:
            self.cap_gp = max(1, -(-cap_parents // bf))
            self.cap_parents = self.cap_gp * bf
        else:
            self.cap_gp, self.cap_parents = 0, max(1, cap_parents)
        capC = self.cap_parents * bf
        kd = np.uint16 if dtype == HIRA_BF16 else np.float32
        vd = np.uint16 if vdtype == HIRA_BF16 else np.float32
        self.children = np.zeros((n_heads, capC, dim), kd)
        self.values = np.zeros((n_heads, capC, self.vdim), vd) if with_values else None
        self.slot2token = np.full((n_heads, capC), -1, np.int32)
        self.parents = np.zeros((n_heads, self.cap_parents, dim), kd)
        self.parent_radii = np.zeros((n_heads, self.cap_parents), np.float32)
        self.parent_sqnorm = np.zeros((n_heads, self.cap_parents), np.float32)
        self.child_counts = np.zeros((n_heads, self.cap_parents), np.int32)
        if depth == 3:
            self.grand_parents = np.zeros((n_heads, self.cap_gp, dim), kd)
            self.gp_radii = np.zeros((n_heads, self.cap_gp), np.float32)
            self.gp_sqnorm = np.zeros((n_heads, self.cap_gp), np.float32)
            self.gp_counts = np.zeros((n_heads, self.cap_gp), np.int32)
        else:
            self.grand_parents = self.gp_radii = self.gp_sqnorm = self.gp_counts = None
        self.used = np.zeros((n_heads, 4), np.int32)
        self.status = np.zeros((1,), np.int32)

    @property
    def cap_children(self):
        return self.cap_parents * self.bf

    @classmethod
    def from_arrays(cls, sd: dict) -> "OracleIndex":
        m = sd["meta"]
        code = lambda s: HIRA_BF16 if "bfloat16" in str(s) else HIRA_F32
        ix = cls(n_heads=m["n_heads"], dim=m["dim"], vdim=m["vdim"], bf=m["bf"], depth=m["depth"],
                 cap_parents=m["cap_parents"], dtype=code(m["dtype"]), vdtype=code(m["vdtype"]),
                 with_values=sd.get("values") is not None)
        for name in cls.ARRAYS:
            if getattr(ix, name) is None or sd.get(name) is None:
                continue
            src = to_host(sd[name])
            dst = getattr(ix, name)
            assert src.shape == dst.shape and src.dtype == dst.dtype, (name, src.shape, dst.shape, src.dtype, dst.dtype)
            setattr(ix, name, src)
        return ix

    def arrays(self) -> dict:
        d = {name: getattr(self, name) for name in self.ARRAYS}
        d["meta"] = dict(n_heads=self.n_heads, dim=self.dim, vdim=self.vdim, bf=self.bf, depth=self.depth,
                         cap_parents=self.cap_parents,
                         dtype="torch.bfloat16" if self.dtype == HIRA_BF16 else "torch.float32",
                         vdtype="torch.bfloat16" if self.vdtype == HIRA_BF16 else "torch.float32")
        return d

    def struct(self):
        s = _IndexStruct()
        s.dtype, s.vdtype, s.depth, s.bf = self.dtype, self.vdtype, self.depth, self.bf
        s.dim, s.vdim, s.n_heads = self.dim, self.vdim, self.n_heads
        s.cap_parents, s.cap_gp = self.cap_parents, self.cap_gp
        for name in self.ARRAYS:
            a = getattr(self, name)
            setattr(s, name, None if a is None else a.ctypes.data)
        return s


def _f32(a):
    return None if a is None else np.ascontiguousarray(to_host(a), dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(to_host(a), dtype=np.int32)


def dot(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return float(lib().oracle_dot(_p(a), _p(b), a.shape[0]))


def search(ix: OracleIndex, q, tau, *, scaling=None, qnorm=None, q2kv=None, flags=0, want_stats=False):
    """Returns (dense (H_q, capC) fp32, keep (H_q, capC) uint8[, stats (H_q, 8) uint32])."""
    q, tau, scaling, qnorm, q2kv = _f32(q), _f32(tau), _f32(scaling), _f32(qnorm), _i32(q2kv)
    hq = q.shape[0]
    dense = np.zeros((hq, ix.cap_children), np.float32)
    keep = np.zeros((hq, ix.cap_children), np.uint8)
    stats = np.zeros((hq, 8), np.uint32) if want_stats else None
    s = ix.struct()
    rc = lib().oracle_search(C.byref(s), _p(q), _p(tau), _p(scaling), _p(qnorm), _p(q2kv), hq, flags, _p(dense),
                             _p(keep), _p(stats))
    assert rc == 0
    return (dense, keep, stats) if want_stats else (dense, keep)


def search_csr(centers, radii, offsets, children, sizes, q, tau, *, scaling=None, q2kv=None):
    """CPU-format index search (levels + CSR adjacency); level 0 = keys."""
    n_levels = len(sizes)
    cs = [_f32(c) for c in centers]
    rs = [_f32(r) for r in radii]
    offs = [None if o is None else np.ascontiguousarray(to_host(o), dtype=np.int64) for o in offsets]
    chs = [None if c is None else np.ascontiguousarray(to_host(c), dtype=np.int64) for c in children]
    q, tau, scaling, q2kv = _f32(q), _f32(tau), _f32(scaling), _i32(q2kv)
    hq, dim = q.shape
    n_heads = cs[0].shape[0]
    arr = lambda lst: (C.c_void_p * n_levels)(*[None if a is None else a.ctypes.data for a in lst])
    sz = np.asarray(sizes, dtype=np.int64)
    out = np.zeros((hq, int(sizes[0])), np.float32)
    keep = np.zeros((hq, int(sizes[0])), np.uint8)
    rc = lib().oracle_search_csr(n_levels, arr(cs), arr(rs), arr(offs), arr(chs), _p(sz), n_heads, dim, _p(q),
                                 _p(tau), _p(scaling), _p(q2kv), hq, _p(out), _p(keep))
    assert rc == 0
    return out, keep


def recompute_radii(ix: OracleIndex):
    s = ix.struct()
    assert lib().oracle_recompute_radii(C.byref(s)) == 0


def append(ix: OracleIndex, new_k, new_v, token_base: int = -1):
    """new_k (n_heads, M, D) in the index dtype (uint16 bits for bf16)."""
    new_k = to_host(new_k)
    new_v = to_host(new_v)
    m = new_k.shape[1]
    s = ix.struct()
    rc = lib().oracle_append(C.byref(s), _p(new_k), _p(new_v), m, C.c_int64(m * ix.dim),
                             C.c_int64(m * ix.vdim), token_base, _p(ix.status))
    assert rc == 0


def attention(ix: OracleIndex, q, scaling, dense, keep, *, q2kv=None, queued_k=None, queued_v=None):
    q, scaling, q2kv = _f32(q), _f32(scaling), _i32(q2kv)
    hq = q.shape[0]
    queued_k, queued_v = to_host(queued_k), to_host(queued_v)
    nq = 0 if queued_k is None else queued_k.shape[1]
    out = np.zeros((hq, ix.vdim), np.float32)
    ml = np.zeros((hq, 2), np.float32)
    s = ix.struct()
    rc = lib().oracle_attention(C.byref(s), _p(q), _p(scaling), _p(q2kv), hq, _p(np.ascontiguousarray(dense)),
                                _p(np.ascontiguousarray(keep)), _p(queued_k), _p(queued_v), nq,
                                C.c_int64(nq * ix.dim), _p(out), _p(ml))
    assert rc == 0
    return out, ml


def threshold(samples, q, method: int, k: int = 1, q2kv=None):
    samples = to_host(samples)
    dtype = HIRA_BF16 if samples.dtype == np.uint16 else HIRA_F32
    q, q2kv = _f32(q), _i32(q2kv)
    h, s_, d = samples.shape
    out = np.zeros((q.shape[0],), np.float32)
    rc = lib().oracle_threshold(_p(samples), dtype, h, s_, d, C.c_int64(s_ * d), _p(q), _p(q2kv), q.shape[0], method,
                                k, _p(out))
    assert rc == 0
    return out


def assign(points, cents):
    points, cents = to_host(points), to_host(cents)
    dtype = HIRA_BF16 if points.dtype == np.uint16 else HIRA_F32
    h, n, d = points.shape
    k = cents.shape[1]
    idx = np.zeros((h, n), np.int32)
    d2 = np.zeros((h, n), np.float32)
    rc = lib().oracle_assign(_p(points), C.c_int64(n * d), _p(cents), dtype, h, n, k, d, _p(idx), _p(d2))
    assert rc == 0
    return idx, d2


def build(ix: OracleIndex, keys, values, *, cent_idx1=None, cent_idx2=None, n_iters: int = 1, token_base: int = 0,
          balance_rounds: int = 0):
    keys, values = to_host(keys), to_host(values)
    c1, c2 = _i32(cent_idx1), _i32(cent_idx2)
    n = keys.shape[1]
    s = ix.struct()
    rc = lib().oracle_build(C.byref(s), _p(keys), _p(values), n, C.c_int64(n * ix.dim), C.c_int64(n * ix.vdim),
                            token_base, _p(c1), _p(c2), n_iters, balance_rounds)
    assert rc == 0


def merge_partials(part_o, part_ml):
    part_o, part_ml = _f32(part_o), _f32(part_ml)
    n_parts, hq, vdim = part_o.shape
    out = np.zeros((hq, vdim), np.float32)
    ml = np.zeros((hq, 2), np.float32)
    assert lib().oracle_merge_partials(_p(part_o), _p(part_ml), n_parts, hq, vdim, _p(out), _p(ml)) == 0
    return out, ml


def num_threads() -> int:
    return int(lib().oracle_num_threads())
