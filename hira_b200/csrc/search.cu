// Level-by-level halfspace search over the blocked index.
//
// One CTA owns one tile of consecutive parent slots of one kv head and up to
// GT query heads of that kv head at once, so every key row is read from HBM
// once per GQA group instead of once per query head (the reference launches
// one program per (parent, query head): kernels/triton_search_wrappers.py:182).
//
// Semantics follow kernels/triton_search_kernels.py:6-148 (gate `dot + r > tau`,
// every child of a kept parent is emitted) or, by flags,
// kernels/cpp/torch_ext_v3.cpp:177-241 (gate `>=`, leaf test `dot >= tau`).
// The kernel is a streaming read: 16-lane groups each read one 256-byte row
// with 128-bit loads, several rows in flight per thread; it is HBM-bound.
#include "common.cuh"

namespace hira {

constexpr int SEARCH_THREADS = 256;
constexpr int SEARCH_HW = SEARCH_THREADS / 16;   // half-warps per CTA
constexpr int SEARCH_WARPS = SEARCH_THREADS / 32;
constexpr int MAX_TILE_ROWS = 1024;
constexpr int SEARCH_UNROLL = 4;

struct SearchParams {
    const void* children;
    const void* parents;
    const void* gps;
    const float* parent_radii;
    const float* gp_radii;
    const int32_t* child_counts;
    const int32_t* gp_counts;
    const int32_t* used;
    const float* q;
    const float* tau;
    const float* scaling;
    const float* qnorm;
    const int32_t* q2kv;
    float* out_dense;
    int32_t* out_idx;
    float* out_score;
    int32_t* out_count;
    uint32_t* stats;
    int n_heads, n_qheads, group, depth, bf, dim;
    int cap_parents, cap_gp, tile_parents, n_tiles, flags;
    uint32_t bf_magic;  // ceil(2^32 / bf): x / bf == __umulhi(x, bf_magic) for x < 2^20, bf <= 1024
};

__device__ __forceinline__ int div_bf(int x, int bf, uint32_t magic) {
    return bf == 1 ? x : (int)__umulhi((uint32_t)x, magic);
}

__device__ __forceinline__ bool gate_keep(float dot, float r, float qn, bool has_qn, float tau, bool ge) {
    const float rr = has_qn ? __fmul_rn(qn, r) : r;
    const float s = __fadd_rn(dot, rr);
    return ge ? (s >= tau) : (s > tau);
}

// bit j of the result = predicate of the lane that owns head j in this half-warp
template <int GT>
__device__ __forceinline__ uint32_t head_mask_from_ballot(uint32_t ballot, int tid) {
    const int half_base = tid & 16;
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        // first lane owning head j
        int l = 0;
        if (GT == 2) l = j * 8;
        if (GT == 4) l = j * 4;
        if (GT == 8) l = j * 2;
        m |= ((ballot >> (half_base + l)) & 1u) << j;
    }
    return m;
}

template <typename T, int GT, int NCH>
__global__ void __launch_bounds__(SEARCH_THREADS, (GT * NCH <= 4) ? 2 : 1)
search_kernel(const SearchParams P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int TP = P.tile_parents;
    const int bf = P.bf;
    const int tile_rows = TP * bf;
    float* s_score = reinterpret_cast<float*>(smem_raw);             // [tile_rows][GT]
    int* s_pcount = reinterpret_cast<int*>(s_score + (size_t)tile_rows * GT);  // [TP]
    unsigned short* s_plist = reinterpret_cast<unsigned short*>(s_pcount + TP);  // [TP]
    unsigned char* s_pmask = reinterpret_cast<unsigned char*>(s_plist + TP);     // [TP]
    unsigned char* s_gpmask = s_pmask + TP;                                      // [TP]

    __shared__ int s_qh[GT];
    __shared__ float s_tau[GT], s_scale[GT], s_qn[GT];
    __shared__ int s_nq, s_npass;
    __shared__ int s_segcnt[SEARCH_WARPS];
    __shared__ uint32_t s_stat[GT][8];

    const int tid = threadIdx.x;
    const int lane = tid & 15;     // lane inside the half-warp
    const int hw = tid >> 4;       // half-warp id
    const int warp = tid >> 5;
    const int wl = tid & 31;
    const int tile = blockIdx.x % P.n_tiles;
    const int h = blockIdx.x / P.n_tiles;
    const int chunk = blockIdx.y;
    const bool ge = P.flags & HIRA_GATE_GE;
    const int leaf_mode = P.flags & (HIRA_LEAF_GE | HIRA_LEAF_GT);
    const bool has_qn = P.qnorm != nullptr;
    const size_t cap_children = (size_t)P.cap_parents * bf;
    const T* children = reinterpret_cast<const T*>(P.children) + (size_t)h * cap_children * P.dim;
    const T* parents = reinterpret_cast<const T*>(P.parents) + (size_t)h * P.cap_parents * P.dim;

    // ---- 1. query heads of this kv head handled by this CTA ------------------
    if (tid < GT * 8) (&s_stat[0][0])[tid] = 0;
    if (P.q2kv == nullptr) {
        if (tid == 0) {
            int n = P.group - chunk * GT;
            n = n < 0 ? 0 : (n > GT ? GT : n);
            s_nq = n;
            for (int j = 0; j < n; ++j) s_qh[j] = h * P.group + chunk * GT + j;
        }
    } else if (warp == 0) {
        // ordered scan of the explicit map; keep matches [chunk*GT, chunk*GT+GT)
        int seen = 0;
        for (int base = 0; base < P.n_qheads; base += 32) {
            const int i = base + wl;
            const bool m = (i < P.n_qheads) && (P.q2kv[i] == h);
            const uint32_t b = __ballot_sync(0xffffffffu, m);
            const int pos = seen + __popc(b & ((1u << wl) - 1u));
            if (m && pos >= chunk * GT && pos < chunk * GT + GT) s_qh[pos - chunk * GT] = i;
            seen += __popc(b);
        }
        if (wl == 0) {
            int n = seen - chunk * GT;
            s_nq = n < 0 ? 0 : (n > GT ? GT : n);
        }
    }
    __syncthreads();
    const int nq = s_nq;
    const int tile_p0 = tile * TP;
    const size_t tile_c0 = (size_t)tile_p0 * bf;
    if (nq == 0) return;  // nothing mapped to this (kv head, chunk): no outputs owned
    if (tid < nq) {
        const int qh = s_qh[tid];
        s_tau[tid] = P.tau[qh];
        s_scale[tid] = P.scaling ? P.scaling[qh] : 1.0f;
        s_qn[tid] = has_qn ? P.qnorm[qh] : 1.0f;
    }

    // tile beyond the slots in use: emit nothing
    const int used_parents = P.used[h * 4 + 0];
    const int used_gp = P.used[h * 4 + 1];
    bool tile_empty;
    if (P.depth == 3) tile_empty = (tile_p0 / bf) >= used_gp;
    else tile_empty = tile_p0 >= used_parents;

    float qreg[GT][NCH][8];
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        if (j < nq && !tile_empty) {
            load_vec_f32<NCH>(P.q + (size_t)s_qh[j] * P.dim, qreg[j], lane, P.dim);
        } else {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) qreg[j][i][e] = 0.f;
        }
    }
    __syncthreads();

    int npass = 0;
    if (!tile_empty) {
        // ---- 2. grandparent gate ---------------------------------------------
        const uint32_t allmask = (1u << nq) - 1u;
        const int g0 = tile_p0 / bf;
        const int ng = (TP + bf - 1) / bf;  // grandparents touched by this tile (TP % bf == 0 or bf % TP == 0)
        if (P.depth == 3) {
            const T* gps = reinterpret_cast<const T*>(P.gps) + (size_t)h * P.cap_gp * P.dim;
            for (int i0 = 0; i0 < ng; i0 += SEARCH_HW) {  // trip count uniform over the CTA: shuffles inside
                const int i = i0 + hw;
                const int g = g0 + i;
                const bool valid = (i < ng) && (g < used_gp);  // uniform inside the half-warp
                float v[GT];
#pragma unroll
                for (int j = 0; j < GT; ++j) v[j] = 0.f;
                if (valid) {
                    Acc2 acc[GT];
#pragma unroll
                    for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
                    for (int ci = 0; ci < NCH; ++ci) {
                        const int c = lane + 16 * ci;
                        if (c * 8 < P.dim) {
                            float a[8];
                            to_float(load_chunk<T>(gps + (size_t)g * P.dim, c), a);
#pragma unroll
                            for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
                }
                const float d = HeadReduce<GT>::run(v, lane);
                const int j = HeadReduce<GT>::head_of_lane(lane);
                bool keep = false;
                if (valid && j < nq)
                    keep = gate_keep(d, P.gp_radii[(size_t)h * P.cap_gp + g], s_qn[j], has_qn, s_tau[j], ge);
                const uint32_t b = __ballot_sync(0xffffffffu, keep);
                const uint32_t m = head_mask_from_ballot<GT>(b, tid);
                if (lane == 0 && i < ng) {
                    s_gpmask[i] = (unsigned char)m;
                    // a grandparent whose parents span several tiles is gated by each of
                    // them; only the tile holding its first parent books the visit
                    if (valid && P.stats && (tile_p0 % bf) == 0) {
                        for (int jj = 0; jj < nq; ++jj) {
                            atomicAdd(&s_stat[jj][0], 1u);
                            if ((m >> jj) & 1u) atomicAdd(&s_stat[jj][1], 1u);
                        }
                    }
                }
            }
            __syncthreads();
        }

        // ---- 3. parent gate ---------------------------------------------------
        for (int i0 = 0; i0 < TP; i0 += SEARCH_HW) {  // uniform trip count
            const int i = i0 + hw;
            const int p = tile_p0 + i;
            bool valid = (i < TP) && (p < P.cap_parents);
            uint32_t gm = allmask;
            if (valid) {
                if (P.depth == 3) {
                    const int g = p / bf;
                    valid = (g < used_gp) && ((p - g * bf) < P.gp_counts[(size_t)h * P.cap_gp + g]);
                    gm = s_gpmask[g - g0];
                } else {
                    valid = p < used_parents;
                }
            }
            const bool work = valid && gm != 0;
            float v[GT];
#pragma unroll
            for (int j = 0; j < GT; ++j) v[j] = 0.f;
            if (work) {
                Acc2 acc[GT];
#pragma unroll
                for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
                for (int ci = 0; ci < NCH; ++ci) {
                    const int c = lane + 16 * ci;
                    if (c * 8 < P.dim) {
                        float a[8];
                        to_float(load_chunk<T>(parents + (size_t)p * P.dim, c), a);
#pragma unroll
                        for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);
                    }
                }
#pragma unroll
                for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
            }
            const float d = HeadReduce<GT>::run(v, lane);
            const int j = HeadReduce<GT>::head_of_lane(lane);
            bool keep = false;
            if (work && j < nq && ((gm >> j) & 1u))
                keep = gate_keep(d, P.parent_radii[(size_t)h * P.cap_parents + p], s_qn[j], has_qn, s_tau[j], ge);
            const uint32_t b = __ballot_sync(0xffffffffu, keep);
            const uint32_t m = head_mask_from_ballot<GT>(b, tid);
            if (lane == 0 && i < TP) {
                int cnt = 0;
                if (valid) {
                    cnt = P.child_counts[(size_t)h * P.cap_parents + p];
                    cnt = cnt > bf ? bf : cnt;
                }
                s_pmask[i] = (unsigned char)m;
                s_pcount[i] = cnt;
                if (work && P.stats) {
                    atomicAdd(&s_stat[0][7], 1u);                       // parent rows read (any head)
                    if (m != 0) atomicAdd(&s_stat[0][6], (uint32_t)cnt);  // child rows read (any head)
                    for (int jj = 0; jj < nq; ++jj) {
                        if ((gm >> jj) & 1u) atomicAdd(&s_stat[jj][2], 1u);
                        if ((m >> jj) & 1u) {
                            atomicAdd(&s_stat[jj][3], 1u);
                            atomicAdd(&s_stat[jj][4], (uint32_t)cnt);
                        }
                    }
                }
            }
        }
        __syncthreads();

        // ---- 4. ordered list of parents kept for at least one head ------------
        if (warp == 0) {
            int n = 0;
            for (int base = 0; base < TP; base += 32) {
                const int i = base + wl;
                const bool m = (i < TP) && s_pmask[i] != 0 && s_pcount[i] > 0;
                const uint32_t b = __ballot_sync(0xffffffffu, m);
                if (m) s_plist[n + __popc(b & ((1u << wl) - 1u))] = (unsigned short)i;
                n += __popc(b);
            }
            if (wl == 0) s_npass = n;
        }
        __syncthreads();
        npass = s_npass;

        // ---- 5. stream the children rows of kept parents ----------------------
        const int total = npass * bf;
        for (int base = 0; base < total; base += SEARCH_HW * SEARCH_UNROLL) {
            RawChunk<T> raw[SEARCH_UNROLL][NCH];
            int sl[SEARCH_UNROLL];  // local slot (pl*bf + child) or -1
#pragma unroll
            for (int u = 0; u < SEARCH_UNROLL; ++u) {
                const int r = base + u * SEARCH_HW + hw;
                sl[u] = -1;
                if (r < total) {
                    const int k = div_bf(r, bf, P.bf_magic);
                    const int child = r - k * bf;
                    const int pl = s_plist[k];
                    if (child < s_pcount[pl]) sl[u] = pl * bf + child;
                }
#pragma unroll
                for (int ci = 0; ci < NCH; ++ci) {
                    const int c = lane + 16 * ci;
                    if (sl[u] >= 0 && c * 8 < P.dim)
                        raw[u][ci] = load_chunk_stream<T>(children + (tile_c0 + sl[u]) * P.dim, c);
                    else
                        raw[u][ci] = zero_chunk<T>();
                }
            }
#pragma unroll
            for (int u = 0; u < SEARCH_UNROLL; ++u) {
                Acc2 acc[GT];
#pragma unroll
                for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
                for (int ci = 0; ci < NCH; ++ci) {
                    float a[8];
                    to_float(raw[u][ci], a);
#pragma unroll
                    for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);
                }
                float v[GT];
#pragma unroll
                for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
                const float d = HeadReduce<GT>::run(v, lane);
                const int j = HeadReduce<GT>::head_of_lane(lane);
                // the first lane owning head j writes
                const bool writer = (GT == 1) ? (lane == 0)
                                  : (GT == 2) ? ((lane & 7) == 0)
                                  : (GT == 4) ? ((lane & 3) == 0)
                                              : ((lane & 1) == 0);
                if (writer && sl[u] >= 0) s_score[(size_t)sl[u] * GT + j] = d;
            }
        }
        __syncthreads();
    }

    // ---- 6. ordered compaction per head + dense output ------------------------
    constexpr int NSEG = SEARCH_WARPS / GT;  // warps per head
    const int j = warp % GT;
    const int seg = warp / GT;
    const int seg_rows = (tile_rows + NSEG - 1) / NSEG;
    const int r_begin = seg * seg_rows;
    const int r_end = min(tile_rows, r_begin + seg_rows);
    const bool active = j < nq;
    const int qh = active ? s_qh[j] : 0;
    const float tau = active ? s_tau[j] : 0.f;
    const float scale = active ? s_scale[j] : 0.f;
    const bool want_compact = P.out_idx != nullptr;

    auto keep_of = [&](int i, float& sc) -> bool {
        // i: local slot inside the tile
        const int pl = div_bf(i, bf, P.bf_magic);
        const int child = i - pl * bf;
        bool k = (npass > 0) && ((s_pmask[pl] >> j) & 1u) && (child < s_pcount[pl]);
        sc = 0.f;
        if (k) {
            sc = s_score[(size_t)i * GT + j];
            if (leaf_mode == HIRA_LEAF_GE) k = sc >= tau;
            else if (leaf_mode == HIRA_LEAF_GT) k = sc > tau;
        }
        return k;
    };

    int mycount = 0;
    if (active && want_compact && npass > 0) {
        for (int base = r_begin; base < r_end; base += 32) {
            const int i = base + wl;
            float sc;
            const bool k = (i < r_end) && keep_of(i, sc);
            mycount += __popc(__ballot_sync(0xffffffffu, k));
        }
    }
    if (wl == 0) s_segcnt[warp] = mycount;
    __syncthreads();
    if (active) {
        int offset = 0, total_cnt = 0;
        for (int s = 0; s < NSEG; ++s) {
            const int c = s_segcnt[s * GT + j];
            if (s < seg) offset += c;
            total_cnt += c;
        }
        const size_t out_base = (size_t)qh * cap_children + tile_c0;
        if (want_compact || P.out_dense) {
            for (int base = r_begin; base < r_end; base += 32) {
                const int i = base + wl;
                float sc = 0.f;
                const bool k = (i < r_end) && (npass > 0) && keep_of(i, sc);
                const float emitted = __fmul_rn(sc, scale);
                if (want_compact) {
                    const uint32_t b = __ballot_sync(0xffffffffu, k);
                    if (k) {
                        const int pos = offset + __popc(b & ((1u << wl) - 1u));
                        P.out_idx[out_base + pos] = (int32_t)(tile_c0 + i);
                        P.out_score[out_base + pos] = emitted;
                    }
                    offset += __popc(b);
                }
                if (P.out_dense && i < r_end && tile_c0 + i < cap_children)
                    P.out_dense[out_base + i] = k ? emitted : 0.f;
            }
        }
        if (seg == 0 && wl == 0) {
            if (want_compact) P.out_count[(size_t)qh * P.n_tiles + tile] = total_cnt;
            if (P.stats) {
                uint32_t* st = P.stats + (size_t)qh * 8;
                for (int k = 0; k < 8; ++k)
                    if (k != 5 && s_stat[j][k]) atomicAdd(st + k, s_stat[j][k]);
                if (total_cnt) atomicAdd(st + 5, (uint32_t)total_cnt);
            }
        }
    }
}

template <typename T, int GT, int NCH>
static int launch_search(const SearchParams& P, int chunks, size_t smem, cudaStream_t stream) {
    auto kern = search_kernel<T, GT, NCH>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("hira_search: cudaFuncSetAttribute(%zu B smem): %s", smem, cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
    }
    dim3 grid((unsigned)(P.n_heads * P.n_tiles), (unsigned)chunks);
    kern<<<grid, SEARCH_THREADS, smem, stream>>>(P);
    HIRA_CHECK_LAUNCH("hira_search launch");
    return HIRA_OK;
}

template <typename T, int NCH>
static int dispatch_gt(const SearchParams& P, int max_group, cudaStream_t stream) {
    int gt = 1;
    while (gt < max_group && gt < 8) gt <<= 1;
    if (NCH == 2 && gt > 4) gt = 4;  // keep the register budget
    const int chunks = (max_group + gt - 1) / gt;
    const size_t tile_rows = (size_t)P.tile_parents * P.bf;
    const size_t smem = tile_rows * gt * sizeof(float) + (size_t)P.tile_parents * (4 + 2 + 1 + 1) + 16;
    switch (gt) {
        case 1: return launch_search<T, 1, NCH>(P, chunks, smem, stream);
        case 2: return launch_search<T, 2, NCH>(P, chunks, smem, stream);
        case 4: return launch_search<T, 4, NCH>(P, chunks, smem, stream);
        default: return launch_search<T, 8, 1>(P, chunks, smem, stream);
    }
}

}  // namespace hira

using namespace hira;

extern "C" int hira_search_tile_parents(const hira_index_t* ix) {
    if (!ix || ix->bf < 1 || ix->bf > MAX_TILE_ROWS) return HIRA_ERR_ARG;
    const int bf = ix->bf;
    int tp;
    if (bf * bf <= MAX_TILE_ROWS) {
        // whole grandparents per tile
        tp = bf * (MAX_TILE_ROWS / (bf * bf));
    } else {
        // largest divisor of bf with tp*bf <= MAX_TILE_ROWS
        tp = 1;
        for (int d = 1; d <= MAX_TILE_ROWS / bf; ++d)
            if (bf % d == 0) tp = d;
    }
    if (tp > ix->cap_parents && ix->cap_parents > 0) {
        // small index: one tile, still aligned to grandparent blocks
        tp = ix->depth == 3 ? ((ix->cap_parents + bf - 1) / bf) * bf : ix->cap_parents;
        if (tp * bf > MAX_TILE_ROWS) tp = bf * (MAX_TILE_ROWS / (bf * bf) > 0 ? MAX_TILE_ROWS / (bf * bf) : 1);
    }
    return tp;
}

extern "C" int hira_search(const hira_index_t* ix, const float* q, const float* tau,
                           const float* scaling, const float* qnorm, const int32_t* q2kv,
                           int32_t n_qheads, int32_t max_group, int32_t flags,
                           int32_t tile_parents, float* out_dense, int32_t* out_idx,
                           float* out_score, int32_t* out_count, uint32_t* stats, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(q && tau, HIRA_ERR_ARG, "hira_search: q and tau must not be NULL");
    HIRA_CHECK_ARG(n_qheads >= 1, HIRA_ERR_SHAPE, "hira_search: n_qheads=%d must be >= 1", n_qheads);
    HIRA_CHECK_ARG((flags & ~0x7) == 0 && (flags & 0x6) != 0x6, HIRA_ERR_ARG, "hira_search: bad flags 0x%x", flags);
    const bool any_compact = out_idx || out_score || out_count;
    HIRA_CHECK_ARG(!any_compact || (out_idx && out_score && out_count), HIRA_ERR_ARG,
                   "hira_search: out_idx, out_score and out_count must be given together");
    HIRA_CHECK_ARG(any_compact || out_dense, HIRA_ERR_ARG, "hira_search: no output buffer given");
    const int bf = ix->bf;
    HIRA_CHECK_ARG(tile_parents >= 1 && (long long)tile_parents * bf <= MAX_TILE_ROWS, HIRA_ERR_SHAPE,
                   "hira_search: tile_parents=%d with bf=%d exceeds %d rows per tile", tile_parents, bf, MAX_TILE_ROWS);
    HIRA_CHECK_ARG(ix->depth == 2 || tile_parents % bf == 0 || bf % tile_parents == 0, HIRA_ERR_SHAPE,
                   "hira_search: depth-3 tiles must align with grandparent blocks (tile_parents=%d, bf=%d)",
                   tile_parents, bf);
    int group;
    if (q2kv == nullptr) {
        HIRA_CHECK_ARG(n_qheads % ix->n_heads == 0, HIRA_ERR_SHAPE,
                       "hira_search: n_qheads=%d not divisible by n_heads=%d and no q2kv given", n_qheads, ix->n_heads);
        group = n_qheads / ix->n_heads;
        max_group = group;
    } else {
        group = 0;
        if (max_group <= 0 || max_group > n_qheads) max_group = n_qheads;
    }
    SearchParams P;
    P.children = ix->children; P.parents = ix->parents; P.gps = ix->grand_parents;
    P.parent_radii = ix->parent_radii; P.gp_radii = ix->gp_radii;
    P.child_counts = ix->child_counts; P.gp_counts = ix->gp_counts; P.used = ix->used;
    P.q = q; P.tau = tau; P.scaling = scaling; P.qnorm = qnorm; P.q2kv = q2kv;
    P.out_dense = out_dense; P.out_idx = out_idx; P.out_score = out_score; P.out_count = out_count;
    P.stats = stats;
    P.n_heads = ix->n_heads; P.n_qheads = n_qheads; P.group = group; P.depth = ix->depth;
    P.bf = bf; P.dim = ix->dim; P.cap_parents = ix->cap_parents; P.cap_gp = ix->cap_gp;
    P.tile_parents = tile_parents;
    P.n_tiles = (ix->cap_parents + tile_parents - 1) / tile_parents;
    P.flags = flags;
    P.bf_magic = (uint32_t)((0x100000000ull + (uint64_t)bf - 1) / (uint64_t)bf);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool two = ix->dim > 128;
    if (ix->dtype == HIRA_BF16)
        return two ? dispatch_gt<__nv_bfloat16, 2>(P, max_group, s) : dispatch_gt<__nv_bfloat16, 1>(P, max_group, s);
    return two ? dispatch_gt<float, 2>(P, max_group, s) : dispatch_gt<float, 1>(P, max_group, s);
}
