// Decode-time key insertion: nearest valid parent, slot claim, K/V row write,
// radius widening up the path, overflow into pre-allocated spare blocks.
//
// Follows CUDAIndexer.update (indexer/cuda.py:544-701, 1200-1231) and its
// Triton kernels (kernels/triton_update_kernels.py:6-364):
//   score(p) = ||c_p||^2 - 2 x.c_p over valid parents, arg-min, ties -> lowest p
//   free slot  -> children[p*bf + count] = x, count += 1,
//                 r_p = max(r_p, ||x - c_p||), r_g = max(r_g, ||c_p - c_g|| + r_p)
//   parent full -> x becomes a new parent (centre x, radius 0, one child); with
//                 three levels it goes under the nearest grandparent if that has
//                 a free parent slot, else under a new grandparent (centre x).
// Differences by design: counts, validity and ||c||^2 are persistent device
// state (the reference recomputes them by scanning the whole index after every
// call, indexer/cuda.py:1233-1298), the arrays are pre-allocated (no torch.cat
// growth, :644-657) and nothing synchronises with the host.  One CTA owns one
// head and inserts its keys one after another, so results are deterministic.
#include "common.cuh"
#include <math_constants.h>

namespace hira {

constexpr int APPEND_THREADS = 512;
constexpr int APPEND_HW = APPEND_THREADS / GROUP;  // 8-lane groups: one centre row per group per step
constexpr int APPEND_UNROLL = 4;

struct BestRec;
struct AppendParams {
    hira_index_t ix;
    const void* new_k;
    const void* new_v;
    int n_new;
    long long k_head_stride, v_head_stride;
    int token_base;
    int32_t* status;
    // two-kernel path: partial arg-mins of the scan kernel, [head][key][part], or NULL
    struct BestRec* partial;
    int n_parts;
    unsigned long long* scan;  // [n_heads] nearest valid parent found by hira_search_scan (n_new == 1), or NULL
    uint32_t bf_magic;  // ceil(2^32 / bf): p / bf == __umulhi(p, bf_magic) for p < 2^20 (0: divide)
};

struct BestRec { float s; int i; };
constexpr int APPEND_MAX_STAGED = 32;  // keys per call the two-kernel path handles

struct Best { float s; int i; };

__device__ __forceinline__ bool better(float s, int i, const Best& b) {
    return s < b.s || (s == b.s && i < b.i);
}

// arg-min of sq[p] - 2 x.c_p over p in [0, n) with valid(p); all threads get it.
// Rows, norms and validity are fetched side by side (an invalid slot inside the scanned
// range is an all-zero row, so reading it is harmless); validity only masks the compare.
template <typename T, int NCH, int TH, typename Valid>
__device__ Best nearest_row(const T* rows, const float* sq, int n, const float (&x)[NCH][8], int dim,
                            Valid valid, Best* s_best) {
    constexpr int NG = TH / GROUP;
    const int tid = threadIdx.x, lane = tid & (GROUP - 1), hw = tid / GROUP;
    Best best{CUDART_INF_F, 0x7fffffff};
    for (int p0 = 0; p0 < n; p0 += NG * APPEND_UNROLL) {  // uniform trip count
        RawChunk<T> raw[APPEND_UNROLL][NCH];
        bool ok[APPEND_UNROLL];
        float sqv[APPEND_UNROLL];
#pragma unroll
        for (int u = 0; u < APPEND_UNROLL; ++u) {
            const int p = p0 + u * NG + hw;
            const bool in = p < n;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int c = lane + GROUP * i;
                if (in && c * 8 < dim) raw[u][i] = load_chunk_coherent<T>(rows + (size_t)p * dim, c);
                else raw[u][i] = zero_chunk<T>();
            }
            sqv[u] = in ? sq[p] : 0.f;
            ok[u] = in && valid(p);
        }
#pragma unroll
        for (int u = 0; u < APPEND_UNROLL; ++u) {
            const int p = p0 + u * NG + hw;
            Acc2 acc{0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                float a[8];
                to_float(raw[u][i], a);
                chunk_fma(acc, a, x[i]);
            }
            const float d = group_sum(__fadd_rn(acc.e, acc.o));
            const float s = __fsub_rn(sqv[u], __fmul_rn(2.0f, d));
            if (ok[u] && better(s, p, best)) best = Best{s, p};
        }
    }
    __syncthreads();
    if (lane == 0) s_best[hw] = best;
    __syncthreads();
    Best b = s_best[0];
    for (int w = 1; w < NG; ++w)
        if (better(s_best[w].s, s_best[w].i, b)) b = s_best[w];
    __syncthreads();
    return b;
}

// Stage 1 of the two-kernel path: CTA (part, head) scans its slice of the parents that are
// valid when the call starts, for every new key, and writes one partial arg-min each.  The
// parents a call creates itself are not in this scan; stage 2 adds them from its own list.
constexpr int SCAN_THREADS = 256;

template <typename T, int NCH>
__global__ void __launch_bounds__(SCAN_THREADS, NCH == 2 ? 3 : 1)
append_scan_kernel(const AppendParams P) {
    __shared__ Best s_best[SCAN_THREADS / GROUP];
    const hira_index_t& ix = P.ix;
    const int h = blockIdx.y, part = blockIdx.x;
    const int lane = threadIdx.x & (GROUP - 1);
    const int bf = ix.bf, dim = ix.dim;
    const size_t capP = ix.cap_parents, capG = ix.cap_gp;
    const T* parents = reinterpret_cast<const T*>(ix.parents) + (size_t)h * capP * dim;
    const float* psq = ix.parent_sqnorm + (size_t)h * capP;
    const int32_t* gc = ix.depth == 3 ? ix.gp_counts + (size_t)h * capG : nullptr;
    const int32_t* used = ix.used + (size_t)h * 4;
    const int n_scan = ix.depth == 3 ? used[1] * bf : used[0];
    const int per = (n_scan + P.n_parts - 1) / P.n_parts;
    const int lo = min(n_scan, part * per), hi = min(n_scan, lo + per);
    const T* new_k = reinterpret_cast<const T*>(P.new_k) + (size_t)h * P.k_head_stride;
    for (int key = 0; key < P.n_new; ++key) {
        float x[NCH][8];
        load_vec<T, NCH>(new_k + (size_t)key * dim, x, lane, dim);
        Best b;
        if (ix.depth == 3)
            b = nearest_row<T, NCH, SCAN_THREADS>(parents + (size_t)lo * dim, psq + lo, hi - lo, x, dim,
                                                  [&](int p) {
                                                      const int pp = p + lo;
                                                      const int g = P.bf_magic ? (int)__umulhi((uint32_t)pp, P.bf_magic) : pp / bf;
                                                      return (pp - g * bf) < gc[g];
                                                  }, s_best);
        else
            b = nearest_row<T, NCH, SCAN_THREADS>(parents + (size_t)lo * dim, psq + lo, hi - lo, x, dim,
                                                  [&](int) { return true; }, s_best);
        if (threadIdx.x == 0) {
            BestRec r;
            r.s = b.s;
            r.i = b.i == 0x7fffffff ? b.i : b.i + lo;
            P.partial[((size_t)h * P.n_new + key) * P.n_parts + part] = r;
        }
    }
}

template <typename T, typename TV, int NCH, int NVCH>
__global__ void __launch_bounds__(APPEND_THREADS)
append_kernel(const AppendParams P) {
    __shared__ Best s_best[APPEND_HW];
    __shared__ int s_newp[APPEND_MAX_STAGED];  // parents created earlier in this call (two-kernel path)
    int n_newp = 0;
    const hira_index_t& ix = P.ix;
    const int h = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & (GROUP - 1), hw = tid / GROUP;
    const int bf = ix.bf, dim = ix.dim, vdim = ix.vdim;
    const size_t capP = ix.cap_parents, capC = capP * bf, capG = ix.cap_gp;
    T* children = reinterpret_cast<T*>(ix.children) + (size_t)h * capC * dim;
    T* parents = reinterpret_cast<T*>(ix.parents) + (size_t)h * capP * dim;
    T* gps = ix.depth == 3 ? reinterpret_cast<T*>(ix.grand_parents) + (size_t)h * capG * dim : nullptr;
    TV* values = ix.values ? reinterpret_cast<TV*>(ix.values) + (size_t)h * capC * vdim : nullptr;
    float* pr = ix.parent_radii + (size_t)h * capP;
    float* psq = ix.parent_sqnorm + (size_t)h * capP;
    int32_t* cc = ix.child_counts + (size_t)h * capP;
    float* gr = ix.depth == 3 ? ix.gp_radii + (size_t)h * capG : nullptr;
    float* gsq = ix.depth == 3 ? ix.gp_sqnorm + (size_t)h * capG : nullptr;
    int32_t* gc = ix.depth == 3 ? ix.gp_counts + (size_t)h * capG : nullptr;
    int32_t* used = ix.used + (size_t)h * 4;
    int32_t* s2t = ix.slot2token ? ix.slot2token + (size_t)h * capC : nullptr;
    const T* new_k = reinterpret_cast<const T*>(P.new_k) + (size_t)h * P.k_head_stride;
    const TV* new_v = P.new_v ? reinterpret_cast<const TV*>(P.new_v) + (size_t)h * P.v_head_stride : nullptr;

    for (int key = 0; key < P.n_new; ++key) {
        // every thread reads the state written by thread 0 in the previous round
        int used_p = used[0];
        int used_g = used[1];
        const int n_keys = used[2];
        float x[NCH][8];
        load_vec<T, NCH>(new_k + (size_t)key * dim, x, lane, dim);

        // ---- nearest valid parent ---------------------------------------------
        Best bp;
        if (P.scan != nullptr) {
            // found by the search that ran just before on the same index state
            const unsigned long long k = P.scan[h];
            bp = (k == ~0ull) ? Best{CUDART_INF_F, 0x7fffffff}
                              : Best{key_to_float((uint32_t)(k >> 32)), (int)(uint32_t)(k & 0xffffffffu)};
            __syncthreads();                      // every thread has read the slot
            if (tid == 0) P.scan[h] = ~0ull;      // ready for the next search
        } else if (P.partial != nullptr) {
            // arg-min over the scanned slices, then over the parents this call created itself
            bp = Best{CUDART_INF_F, 0x7fffffff};
            const BestRec* pr_ = P.partial + ((size_t)h * P.n_new + key) * P.n_parts;
            for (int s2 = 0; s2 < P.n_parts; ++s2) {
                const BestRec r = pr_[s2];
                if (better(r.s, r.i, bp)) bp = Best{r.s, r.i};
            }
            for (int e = 0; e < n_newp; ++e) {  // uniform trip count; every group computes the same row
                const int p = s_newp[e];
                Acc2 acc{0.f, 0.f};
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const int c = lane + GROUP * i;
                    if (c * 8 < dim) {
                        float a[8];
                        to_float(load_chunk_coherent<T>(parents + (size_t)p * dim, c), a);
                        chunk_fma(acc, a, x[i]);
                    }
                }
                const float d = group_sum(__fadd_rn(acc.e, acc.o));
                const float sc = __fsub_rn(psq[p], __fmul_rn(2.0f, d));
                if (better(sc, p, bp)) bp = Best{sc, p};
            }
        } else if (ix.depth == 3) {
            const int n_scan = used_g * bf;
            bp = nearest_row<T, NCH, APPEND_THREADS>(parents, psq, n_scan, x, dim,
                                     [&](int p) {
                                         const int g = P.bf_magic ? (int)__umulhi((uint32_t)p, P.bf_magic) : p / bf;
                                         return (p - g * bf) < gc[g];
                                     }, s_best);
        } else {
            bp = nearest_row<T, NCH, APPEND_THREADS>(parents, psq, used_p, x, dim, [&](int) { return true; }, s_best);
        }
        const bool have_parent = bp.i != 0x7fffffff;
        const bool placed = have_parent && cc[bp.i] < bf;

        int p_dst = -1, g_dst = -1;
        bool new_gp = false;
        if (!placed) {
            if (ix.depth == 3) {
                // nearest grandparent among those in use (no validity mask: indexer/cuda.py:918-920)
                const Best bg = nearest_row<T, NCH, APPEND_THREADS>(gps, gsq, used_g, x, dim, [&](int) { return true; }, s_best);
                if (bg.i != 0x7fffffff && gc[bg.i] < bf) {
                    g_dst = bg.i;
                    p_dst = g_dst * bf + gc[g_dst];
                } else if (used_g < (int)capG) {
                    g_dst = used_g;
                    p_dst = g_dst * bf;
                    new_gp = true;
                } else {
                    if (tid == 0) atomicOr(P.status, HIRA_STATUS_GP_FULL);
                }
            } else {
                if (used_p < (int)capP) p_dst = used_p;
                else if (tid == 0) atomicOr(P.status, HIRA_STATUS_PARENTS_FULL);
            }
        }
        __syncthreads();  // all reads of the old state are done

        // the int8 side copy of the new child row (dim == 128), by the 8 lanes of group 0; the row's
        // values are those just stored (x holds the key in the index dtype's precision)
        auto write_q8 = [&](int slot) {
            if constexpr (NCH == 2) {
                if (ix.children_q8 != nullptr) {
                    const size_t at = (size_t)h * capC + slot;
                    q8_write_row(x, ix.q8_chan_scale + (size_t)h * HIRA_Q8_CHAN,
                                 reinterpret_cast<int8_t*>(ix.children_q8) + at * 128,
                                 reinterpret_cast<uint32_t*>(ix.children_q8_meta) + at, slot & 7, lane);
                }
            }
        };
        // ---- warp 0 applies the insertion ---------------------------------------
        if (tid < 32) {
            const int token = P.token_base < 0 ? n_keys : P.token_base + key;
            if (placed) {
                const int p = bp.i;
                const int slot = p * bf + cc[p];
                const float d2 = row_dist2_reg<T, NCH>(parents + (size_t)p * dim, x, lane, dim);
                const float r_new = fmaxf(pr[p], __fsqrt_rn(d2));
                float rg_new = 0.f;
                if (ix.depth == 3) {
                    const int g = p / bf;
                    const float dg2 = row_dist2_coherent<T, T, NCH>(parents + (size_t)p * dim, gps + (size_t)g * dim, lane, dim);
                    rg_new = fmaxf(gr[g], __fadd_rn(__fsqrt_rn(dg2), r_new));
                }
                if (hw == 0) {
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const int c = lane + GROUP * i;
                        if (c * 8 < dim) store_chunk(children + (size_t)slot * dim, c, x[i]);
                    }
                    write_q8(slot);
                    if (values) {
#pragma unroll
                        for (int i = 0; i < NVCH; ++i) {
                            const int c = lane + GROUP * i;
                            if (c * 8 < vdim) {
                                float v[8];
                                to_float(load_chunk<TV>(new_v + (size_t)key * vdim, c), v);
                                store_chunk(values + (size_t)slot * vdim, c, v);
                            }
                        }
                    }
                    if (lane == 0) {
                        pr[p] = r_new;
                        if (ix.depth == 3) gr[p / bf] = rg_new;
                        cc[p] += 1;
                        used[2] = n_keys + 1;
                        if (s2t) s2t[slot] = token;
                    }
                }
            } else if (p_dst >= 0) {
                const int slot = p_dst * bf;
                const float xsq = reg_sqnorm<NCH>(x);
                float rg_new = 0.f;
                if (ix.depth == 3 && !new_gp) {
                    const float dg2 = row_dist2_reg<T, NCH>(gps + (size_t)g_dst * dim, x, lane, dim);
                    rg_new = fmaxf(gr[g_dst], __fsqrt_rn(dg2));  // ||x - g|| + radius 0
                }
                if (hw == 0) {
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const int c = lane + GROUP * i;
                        if (c * 8 < dim) {
                            store_chunk(children + (size_t)slot * dim, c, x[i]);
                            store_chunk(parents + (size_t)p_dst * dim, c, x[i]);
                            if (new_gp) store_chunk(gps + (size_t)g_dst * dim, c, x[i]);
                        }
                    }
                    write_q8(slot);
                    if (values) {
#pragma unroll
                        for (int i = 0; i < NVCH; ++i) {
                            const int c = lane + GROUP * i;
                            if (c * 8 < vdim) {
                                float v[8];
                                to_float(load_chunk<TV>(new_v + (size_t)key * vdim, c), v);
                                store_chunk(values + (size_t)slot * vdim, c, v);
                            }
                        }
                    }
                    if (lane == 0) {
                        pr[p_dst] = 0.f;
                        psq[p_dst] = xsq;
                        cc[p_dst] = 1;
                        if (ix.depth == 3) {
                            if (new_gp) {
                                gr[g_dst] = 0.f;
                                gsq[g_dst] = xsq;
                                gc[g_dst] = 1;
                                used[1] = used_g + 1;
                            } else {
                                gr[g_dst] = rg_new;
                                gc[g_dst] += 1;
                            }
                        }
                        if (p_dst + 1 > used_p) used[0] = p_dst + 1;
                        used[2] = n_keys + 1;
                        if (s2t) s2t[slot] = token;
                    }
                }
            }
        }
        if (!placed && p_dst >= 0 && P.partial != nullptr && n_newp < APPEND_MAX_STAGED) {
            if (tid == 0) s_newp[n_newp] = p_dst;
            ++n_newp;
        }
        __syncthreads();  // make the insertion visible to the next key's scan
    }
}

template <typename T, typename TV>
static int launch_append(const AppendParams& P, cudaStream_t s) {
    const bool k2 = P.ix.dim > 128, v2 = P.ix.vdim > 128;   // chunks per lane: 2 up to 128 elements, else 4
    const int grid = P.ix.n_heads;
    if (P.partial != nullptr) {
        dim3 g1((unsigned)P.n_parts, (unsigned)P.ix.n_heads);
        if (k2) append_scan_kernel<T, 4><<<g1, SCAN_THREADS, 0, s>>>(P);
        else append_scan_kernel<T, 2><<<g1, SCAN_THREADS, 0, s>>>(P);
        HIRA_CHECK_LAUNCH("hira_append scan launch");
    }
    if (!k2 && !v2) append_kernel<T, TV, 2, 2><<<grid, APPEND_THREADS, 0, s>>>(P);
    else if (k2 && !v2) append_kernel<T, TV, 4, 2><<<grid, APPEND_THREADS, 0, s>>>(P);
    else if (!k2 && v2) append_kernel<T, TV, 2, 4><<<grid, APPEND_THREADS, 0, s>>>(P);
    else append_kernel<T, TV, 4, 4><<<grid, APPEND_THREADS, 0, s>>>(P);
    HIRA_CHECK_LAUNCH("hira_append launch");
    return HIRA_OK;
}

}  // namespace hira

using namespace hira;

static int append_parts(const hira_index_t* ix) {
    // enough CTAs to fill the GPU, slices of at least 128 parents
    int parts = (8 * 148 + ix->n_heads - 1) / ix->n_heads;
    const int max_parts = ix->cap_parents / 128;
    if (parts > max_parts) parts = max_parts;
    if (parts > 64) parts = 64;
    return parts < 1 ? 1 : parts;
}

extern "C" size_t hira_append_workspace_bytes(const hira_index_t* ix, int32_t n_new) {
    if (!ix || n_new < 1 || n_new > APPEND_MAX_STAGED || ix->n_heads < 1 || ix->cap_parents < 1) return 0;
    return (size_t)ix->n_heads * n_new * append_parts(ix) * sizeof(BestRec);
}

extern "C" int hira_append(const hira_index_t* ix, const void* new_k, const void* new_v, int32_t n_new,
                           int64_t k_head_stride, int64_t v_head_stride, int32_t token_base,
                           int32_t* status, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(new_k && status, HIRA_ERR_ARG, "hira_append: new_k and status must not be NULL");
    HIRA_CHECK_ARG(n_new >= 0, HIRA_ERR_SHAPE, "hira_append: n_new=%d", n_new);
    HIRA_CHECK_ARG((ix->values == nullptr) == (new_v == nullptr), HIRA_ERR_ARG,
                   "hira_append: values must be given iff the index stores values");
    HIRA_CHECK_ARG(ix->parent_sqnorm && (ix->depth == 2 || ix->gp_sqnorm), HIRA_ERR_ARG,
                   "hira_append: the index needs its parent_sqnorm / gp_sqnorm caches");
    if (n_new == 0) return HIRA_OK;
    AppendParams P;
    P.ix = *ix; P.new_k = new_k; P.new_v = new_v; P.n_new = n_new;
    P.k_head_stride = k_head_stride; P.v_head_stride = v_head_stride;
    P.token_base = token_base; P.status = status;
    P.partial = nullptr; P.n_parts = 0; P.scan = nullptr;
    P.bf_magic = (ix->bf > 1 && ix->cap_parents < (1 << 20))
                     ? (uint32_t)((0x100000000ull + (uint64_t)ix->bf - 1) / (uint64_t)ix->bf) : 0u;
    const size_t need = hira_append_workspace_bytes(ix, n_new);
    if (workspace != nullptr && need > 0 && workspace_bytes >= need && append_parts(ix) > 1) {
        P.partial = reinterpret_cast<BestRec*>(workspace);
        P.n_parts = append_parts(ix);
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool kb = ix->dtype == HIRA_BF16, vb = ix->vdtype == HIRA_BF16 || !ix->values;
    if (kb && vb) return launch_append<__nv_bfloat16, __nv_bfloat16>(P, s);
    if (kb && !vb) return launch_append<__nv_bfloat16, float>(P, s);
    if (!kb && vb && ix->values) return launch_append<float, __nv_bfloat16>(P, s);
    return launch_append<float, float>(P, s);
}

extern "C" int hira_append_scanned(const hira_index_t* ix, const void* new_k, const void* new_v,
                                   int64_t k_head_stride, int64_t v_head_stride, int32_t token_base,
                                   int32_t* status, uint64_t* scan, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(new_k && status && scan, HIRA_ERR_ARG, "hira_append_scanned: new_k, status and scan must not be NULL");
    HIRA_CHECK_ARG((ix->values == nullptr) == (new_v == nullptr), HIRA_ERR_ARG,
                   "hira_append_scanned: values must be given iff the index stores values");
    HIRA_CHECK_ARG(ix->parent_sqnorm && (ix->depth == 2 || ix->gp_sqnorm), HIRA_ERR_ARG,
                   "hira_append_scanned: the index needs its parent_sqnorm / gp_sqnorm caches");
    AppendParams P;
    P.ix = *ix; P.new_k = new_k; P.new_v = new_v; P.n_new = 1;
    P.k_head_stride = k_head_stride; P.v_head_stride = v_head_stride;
    P.token_base = token_base; P.status = status;
    P.partial = nullptr; P.n_parts = 0;
    P.scan = reinterpret_cast<unsigned long long*>(scan);
    P.bf_magic = (ix->bf > 1 && ix->cap_parents < (1 << 20))
                     ? (uint32_t)((0x100000000ull + (uint64_t)ix->bf - 1) / (uint64_t)ix->bf) : 0u;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool kb = ix->dtype == HIRA_BF16, vb = ix->vdtype == HIRA_BF16 || !ix->values;
    if (kb && vb) return launch_append<__nv_bfloat16, __nv_bfloat16>(P, s);
    if (kb && !vb) return launch_append<__nv_bfloat16, float>(P, s);
    if (!kb && vb && ix->values) return launch_append<float, __nv_bfloat16>(P, s);
    return launch_append<float, float>(P, s);
}
