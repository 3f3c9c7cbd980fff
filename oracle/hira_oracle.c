/*
 * hira_oracle.c -- CPU restatement of the reference's algorithms for the
 * decode hot path.  TEST INFRASTRUCTURE ONLY: the checker that tests/,
 * __graft_entry__.smoke() and bench.py's cpu_baseline leg compare the CUDA
 * library against.  Nothing in the product path may call into it.
 *
 * Every function works on HOST memory and uses the same hira_index_t struct
 * (include/hira_b200.h) with host pointers, so an index can be copied between
 * the device library and the oracle array by array.
 *
 * Arithmetic: the reference's CPU kernels are built with -ffast-math and an
 * `omp simd` reduction (kernels/cpp/torch_ext_loader.py:37-67,
 * kernels/cpp/torch_ext_v3.cpp:24-34) and its GPU kernels use tl.sum
 * (kernels/triton_search_kernels.py:46,60), so the reference itself fixes no
 * summation order.  The oracle fixes one -- the "canonical tree" below, the
 * same one the CUDA kernels evaluate -- so that library-vs-oracle comparisons
 * are bit-exact; oracle-vs-reference comparisons use guard-banded thresholds
 * (tests/golden).
 *
 * Parity pins: tests/golden/ holds outputs of the reference's own
 * fused_tree_search_v3 (C++), two_level_filter kernels (Triton interpreter),
 * update kernels and radius routines on seeded inputs; tests/test_oracle_golden.py
 * checks this file against them.  The attention and threshold functions have no
 * reference implementation to pin against (attention/hira_attention.py:1-3,
 * cache/threshold_finder.py:1-14): parity unpinned for those two.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/hira_b200.h"

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- element access -------------------------------------------------------- */
static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) { /* round to nearest even, NaN kept quiet */
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float ld(const void* base, int dtype, size_t i) {
    return dtype == HIRA_BF16 ? bf16_to_f32(((const uint16_t*)base)[i]) : ((const float*)base)[i];
}
static inline void st(void* base, int dtype, size_t i, float v) {
    if (dtype == HIRA_BF16) ((uint16_t*)base)[i] = f32_to_bf16(v);
    else ((float*)base)[i] = v;
}
static void load_row(const void* base, int dtype, size_t row, int dim, float* out) {
    for (int d = 0; d < dim; ++d) out[d] = ld(base, dtype, row * (size_t)dim + d);
}

/* ---- canonical dot product ---------------------------------------------------
 * 8 lanes; lane l owns the 8-element chunks c with c % 8 == l; per lane an even
 * and an odd FMA chain over its chunks in increasing order; lane partial =
 * even + odd; butterfly over the lanes with strides 4, 2, 1. */
float oracle_dot(const float* a, const float* b, int dim) {
    float p[8];
    for (int l = 0; l < 8; ++l) {
        float e = 0.0f, o = 0.0f;
        for (int c = l; c * 8 < dim; c += 8) {
            for (int j = 0; j < 4; ++j) {
                e = fmaf(a[8 * c + 2 * j], b[8 * c + 2 * j], e);
                o = fmaf(a[8 * c + 2 * j + 1], b[8 * c + 2 * j + 1], o);
            }
        }
        p[l] = e + o;
    }
    for (int s = 4; s >= 1; s >>= 1) {
        float t[8];
        for (int l = 0; l < 8; ++l) t[l] = p[l] + p[l ^ s];
        memcpy(p, t, sizeof(p));
    }
    return p[0];
}
static float dist2(const float* a, const float* b, int dim) { /* canonical ||a-b||^2 */
    float d[256];
    for (int i = 0; i < dim; ++i) d[i] = a[i] - b[i];
    return oracle_dot(d, d, dim);
}
/* the assignment's arithmetic: one sequential FMA chain */
static float dot_seq(const float* a, const float* b, int dim) {
    float acc = 0.0f;
    for (int d = 0; d < dim; ++d) acc = fmaf(a[d], b[d], acc);
    return acc;
}

static int parent_valid(const hira_index_t* ix, int h, int p) {
    if (p < 0 || p >= ix->cap_parents) return 0;
    if (ix->depth == 3) {
        const int g = p / ix->bf;
        return g < ix->used[h * 4 + 1] && (p - g * ix->bf) < ix->gp_counts[(size_t)h * ix->cap_gp + g];
    }
    return p < ix->used[h * 4 + 0];
}

static int gate(float dot, float r, const float* qnorm, int qh, float tau, int ge) {
    const float rr = qnorm ? qnorm[qh] * r : r;
    const float s = dot + rr;
    return ge ? (s >= tau) : (s > tau);
}

/* ---- search over the blocked layout --------------------------------------------
 * Gate and emission rules: kernels/triton_search_kernels.py:6-63 (two levels),
 * :66-148 (three levels): prune a node iff dot + r <= tau, emit scaling*dot for
 * every child of a kept parent.  With HIRA_GATE_GE / HIRA_LEAF_GE the rules of
 * kernels/cpp/torch_ext_v3.cpp:177-241: keep iff dot + r >= tau, emit iff
 * dot >= tau.  out_dense[qh][slot] = emitted score or 0; out_keep[qh][slot] = 1
 * where emitted (either may be NULL). */
int oracle_search(const hira_index_t* ix, const float* q, const float* tau, const float* scaling,
                  const float* qnorm, const int32_t* q2kv, int n_qheads, int flags, float* out_dense,
                  uint8_t* out_keep, uint32_t* stats) {
    const int bf = ix->bf, dim = ix->dim;
    const size_t capC = (size_t)ix->cap_parents * bf;
    const int ge = flags & HIRA_GATE_GE;
    const int leaf = flags & (HIRA_LEAF_GE | HIRA_LEAF_GT);
    const int group = q2kv ? 1 : n_qheads / ix->n_heads;
    if (out_dense) memset(out_dense, 0, sizeof(float) * n_qheads * capC);
    if (out_keep) memset(out_keep, 0, (size_t)n_qheads * capC);
#pragma omp parallel for schedule(dynamic, 1)
    for (int qh = 0; qh < n_qheads; ++qh) {
        const int h = q2kv ? q2kv[qh] : qh / group;
        const float* qv = q + (size_t)qh * dim;
        const float sc = scaling ? scaling[qh] : 1.0f;
        float row[256];
        const int n_gp = ix->depth == 3 ? ix->used[h * 4 + 1] : 1;
        for (int g = 0; g < n_gp; ++g) {
            int p_begin = 0, p_end = ix->used[h * 4 + 0];
            if (ix->depth == 3) {
                load_row(ix->grand_parents, ix->dtype, (size_t)h * ix->cap_gp + g, dim, row);
                const float d = oracle_dot(row, qv, dim);
                if (stats) stats[qh * 8 + 0]++;
                if (!gate(d, ix->gp_radii[(size_t)h * ix->cap_gp + g], qnorm, qh, tau[qh], ge)) continue;
                if (stats) stats[qh * 8 + 1]++;
                p_begin = g * bf;
                p_end = p_begin + bf;
            }
            for (int p = p_begin; p < p_end; ++p) {
                if (!parent_valid(ix, h, p)) continue;
                load_row(ix->parents, ix->dtype, (size_t)h * ix->cap_parents + p, dim, row);
                const float d = oracle_dot(row, qv, dim);
                if (stats) stats[qh * 8 + 2]++;
                if (!gate(d, ix->parent_radii[(size_t)h * ix->cap_parents + p], qnorm, qh, tau[qh], ge)) continue;
                int cnt = ix->child_counts[(size_t)h * ix->cap_parents + p];
                if (cnt > bf) cnt = bf;
                if (stats) { stats[qh * 8 + 3]++; stats[qh * 8 + 4] += cnt; }
                for (int c = 0; c < cnt; ++c) {
                    const size_t slot = (size_t)p * bf + c;
                    load_row(ix->children, ix->dtype, (size_t)h * capC + slot, dim, row);
                    const float s = oracle_dot(row, qv, dim);
                    int keep = 1;
                    if (leaf == HIRA_LEAF_GE) keep = s >= tau[qh];
                    else if (leaf == HIRA_LEAF_GT) keep = s > tau[qh];
                    if (!keep) continue;
                    if (stats) stats[qh * 8 + 5]++;
                    if (out_dense) out_dense[(size_t)qh * capC + slot] = s * sc;
                    if (out_keep) out_keep[(size_t)qh * capC + slot] = 1;
                }
            }
        }
    }
    return 0;
}

/* ---- search over a CPU-format index (levels + CSR adjacency) ------------------
 * Restates fused_tree_search_v3 (kernels/cpp/torch_ext_v3.cpp:149-244): root
 * gate over all nodes of the top level, per level expand the children of active
 * parents through offsets/children and gate them, exact-filter the leaves.
 * level 0 = keys.  centers[l]: (H, K_l, D) fp32; radii[l]: (H, K_l);
 * offsets[l]: (H, K_{l+1}+1) int64 and children[l]: (H, K_l) int64 for
 * l < n_levels-1.  out: (H_q, K_0) fp32, zero where not kept. */
int oracle_search_csr(int n_levels, const float* const* centers, const float* const* radii,
                      const int64_t* const* offsets, const int64_t* const* children, const int64_t* sizes,
                      int n_heads, int dim, const float* q, const float* tau, const float* scaling,
                      const int32_t* q2kv, int n_qheads, float* out, uint8_t* out_keep) {
    const int64_t N = sizes[0];
    const int group = q2kv ? 1 : n_qheads / n_heads;
    memset(out, 0, sizeof(float) * (size_t)n_qheads * N);
    if (out_keep) memset(out_keep, 0, (size_t)n_qheads * N);
#pragma omp parallel for schedule(dynamic, 1)
    for (int qh = 0; qh < n_qheads; ++qh) {
        const int h = q2kv ? q2kv[qh] : qh / group;
        const float* qv = q + (size_t)qh * dim;
        const float th = tau[qh], sc = scaling ? scaling[qh] : 1.0f;
        if (n_levels == 1) {
            for (int64_t i = 0; i < N; ++i) {
                const float s = oracle_dot(centers[0] + ((size_t)h * N + i) * dim, qv, dim);
                if (s >= th) { out[(size_t)qh * N + i] = s * sc; if (out_keep) out_keep[(size_t)qh * N + i] = 1; }
            }
            continue;
        }
        int64_t cap = 0;
        for (int l = 0; l < n_levels; ++l) if (sizes[l] > cap) cap = sizes[l];
        int64_t* active = (int64_t*)malloc(sizeof(int64_t) * cap);
        int64_t* next = (int64_t*)malloc(sizeof(int64_t) * cap);
        int64_t na = 0;
        const int root = n_levels - 1;
        const int64_t Kr = sizes[root];
        for (int64_t c = 0; c < Kr; ++c) {
            const float s = oracle_dot(centers[root] + ((size_t)h * Kr + c) * dim, qv, dim);
            if (s + radii[root][(size_t)h * Kr + c] >= th) active[na++] = c;
        }
        for (int l = root - 1; l >= 1 && na > 0; --l) {
            const int64_t K = sizes[l], P = sizes[l + 1];
            const int64_t* off = offsets[l] + (size_t)h * (P + 1);
            const int64_t* ch = children[l] + (size_t)h * K;
            int64_t nn = 0;
            for (int64_t a = 0; a < na; ++a) {
                for (int64_t t = off[active[a]]; t < off[active[a] + 1]; ++t) {
                    const int64_t c = ch[t];
                    const float s = oracle_dot(centers[l] + ((size_t)h * K + c) * dim, qv, dim);
                    if (s + radii[l][(size_t)h * K + c] >= th) next[nn++] = c;
                }
            }
            int64_t* tmp = active; active = next; next = tmp;
            na = nn;
        }
        if (na > 0) {
            const int64_t P0 = sizes[1];
            const int64_t* off = offsets[0] + (size_t)h * (P0 + 1);
            const int64_t* ch = children[0] + (size_t)h * N;
            for (int64_t a = 0; a < na; ++a) {
                for (int64_t t = off[active[a]]; t < off[active[a] + 1]; ++t) {
                    const int64_t i = ch[t];
                    const float s = oracle_dot(centers[0] + ((size_t)h * N + i) * dim, qv, dim);
                    if (s >= th) { out[(size_t)qh * N + i] = s * sc; if (out_keep) out_keep[(size_t)qh * N + i] = 1; }
                }
            }
        }
        free(active);
        free(next);
    }
    return 0;
}

/* ---- radii from the layout -----------------------------------------------------
 * indexer/cuda.py:114-150: r_p = max over filled children ||c - p||;
 * :152-198: r_g = max over filled parents (||p - g|| + r_p); empty -> 0.
 * Also refreshes the ||c||^2 caches (canonical). */
int oracle_recompute_radii(const hira_index_t* ix) {
    const int bf = ix->bf, dim = ix->dim;
    const size_t capC = (size_t)ix->cap_parents * bf;
    float a[256], b[256];
    for (int h = 0; h < ix->n_heads; ++h) {
        for (int p = 0; p < ix->cap_parents; ++p) {
            float r = 0.0f, sq = 0.0f;
            if (parent_valid(ix, h, p)) {
                load_row(ix->parents, ix->dtype, (size_t)h * ix->cap_parents + p, dim, a);
                sq = oracle_dot(a, a, dim);
                int cnt = ix->child_counts[(size_t)h * ix->cap_parents + p];
                if (cnt > bf) cnt = bf;
                for (int c = 0; c < cnt; ++c) {
                    load_row(ix->children, ix->dtype, (size_t)h * capC + (size_t)p * bf + c, dim, b);
                    const float d = sqrtf(dist2(a, b, dim));
                    if (d > r) r = d;
                }
            }
            ix->parent_radii[(size_t)h * ix->cap_parents + p] = r;
            if (ix->parent_sqnorm) ix->parent_sqnorm[(size_t)h * ix->cap_parents + p] = sq;
        }
        if (ix->depth != 3) continue;
        for (int g = 0; g < ix->cap_gp; ++g) {
            float r = 0.0f, sq = 0.0f;
            if (g < ix->used[h * 4 + 1]) {
                load_row(ix->grand_parents, ix->dtype, (size_t)h * ix->cap_gp + g, dim, a);
                sq = oracle_dot(a, a, dim);
                int cnt = ix->gp_counts[(size_t)h * ix->cap_gp + g];
                if (cnt > bf) cnt = bf;
                for (int c = 0; c < cnt; ++c) {
                    const size_t p = (size_t)g * bf + c;
                    load_row(ix->parents, ix->dtype, (size_t)h * ix->cap_parents + p, dim, b);
                    const float t = sqrtf(dist2(a, b, dim)) + ix->parent_radii[(size_t)h * ix->cap_parents + p];
                    if (t > r) r = t;
                }
            }
            ix->gp_radii[(size_t)h * ix->cap_gp + g] = r;
            if (ix->gp_sqnorm) ix->gp_sqnorm[(size_t)h * ix->cap_gp + g] = sq;
        }
    }
    return 0;
}

/* ---- append --------------------------------------------------------------------
 * CUDAIndexer.update for one key at a time (indexer/cuda.py:544-701):
 * nearest valid parent by ||c||^2 - 2 x.c, ties to the lowest index
 * (kernels/triton_update_kernels.py:66-82,353-364); slot claim
 * (:126-193); radius max (:238-290); grandparent radius
 * (indexer/cuda.py:1200-1231); orphan -> own parent of radius 0
 * (:730-733,818-820,877-887) under the nearest grandparent with a free slot
 * (:917-962, no validity mask :918-920) or a new grandparent (:1070-1072). */
static int nearest(const void* rows, int dtype, const float* sq, int n, const float* x, int dim,
                   const hira_index_t* ix, int h, int check_valid) {
    float best = INFINITY;
    int bi = -1;
    float row[256];
    for (int p = 0; p < n; ++p) {
        if (check_valid && !parent_valid(ix, h, p)) continue;
        load_row(rows, dtype, p, dim, row);
        const float s = sq[p] - 2.0f * oracle_dot(row, x, dim);
        if (s < best) { best = s; bi = p; }
    }
    return bi;
}

int oracle_append(const hira_index_t* ix, const void* new_k, const void* new_v, int n_new,
                  int64_t k_head_stride, int64_t v_head_stride, int token_base, int32_t* status) {
    const int bf = ix->bf, dim = ix->dim, vdim = ix->vdim;
    const size_t capP = ix->cap_parents, capC = capP * bf, capG = ix->cap_gp;
    float x[256], c[256], g[256];
    for (int h = 0; h < ix->n_heads; ++h) {
        int32_t* used = ix->used + h * 4;
        const size_t es = ix->dtype == HIRA_BF16 ? 2 : 4, vs = ix->vdtype == HIRA_BF16 ? 2 : 4;
        char* children = (char*)ix->children + (size_t)h * capC * dim * es;
        char* parents = (char*)ix->parents + (size_t)h * capP * dim * es;
        char* gps = ix->depth == 3 ? (char*)ix->grand_parents + (size_t)h * capG * dim * es : NULL;
        char* values = ix->values ? (char*)ix->values + (size_t)h * capC * vdim * vs : NULL;
        float* pr = ix->parent_radii + (size_t)h * capP;
        float* psq = ix->parent_sqnorm + (size_t)h * capP;
        int32_t* cc = ix->child_counts + (size_t)h * capP;
        float* gr = ix->depth == 3 ? ix->gp_radii + (size_t)h * capG : NULL;
        float* gsq = ix->depth == 3 ? ix->gp_sqnorm + (size_t)h * capG : NULL;
        int32_t* gc = ix->depth == 3 ? ix->gp_counts + (size_t)h * capG : NULL;
        int32_t* s2t = ix->slot2token ? ix->slot2token + (size_t)h * capC : NULL;
        for (int key = 0; key < n_new; ++key) {
            load_row((const char*)new_k + (size_t)h * k_head_stride * es, ix->dtype, key, dim, x);
            const int n_scan = ix->depth == 3 ? used[1] * bf : used[0];
            const int p = nearest(parents, ix->dtype, psq, n_scan, x, dim, ix, h, ix->depth == 3);
            const int token = token_base < 0 ? used[2] : token_base + key;
            int slot = -1;
            if (p >= 0 && cc[p] < bf) {
                slot = p * bf + cc[p];
                load_row(parents, ix->dtype, p, dim, c);
                const float d = sqrtf(dist2(x, c, dim));
                if (d > pr[p]) pr[p] = d;
                if (ix->depth == 3) {
                    const int gi = p / bf;
                    load_row(gps, ix->dtype, gi, dim, g);
                    const float t = sqrtf(dist2(c, g, dim)) + pr[p];
                    if (t > gr[gi]) gr[gi] = t;
                }
                cc[p] += 1;
            } else {
                int p_dst = -1;
                if (ix->depth == 3) {
                    const int gi = nearest(gps, ix->dtype, gsq, used[1], x, dim, ix, h, 0);
                    if (gi >= 0 && gc[gi] < bf) {
                        p_dst = gi * bf + gc[gi];
                        load_row(gps, ix->dtype, gi, dim, g);
                        const float t = sqrtf(dist2(x, g, dim));
                        if (t > gr[gi]) gr[gi] = t;
                        gc[gi] += 1;
                    } else if (used[1] < (int)capG) {
                        const int gn = used[1];
                        p_dst = gn * bf;
                        for (int d = 0; d < dim; ++d) st(gps, ix->dtype, (size_t)gn * dim + d, x[d]);
                        gr[gn] = 0.0f;
                        gsq[gn] = oracle_dot(x, x, dim);
                        gc[gn] = 1;
                        used[1] = gn + 1;
                    } else {
                        *status |= HIRA_STATUS_GP_FULL;
                    }
                } else {
                    if (used[0] < (int)capP) p_dst = used[0];
                    else *status |= HIRA_STATUS_PARENTS_FULL;
                }
                if (p_dst >= 0) {
                    slot = p_dst * bf;
                    for (int d = 0; d < dim; ++d) st(parents, ix->dtype, (size_t)p_dst * dim + d, x[d]);
                    pr[p_dst] = 0.0f;
                    psq[p_dst] = oracle_dot(x, x, dim);
                    cc[p_dst] = 1;
                    if (p_dst + 1 > used[0]) used[0] = p_dst + 1;
                }
            }
            if (slot >= 0) {
                for (int d = 0; d < dim; ++d) st(children, ix->dtype, (size_t)slot * dim + d, x[d]);
                if (values)
                    for (int d = 0; d < vdim; ++d)
                        st(values, ix->vdtype, (size_t)slot * vdim + d,
                           ld((const char*)new_v + (size_t)h * v_head_stride * vs, ix->vdtype, (size_t)key * vdim + d));
                if (s2t) s2t[slot] = token;
                used[2] += 1;
            }
        }
    }
    return 0;
}

/* ---- attention over emitted children + queued keys ------------------------------
 * No reference implementation exists (attention/hira_attention.py:1-3): a plain
 * fp64 softmax over the logits keep*score and scaling*(q.k_queued), times the
 * slot-aligned values.  out [n_qheads][vdim] fp32, out_ml [n_qheads][2]. */
int oracle_attention(const hira_index_t* ix, const float* q, const float* scaling, const int32_t* q2kv,
                     int n_qheads, const float* dense_score, const uint8_t* keep, const void* queued_k,
                     const void* queued_v, int n_queued, int64_t queued_head_stride, float* out, float* out_ml) {
    const int dim = ix->dim, vdim = ix->vdim;
    const size_t capC = (size_t)ix->cap_parents * ix->bf;
    const int group = q2kv ? 1 : n_qheads / ix->n_heads;
    const size_t es = ix->dtype == HIRA_BF16 ? 2 : 4, vs = ix->vdtype == HIRA_BF16 ? 2 : 4;
#pragma omp parallel for schedule(dynamic, 1)
    for (int qh = 0; qh < n_qheads; ++qh) {
        const int h = q2kv ? q2kv[qh] : qh / group;
        const float sc = scaling ? scaling[qh] : 1.0f;
        double* ql = (double*)malloc(sizeof(double) * (n_queued > 0 ? n_queued : 1));
        double m = -INFINITY;
        float row[256];
        for (size_t s = 0; s < capC; ++s)
            if (keep[(size_t)qh * capC + s] && dense_score[(size_t)qh * capC + s] > m) m = dense_score[(size_t)qh * capC + s];
        for (int j = 0; j < n_queued; ++j) {
            load_row((const char*)queued_k + (size_t)h * queued_head_stride * es, ix->dtype, j, dim, row);
            ql[j] = (double)(oracle_dot(row, q + (size_t)qh * dim, dim) * sc);
            if (ql[j] > m) m = ql[j];
        }
        double l = 0.0;
        double acc[256];
        for (int d = 0; d < vdim; ++d) acc[d] = 0.0;
        for (size_t s = 0; s < capC; ++s) {
            if (!keep[(size_t)qh * capC + s]) continue;
            const double p = exp((double)dense_score[(size_t)qh * capC + s] - m);
            l += p;
            for (int d = 0; d < vdim; ++d) acc[d] += p * (double)ld(ix->values, ix->vdtype, ((size_t)h * capC + s) * vdim + d);
        }
        for (int j = 0; j < n_queued; ++j) {
            const double p = exp(ql[j] - m);
            l += p;
            for (int d = 0; d < vdim; ++d)
                acc[d] += p * (double)ld((const char*)queued_v + (size_t)h * queued_head_stride * vs, ix->vdtype, (size_t)j * vdim + d);
        }
        for (int d = 0; d < vdim; ++d) out[(size_t)qh * vdim + d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
        if (out_ml) { out_ml[2 * qh] = (float)m; out_ml[2 * qh + 1] = (float)l; }
        free(ql);
    }
    return 0;
}

/* ---- thresholds -------------------------------------------------------------------
 * sample_max / sample_mean_topk as their names state (cache/threshold_finder.py:1-14,
 * unimplemented in the reference), plus the k-th largest sample score. */
static int cmp_desc(const void* a, const void* b) {
    const float x = *(const float*)a, y = *(const float*)b;
    return (x < y) - (x > y);
}
int oracle_threshold(const void* samples, int dtype, int n_heads, int n_samples, int dim, int64_t head_stride,
                     const float* q, const int32_t* q2kv, int n_qheads, int method, int k, float* tau_out) {
    const int group = q2kv ? 1 : n_qheads / n_heads;
    const size_t es = dtype == HIRA_BF16 ? 2 : 4;
    float* s = (float*)malloc(sizeof(float) * n_samples);
    float row[256];
    for (int qh = 0; qh < n_qheads; ++qh) {
        const int h = q2kv ? q2kv[qh] : qh / group;
        for (int i = 0; i < n_samples; ++i) {
            load_row((const char*)samples + (size_t)h * head_stride * es, dtype, i, dim, row);
            s[i] = oracle_dot(row, q + (size_t)qh * dim, dim);
        }
        qsort(s, n_samples, sizeof(float), cmp_desc);
        if (method == HIRA_TAU_SAMPLE_MAX) tau_out[qh] = s[0];
        else if (method == HIRA_TAU_SAMPLE_KTH) tau_out[qh] = s[k - 1];
        else {
            float sum = 0.0f;
            for (int i = 0; i < k; ++i) sum = sum + s[i];
            tau_out[qh] = sum / (float)k;
        }
    }
    free(s);
    return 0;
}

/* ---- assignment (the build's contraction) ------------------------------------------
 * torch.cdist + argmin (indexer/cuda.py:244-245) restated as arg-min of
 * ||c||^2 - 2 x.c with sequential-chain dots, ties to the lowest index;
 * out_d2 = max(||x||^2 + min, 0). */
int oracle_assign(const void* points, int64_t p_head_stride, const void* cents, int dtype, int n_heads, int n,
                  int k, int dim, int32_t* out_idx, float* out_d2) {
    const size_t es = dtype == HIRA_BF16 ? 2 : 4;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; ++h) {
        float* C = (float*)malloc(sizeof(float) * (size_t)k * dim);
        float* csq = (float*)malloc(sizeof(float) * k);
        float x[256];
        for (int c = 0; c < k; ++c) {
            load_row(cents, dtype, (size_t)h * k + c, dim, C + (size_t)c * dim);
            csq[c] = dot_seq(C + (size_t)c * dim, C + (size_t)c * dim, dim);
        }
        for (int i = 0; i < n; ++i) {
            load_row((const char*)points + (size_t)h * p_head_stride * es, dtype, i, dim, x);
            float best = INFINITY;
            int bi = 0x7fffffff;
            for (int c = 0; c < k; ++c) {
                const float s = csq[c] - 2.0f * dot_seq(x, C + (size_t)c * dim, dim);
                if (s < best) { best = s; bi = c; }
            }
            const float d2 = dot_seq(x, x, dim) + best;
            out_idx[(size_t)h * n + i] = bi;
            out_d2[(size_t)h * n + i] = d2 > 0.0f ? d2 : 0.0f;
        }
        free(C);
        free(csq);
    }
    return 0;
}

/* ---- build ---------------------------------------------------------------------------
 * One level (indexer/cuda.py:200-336): centres = chosen points, assignment,
 * each centre keeps its bf closest (ties by point id), overflow goes to free
 * slots -- here deterministically: overflow in (centre, distance, id) order
 * fills free slots in ascending slot order (the reference draws a randperm,
 * :327-329).  n_iters > 1 inserts Lloyd mean updates (members summed in
 * (distance, id) order, fp32) before the final assignment. */
typedef struct { uint64_t key; uint32_t id; } sort_item;
static int cmp_item(const void* a, const void* b) {
    const sort_item* x = (const sort_item*)a; const sort_item* y = (const sort_item*)b;
    if (x->key != y->key) return x->key < y->key ? -1 : 1;
    return (x->id > y->id) - (x->id < y->id);
}
/* arg-min over the centres that still have room (balanced rounds), same arithmetic as oracle_assign */
static void assign_masked_head(const void* points, int64_t p_head_stride, const void* cents, int dtype, int h, int n,
                               int k, int dim, int bf, const int32_t* filled, const int32_t* slot, int32_t* out_idx,
                               float* out_d2) {
    const size_t es = dtype == HIRA_BF16 ? 2 : 4;
    float* C = (float*)malloc(sizeof(float) * (size_t)k * dim);
    float* csq = (float*)malloc(sizeof(float) * k);
    for (int c = 0; c < k; ++c) {
        load_row(cents, dtype, (size_t)h * k + c, dim, C + (size_t)c * dim);
        csq[c] = dot_seq(C + (size_t)c * dim, C + (size_t)c * dim, dim);
    }
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n; ++i) {
        if (slot[i] >= 0) continue;
        float x[256];
        load_row((const char*)points + (size_t)h * p_head_stride * es, dtype, i, dim, x);
        float best = INFINITY;
        int bi = 0x7fffffff;
        for (int c = 0; c < k; ++c) {
            if (filled[c] >= bf) continue;
            const float s = csq[c] - 2.0f * dot_seq(x, C + (size_t)c * dim, dim);
            if (s < best) { best = s; bi = c; }
        }
        const float d2 = dot_seq(x, x, dim) + best;
        out_idx[i] = bi;
        out_d2[i] = d2 > 0.0f ? d2 : 0.0f;
    }
    free(C);
    free(csq);
}

static void build_level(const void* points, int64_t p_head_stride, int dtype, int n_heads, int n, int k, int bf,
                        int dim, const int32_t* cent_idx, int n_iters, int balance_rounds,
                        void* cents /* [H][k][dim] dtype */, int32_t* slot /* [H][n] */, int32_t* fill /* [H][k] */) {
    const size_t es = dtype == HIRA_BF16 ? 2 : 4;
    int32_t* a_idx = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_heads * n);
    float* a_d2 = (float*)malloc(sizeof(float) * (size_t)n_heads * n);
    for (int h = 0; h < n_heads; ++h)
        for (int c = 0; c < k; ++c) {
            int src = cent_idx ? cent_idx[(size_t)h * k + c] : (int)(((int64_t)c * n) / k);
            if (src < 0) src = 0;
            if (src >= n) src = n - 1;
            memcpy((char*)cents + ((size_t)h * k + c) * dim * es,
                   (const char*)points + ((size_t)h * p_head_stride + (size_t)src * dim) * es, dim * es);
        }
    const int iters = n_iters < 1 ? 1 : n_iters;
    sort_item* items = (sort_item*)malloc(sizeof(sort_item) * n);
    int32_t* start = (int32_t*)malloc(sizeof(int32_t) * (k + 1));
    int32_t* filled = (int32_t*)malloc(sizeof(int32_t) * k);
    for (int it = 0; it < iters; ++it) {
        oracle_assign(points, p_head_stride, cents, dtype, n_heads, n, k, dim, a_idx, a_d2);
        for (int h = 0; h < n_heads; ++h) {
            int32_t* hslot = slot + (size_t)h * n;
            int32_t* hidx = a_idx + (size_t)h * n;
            float* hd2 = a_d2 + (size_t)h * n;
            int n_items = 0;
            for (int i = 0; i < n; ++i) {
                uint32_t bits;
                memcpy(&bits, &hd2[i], 4);
                items[i].key = ((uint64_t)(uint32_t)hidx[i] << 32) | bits;
                items[i].id = (uint32_t)i;
            }
            n_items = n;
            qsort(items, n_items, sizeof(sort_item), cmp_item);
            int pos = 0;
            for (int c = 0; c <= k; ++c) {
                while (pos < n_items && (int)(items[pos].key >> 32) < c) ++pos;
                start[c] = pos;
            }
            if (it + 1 < iters) {
                float sum[256], row[256];
                for (int c = 0; c < k; ++c) {
                    if (start[c + 1] <= start[c]) continue;
                    for (int d = 0; d < dim; ++d) sum[d] = 0.0f;
                    for (int m = start[c]; m < start[c + 1]; ++m) {
                        load_row((const char*)points + (size_t)h * p_head_stride * es, dtype, items[m].id, dim, row);
                        for (int d = 0; d < dim; ++d) sum[d] = sum[d] + row[d];
                    }
                    const float cnt = (float)(start[c + 1] - start[c]);
                    for (int d = 0; d < dim; ++d) st(cents, dtype, ((size_t)h * k + c) * dim + d, sum[d] / cnt);
                }
                continue;
            }
            /* capacity-aware rounds: every centre accepts, closest first, what it has room for; points
             * left over choose again among the centres with room (balance_rounds times) */
            for (int c = 0; c < k; ++c) filled[c] = 0;
            if (balance_rounds > 0)
                for (int i = 0; i < n; ++i) hslot[i] = -1;
            for (int r = 0; r < balance_rounds; ++r) {
                for (int c = 0; c < k; ++c) {
                    const int room = bf - filled[c];
                    int acc = 0;
                    for (int m = start[c]; m < start[c + 1] && acc < room; ++m, ++acc)
                        hslot[items[m].id] = c * bf + filled[c] + acc;
                    filled[c] += acc;
                }
                assign_masked_head(points, p_head_stride, cents, dtype, h, n, k, dim, bf, filled, hslot, hidx, hd2);
                n_items = 0;
                for (int i = 0; i < n; ++i) {
                    if (hslot[i] >= 0) continue;
                    uint32_t bits;
                    memcpy(&bits, &hd2[i], 4);
                    items[n_items].key = ((uint64_t)(uint32_t)hidx[i] << 32) | bits;
                    items[n_items].id = (uint32_t)i;
                    ++n_items;
                }
                qsort(items, n_items, sizeof(sort_item), cmp_item);
                pos = 0;
                for (int c = 0; c <= k; ++c) {
                    while (pos < n_items && (int)(items[pos].key >> 32) < c) ++pos;
                    start[c] = pos;
                }
            }
            /* final pass: placement of what the last sort holds */
            int* fbase = (int*)malloc(sizeof(int) * (k + 1));
            int f = 0;
            for (int c = 0; c < k; ++c) {
                const int cnt = start[c + 1] - start[c], room = bf - filled[c];
                fbase[c] = f;
                f += room - cnt > 0 ? room - cnt : 0;
                fill[(size_t)h * k + c] = filled[c] + (cnt < room ? cnt : room);
            }
            fbase[k] = f;
            int L = 0, c2 = 0;
            for (int c = 0; c < k; ++c) {
                const int room = bf - filled[c];
                for (int m = start[c]; m < start[c + 1]; ++m) {
                    const int rank = m - start[c];
                    if (rank < room) { hslot[items[m].id] = c * bf + filled[c] + rank; continue; }
                    while (fbase[c2 + 1] <= L) ++c2;
                    const int cnt2 = start[c2 + 1] - start[c2], room2 = bf - filled[c2];
                    hslot[items[m].id] = c2 * bf + filled[c2] + (cnt2 < room2 ? cnt2 : room2) + (L - fbase[c2]);
                    fill[(size_t)h * k + c2] += 1;
                    ++L;
                }
            }
            free(fbase);
        }
    }
    free(items); free(start); free(filled); free(a_idx); free(a_d2);
}

int oracle_build(const hira_index_t* ix, const void* keys, const void* values, int n_keys, int64_t k_head_stride,
                 int64_t v_head_stride, int token_base, const int32_t* cent_idx1, const int32_t* cent_idx2,
                 int n_iters, int balance_rounds) {
    const int H = ix->n_heads, bf = ix->bf, dim = ix->dim, vdim = ix->vdim;
    const size_t es = ix->dtype == HIRA_BF16 ? 2 : 4, vs = ix->vdtype == HIRA_BF16 ? 2 : 4;
    const size_t capP = ix->cap_parents, capC = capP * bf, capG = ix->cap_gp;
    const int k1 = (n_keys + bf - 1) / bf, k2 = (k1 + bf - 1) / bf;
    memset(ix->children, 0, (size_t)H * capC * dim * es);
    if (ix->values) memset(ix->values, 0, (size_t)H * capC * vdim * vs);
    if (ix->slot2token) memset(ix->slot2token, 0xff, (size_t)H * capC * 4);
    memset(ix->parents, 0, (size_t)H * capP * dim * es);
    memset(ix->parent_radii, 0, (size_t)H * capP * 4);
    if (ix->parent_sqnorm) memset(ix->parent_sqnorm, 0, (size_t)H * capP * 4);
    memset(ix->child_counts, 0, (size_t)H * capP * 4);
    if (ix->depth == 3) {
        memset(ix->grand_parents, 0, (size_t)H * capG * dim * es);
        memset(ix->gp_radii, 0, (size_t)H * capG * 4);
        if (ix->gp_sqnorm) memset(ix->gp_sqnorm, 0, (size_t)H * capG * 4);
        memset(ix->gp_counts, 0, (size_t)H * capG * 4);
    }
    for (int h = 0; h < H; ++h) { ix->used[h * 4] = 0; ix->used[h * 4 + 1] = 0; ix->used[h * 4 + 2] = 0; ix->used[h * 4 + 3] = 0; }
    if (n_keys == 0) return 0;
    void* cents1 = malloc((size_t)H * k1 * dim * es);
    void* cents2 = malloc((size_t)H * k2 * dim * es);
    int32_t* slot1 = (int32_t*)malloc(sizeof(int32_t) * (size_t)H * n_keys);
    int32_t* slot2 = (int32_t*)malloc(sizeof(int32_t) * (size_t)H * k1);
    int32_t* fill1 = (int32_t*)malloc(sizeof(int32_t) * (size_t)H * k1);
    int32_t* fill2 = (int32_t*)malloc(sizeof(int32_t) * (size_t)H * k2);
    build_level(keys, k_head_stride, ix->dtype, H, n_keys, k1, bf, dim, cent_idx1, n_iters, balance_rounds, cents1, slot1, fill1);
    if (ix->depth == 3)
        build_level(cents1, (int64_t)k1 * dim, ix->dtype, H, k1, k2, bf, dim, cent_idx2, n_iters, balance_rounds, cents2, slot2, fill2);
    for (int h = 0; h < H; ++h) {
        for (int c = 0; c < k1; ++c) {
            const int s = ix->depth == 3 ? slot2[(size_t)h * k1 + c] : c;
            memcpy((char*)ix->parents + ((size_t)h * capP + s) * dim * es, (char*)cents1 + ((size_t)h * k1 + c) * dim * es, dim * es);
            ix->child_counts[(size_t)h * capP + s] = fill1[(size_t)h * k1 + c];
        }
        if (ix->depth == 3)
            for (int g = 0; g < k2; ++g) {
                memcpy((char*)ix->grand_parents + ((size_t)h * capG + g) * dim * es, (char*)cents2 + ((size_t)h * k2 + g) * dim * es, dim * es);
                ix->gp_counts[(size_t)h * capG + g] = fill2[(size_t)h * k2 + g];
            }
        for (int i = 0; i < n_keys; ++i) {
            int s = slot1[(size_t)h * n_keys + i];
            if (ix->depth == 3) { const int c = s / bf, r = s - c * bf; s = slot2[(size_t)h * k1 + c] * bf + r; }
            memcpy((char*)ix->children + ((size_t)h * capC + s) * dim * es,
                   (const char*)keys + ((size_t)h * k_head_stride + (size_t)i * dim) * es, dim * es);
            if (ix->values)
                memcpy((char*)ix->values + ((size_t)h * capC + s) * vdim * vs,
                       (const char*)values + ((size_t)h * v_head_stride + (size_t)i * vdim) * vs, vdim * vs);
            if (ix->slot2token) ix->slot2token[(size_t)h * capC + s] = token_base + i;
        }
        ix->used[h * 4 + 0] = ix->depth == 3 ? k2 * bf : k1;
        ix->used[h * 4 + 1] = ix->depth == 3 ? k2 : 0;
        ix->used[h * 4 + 2] = n_keys;
    }
    free(cents1); free(cents2); free(slot1); free(slot2); free(fill1); free(fill2);
    return oracle_recompute_radii(ix);
}

/* ---- merge of partial softmax results ------------------------------------------------ */
int oracle_merge_partials(const float* part_o, const float* part_ml, int n_parts, int n_qheads, int vdim,
                          float* out, float* out_ml) {
    for (int qh = 0; qh < n_qheads; ++qh) {
        double M = -INFINITY, L = 0.0;
        for (int s = 0; s < n_parts; ++s) {
            const double m = part_ml[((size_t)s * n_qheads + qh) * 2];
            if (m > M) M = m;
        }
        for (int s = 0; s < n_parts; ++s) {
            const double m = part_ml[((size_t)s * n_qheads + qh) * 2], l = part_ml[((size_t)s * n_qheads + qh) * 2 + 1];
            if (m > -INFINITY) L += l * exp(m - M);
        }
        for (int d = 0; d < vdim; ++d) {
            double o = 0.0;
            for (int s = 0; s < n_parts; ++s) {
                const double m = part_ml[((size_t)s * n_qheads + qh) * 2], l = part_ml[((size_t)s * n_qheads + qh) * 2 + 1];
                if (m > -INFINITY) o += l * exp(m - M) * part_o[((size_t)s * n_qheads + qh) * vdim + d];
            }
            out[(size_t)qh * vdim + d] = L > 0.0 ? (float)(o / L) : 0.0f;
        }
        if (out_ml) { out_ml[2 * qh] = (float)M; out_ml[2 * qh + 1] = (float)L; }
    }
    return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
