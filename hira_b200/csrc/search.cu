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
// The kernel is a streaming read: 8-lane groups each read one row with 128-bit
// asynchronous copies, several rows in flight per thread; it is HBM-bound.
#include "common.cuh"
#include "search_common.cuh"
#include <math_constants.h>

namespace hira {

template <typename T, int GT, int NCH, int STAGES, int MINB, bool FULLD, int TH, int RPI, bool SCAN>
__global__ void __launch_bounds__(TH, MINB)
search_kernel(const SearchParams P) {
    constexpr int SEARCH_THREADS = TH;
    constexpr int SEARCH_GROUPS = TH / GROUP;  // 8-lane groups per CTA
    constexpr int PRE = 2;                      // parent-gate iterations whose loads are issued up front
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int TP = P.tile_parents;
    const int bf = P.bf;
    const int tile_rows = TP * bf;
    float* s_score = reinterpret_cast<float*>(smem_raw);                         // [tile_rows][GT]
    int* s_pcount = reinterpret_cast<int*>(s_score + (size_t)tile_rows * GT);    // [TP]
    unsigned short* s_plist = reinterpret_cast<unsigned short*>(s_pcount + TP);  // [TP]
    unsigned char* s_pmask = reinterpret_cast<unsigned char*>(s_plist + TP);     // [TP]
    unsigned char* s_gpmask = s_pmask + TP;                                      // [TP]

    __shared__ int s_qh[GT];
    __shared__ float s_scale[GT];
    __shared__ int s_nq, s_npass, s_dense;
    __shared__ uint32_t s_stat[GT][8];
    __shared__ unsigned long long s_scan[TH / GROUP];
    __shared__ __align__(16) float s_xkey[SCAN ? GROUP * NCH * 8 : 4];  // the scanned key: [lane][chunk][8]

    const int tid = threadIdx.x;
    const int lane = tid & (GROUP - 1);  // lane inside the 8-lane group
    const int grp = tid / GROUP;         // group id: one row per group per step
    const int warp = tid >> 5;
    const int wl = tid & 31;
    // chunks of one tile are neighbours in the grid: they run at the same time and the later
    // ones find the tile's rows in L2
    const int chunk = blockIdx.x;
    const int tile = blockIdx.y;
    const int h = blockIdx.z;
    const bool ge = P.flags & HIRA_GATE_GE;
    const int leaf_mode = P.flags & (HIRA_LEAF_GE | HIRA_LEAF_GT);
    const bool has_qn = P.qnorm != nullptr;
    const size_t cap_children = (size_t)P.cap_parents * bf;
    const T* children = reinterpret_cast<const T*>(P.children) + (size_t)h * cap_children * P.dim;
    const T* parents = reinterpret_cast<const T*>(P.parents) + (size_t)h * P.cap_parents * P.dim;

    // ---- 1. query heads of this kv head handled by this CTA ------------------
    if (tid < GT * 8) (&s_stat[0][0])[tid] = 0;
    int nq;
    int qh_of[GT];
    if (P.q2kv == nullptr) {
        nq = P.group - chunk * GT;
        nq = nq < 0 ? 0 : (nq > GT ? GT : nq);
#pragma unroll
        for (int j = 0; j < GT; ++j) qh_of[j] = h * P.group + chunk * GT + (j < nq ? j : 0);
        if (tid < nq) s_qh[tid] = h * P.group + chunk * GT + tid;
    } else {
        if (warp == 0) {
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
        nq = s_nq;
#pragma unroll
        for (int j = 0; j < GT; ++j) qh_of[j] = s_qh[j < nq ? j : 0];
    }
    if (nq == 0) return;  // nothing mapped to this (kv head, chunk): no outputs owned (uniform over the CTA)
    const int tile_p0 = tile * TP;
    const size_t tile_c0 = (size_t)tile_p0 * bf;
    const int my_head = HeadReduce<GT>::head_of_lane(lane);
    const bool head_on = my_head < nq;

    // ---- 2. every load the gates need, issued together (one memory latency, not five) ----
    const int used_parents = P.used[h * 4 + 0];
    const int used_gp = P.used[h * 4 + 1];
    // tiles align with grandparent blocks (TP % bf == 0 or bf % TP == 0): the tile's first
    // grandparent and the number it touches come from the host, divisions by bf use its magic
    const int g0 = P.tile_gp_shift >= 0 ? (tile >> P.tile_gp_shift)
                                        : (P.tile_gp_shift == -1 ? tile * P.ng : div_bf(tile * TP, bf, P.bf_magic));
    const int ng = P.ng;
    int my_qh = qh_of[0];
#pragma unroll
    for (int j = 1; j < GT; ++j)
        if (my_head == j) my_qh = qh_of[j];
    const float my_tau = head_on ? P.tau[my_qh] : 0.f;
    const float my_qn = (head_on && has_qn) ? P.qnorm[my_qh] : 1.f;
    if (tid < nq) s_scale[tid] = P.scaling ? P.scaling[s_qh[tid]] : 1.0f;  // s_qh[tid] was written by this thread or before the barrier above
    float qreg[GT][NCH][8];
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        if (j < nq) {
            load_vec_f32<NCH>(P.q + (size_t)qh_of[j] * P.dim, qreg[j], lane, P.dim);
        } else {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) qreg[j][i][e] = 0.f;
        }
    }
    // grandparent row of this group (first pass of the loop below) and its radius
    RawChunk<T> graw[NCH];
    float grad = 0.f;
    const bool gp_mine = P.depth == 3 && grp < ng && (g0 + grp) < P.cap_gp;
    {
        const T* gps = reinterpret_cast<const T*>(P.gps) + (size_t)h * P.cap_gp * P.dim;
        load_row_raw<T, NCH>(graw, gps + (size_t)(g0 + grp) * P.dim, lane, P.dim, gp_mine);
        if (gp_mine) grad = P.gp_radii[(size_t)h * P.cap_gp + g0 + grp];
    }
    // parent rows of this group for the first PRE passes, with radius, child count and slot validity
    RawChunk<T> praw[PRE][NCH];
    float prad[PRE];
    int pcnt[PRE], pgc[PRE];
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
        const int i = u * SEARCH_GROUPS + grp;
        const int p = tile_p0 + i;
        const bool in = (i < TP) && (p < P.cap_parents);
        load_row_raw<T, NCH>(praw[u], parents + (size_t)p * P.dim, lane, P.dim, in);
        prad[u] = in ? P.parent_radii[(size_t)h * P.cap_parents + p] : 0.f;
        pcnt[u] = in ? P.child_counts[(size_t)h * P.cap_parents + p] : 0;
        pgc[u] = (in && P.depth == 3) ? P.gp_counts[(size_t)h * P.cap_gp + g0 + div_bf(p - g0 * bf, bf, P.bf_magic)] : 0;
    }
    // the new key of this head and the cached squared norms of the same parents, for the scan
    const bool do_scan = SCAN && chunk == 0;  // SCAN: the launch was given a scan_out
    float psq[PRE];
    if (do_scan) {
        if constexpr (SCAN) {
            if (tid < GROUP) {  // kept in shared memory: the gates have no registers to spare
                float xk[NCH][8];
                load_vec<T, NCH>(reinterpret_cast<const T*>(P.scan_key) + (size_t)h * P.scan_key_stride, xk, lane, P.dim);
#pragma unroll
                for (int ci = 0; ci < NCH; ++ci)
#pragma unroll
                    for (int e = 0; e < 8; ++e) s_xkey[(lane * NCH + ci) * 8 + e] = xk[ci][e];
            }
        }
#pragma unroll
        for (int u = 0; u < PRE; ++u) {
            const int p = tile_p0 + u * SEARCH_GROUPS + grp;
            psq[u] = (u * SEARCH_GROUPS + grp < TP && p < P.cap_parents) ? P.parent_sqnorm[(size_t)h * P.cap_parents + p] : 0.f;
        }
    }
    unsigned long long scan_best = ~0ull;  // the same in the 8 lanes of a group
    // score buffer starts as "nothing emitted"
    {
        uint4* sc4 = reinterpret_cast<uint4*>(s_score);
        const int n4 = tile_rows * GT / 4;
        for (int i = tid; i < n4; i += SEARCH_THREADS) sc4[i] = make_uint4(NOT_EMITTED, NOT_EMITTED, NOT_EMITTED, NOT_EMITTED);
        for (int i = n4 * 4 + tid; i < tile_rows * GT; i += SEARCH_THREADS)
            reinterpret_cast<uint32_t*>(s_score)[i] = NOT_EMITTED;
    }

    // tile beyond the slots in use: emit nothing
    bool tile_empty;
    if (P.depth == 3) tile_empty = g0 >= used_gp;
    else tile_empty = tile_p0 >= used_parents;

    if (!tile_empty) {
        // ---- 3a. grandparent gate --------------------------------------------
        const uint32_t allmask = (1u << nq) - 1u;
        if (P.depth == 3) {
            const T* gps = reinterpret_cast<const T*>(P.gps) + (size_t)h * P.cap_gp * P.dim;
            for (int i0 = 0; i0 < ng; i0 += SEARCH_GROUPS) {  // trip count uniform over the CTA: ballot inside
                const int i = i0 + grp;
                const int g = g0 + i;
                const bool valid = (i < ng) && (g < used_gp);  // uniform inside the group
                float d, r;
                if (i0 == 0) {
                    d = gate_dot_raw<T, GT, NCH>(graw, qreg, lane);
                    r = grad;
                } else {
                    d = gate_dot<T, GT, NCH>(gps + (size_t)g * P.dim, qreg, lane, P.dim, valid);
                    r = valid ? P.gp_radii[(size_t)h * P.cap_gp + g] : 0.f;
                }
                const bool keep = valid && head_on && gate_keep(d, r, my_qn, has_qn, my_tau, ge);
                const uint32_t b = __ballot_sync(0xffffffffu, keep);
                const uint32_t m = head_mask_from_ballot<GT>(b, tid);
                if (lane == 0 && i < ng) {
                    s_gpmask[i] = (unsigned char)m;
                    // a grandparent whose parents span several tiles is gated by each of
                    // them; only the tile holding its first parent books the visit
                    if (valid && P.stats && tile_p0 == g0 * bf) {
                        for (int jj = 0; jj < nq; ++jj) {
                            atomicAdd(&s_stat[jj][0], 1u);
                            if ((m >> jj) & 1u) atomicAdd(&s_stat[jj][1], 1u);
                        }
                    }
                }
            }
        }
        __syncthreads();  // s_gpmask, s_stat zeroing, score sentinel

        // ---- 3b. parent gate --------------------------------------------------
        auto gate_parent = [&](int i0, float d, float r, int cnt, int gc, float scan_s) {
            const int i = i0 + grp;
            const int p = tile_p0 + i;
            const bool in = (i < TP) && (p < P.cap_parents);
            bool valid = in;
            uint32_t gm = allmask;
            if (in) {
                if (P.depth == 3) {
                    const int g = g0 + div_bf(p - g0 * bf, bf, P.bf_magic);
                    valid = (g < used_gp) && ((p - g * bf) < gc);
                    gm = s_gpmask[g - g0];
                } else {
                    valid = p < used_parents;
                }
            }
            if (do_scan && valid) {  // every valid parent is a candidate, whatever the gates say
                const unsigned long long key = ((unsigned long long)order_key(scan_s) << 32) | (uint32_t)p;
                if (key < scan_best) scan_best = key;
            }
            const bool work = valid && gm != 0;
            const bool keep = work && head_on && ((gm >> my_head) & 1u) && gate_keep(d, r, my_qn, has_qn, my_tau, ge);
            const uint32_t b = __ballot_sync(0xffffffffu, keep);
            const uint32_t m = head_mask_from_ballot<GT>(b, tid);
            if (lane == 0 && i < TP) {
                cnt = valid ? (cnt > bf ? bf : cnt) : 0;
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
        };
        // sq - 2 x.c of a parent row against the new key: the score the append's nearest-parent
        // search minimises, in the same arithmetic (chunk order, 8-lane tree)
        auto scan_score = [&](const RawChunk<T> (&raw)[NCH], float sq) -> float {
            if constexpr (SCAN) {
                Acc2 acc{0.f, 0.f};
#pragma unroll
                for (int ci = 0; ci < NCH; ++ci) {
                    float a[8], xk[8];
                    to_float(raw[ci], a);
                    const float4 x0 = *reinterpret_cast<const float4*>(&s_xkey[(lane * NCH + ci) * 8]);
                    const float4 x1 = *reinterpret_cast<const float4*>(&s_xkey[(lane * NCH + ci) * 8 + 4]);
                    xk[0] = x0.x; xk[1] = x0.y; xk[2] = x0.z; xk[3] = x0.w;
                    xk[4] = x1.x; xk[5] = x1.y; xk[6] = x1.z; xk[7] = x1.w;
                    chunk_fma(acc, a, xk);
                }
                const float d = group_sum(__fadd_rn(acc.e, acc.o));
                return __fsub_rn(sq, __fmul_rn(2.0f, d));
            } else {
                return 0.f;
            }
        };
#pragma unroll
        for (int u = 0; u < PRE; ++u) {  // rows loaded in step 2; the trip test is uniform over the CTA
            if (u * SEARCH_GROUPS < TP) {
                float ss = 0.f;
                if (do_scan) ss = scan_score(praw[u], psq[u]);  // uniform over the CTA
                gate_parent(u * SEARCH_GROUPS, gate_dot_raw<T, GT, NCH>(praw[u], qreg, lane), prad[u], pcnt[u], pgc[u], ss);
            }
        }
        for (int i0 = PRE * SEARCH_GROUPS; i0 < TP; i0 += SEARCH_GROUPS) {  // uniform trip count
            const int p = tile_p0 + i0 + grp;
            const bool in = (i0 + grp < TP) && (p < P.cap_parents);
            const float d = gate_dot<T, GT, NCH>(parents + (size_t)p * P.dim, qreg, lane, P.dim, in);
            const float r = in ? P.parent_radii[(size_t)h * P.cap_parents + p] : 0.f;
            const int cnt = in ? P.child_counts[(size_t)h * P.cap_parents + p] : 0;
            const int gc = (in && P.depth == 3) ? P.gp_counts[(size_t)h * P.cap_gp + g0 + div_bf(p - g0 * bf, bf, P.bf_magic)] : 0;
            float ss = 0.f;
            if (do_scan) {  // uniform over the CTA
                RawChunk<T> raw[NCH];
                load_row_raw<T, NCH>(raw, parents + (size_t)p * P.dim, lane, P.dim, in);
                ss = scan_score(raw, in ? P.parent_sqnorm[(size_t)h * P.cap_parents + p] : 0.f);
            }
            gate_parent(i0, d, r, cnt, gc, ss);
        }
        if (do_scan && lane == 0) s_scan[grp] = scan_best;
        __syncthreads();

        // ---- 4. ordered list of parents kept for at least one head ------------
        // one packed word per kept parent: local parent id << 19 | head mask << 11 | child count
        uint32_t* s_pl = reinterpret_cast<uint32_t*>(s_pcount);  // reuses s_pcount after the pass below
        if (warp == 0) {
            int n = 0;
            bool dense = true;  // every parent slot of the tile is full and kept for every head
            for (int base = 0; base < TP; base += 32) {
                const int i = base + wl;
                uint32_t word = 0;
                bool m = false;
                if (i < TP) {
                    const uint32_t cnt = (uint32_t)s_pcount[i], msk = s_pmask[i];
                    m = msk != 0 && cnt > 0;
                    word = ((uint32_t)i << 19) | (msk << 11) | cnt;
                    dense = dense && msk == allmask && cnt == (uint32_t)bf;
                }
                const uint32_t b = __ballot_sync(0xffffffffu, m);
                __syncwarp();  // every lane has read s_pcount[base..base+31] before slots <= base+31 are overwritten
                if (m) s_pl[n + __popc(b & ((1u << wl) - 1u))] = word;
                n += __popc(b);
            }
            dense = __all_sync(0xffffffffu, dense);
            if (wl == 0) {
                s_npass = n;
                s_dense = dense;
            }
        } else if (warp == 1 && do_scan) {  // meanwhile: nearest parent of the tile -> nearest of the head
            unsigned long long best = wl < SEARCH_GROUPS ? s_scan[wl] : ~0ull;
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) {
                const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, sft);
                best = o < best ? o : best;
            }
            if (wl == 0 && best != ~0ull) atomicMin(P.scan_out + h, best);
        }
        __syncthreads();
        const int npass = s_npass;

        // ---- 5. stream the children rows of kept parents ----------------------
        // The kept parents form a flat list of npass*bf rows; 8-lane group g walks the R
        // consecutive rows [g*R, (g+1)*R) of it, so its row pointer and score index just
        // step forward and the parent word is reloaded once per bf rows.  Each thread owns
        // a private ring of STAGES slots in shared memory and keeps STAGES-1 steps (of RPI
        // rows) of asynchronous 16-byte copies (cp.async, L2 only) in flight ahead of the
        // rows it is working on; only the issuing thread reads a slot, so no barrier is
        // needed and the depth of the prefetch costs no registers.
        constexpr int TPP = (int)(sizeof(T) / 2);   // 16-byte pieces per chunk
        constexpr int PIECES = NCH * TPP;           // 16-byte pieces per thread per row
        constexpr int PIECE_STRIDE = SEARCH_THREADS * 16;
        constexpr int STAGE_STRIDE = RPI * PIECES * PIECE_STRIDE;
        const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(smem_raw + P.ring_offset) + tid * 16;
        const unsigned char* ring_g = smem_raw + P.ring_offset + tid * 16;
        const int row_bytes = P.dim * (int)sizeof(T);
        const char* gbase = reinterpret_cast<const char*>(children) + tile_c0 * (size_t)row_bytes + lane * 8 * sizeof(T);
        const bool writer = HeadReduce<GT>::is_writer(lane);
        const bool emit_all = leaf_mode == HIRA_LEAF_CANDIDATES;
        // d > tau  <=>  d >= nextafter(tau): one comparison serves both leaf rules
        const float leaf_thr = (leaf_mode == HIRA_LEAF_GT) ? nextafterf(my_tau, CUDART_INF_F) : my_tau;
        // dot products of the row in ring slot (cons_off, u) with the CTA's heads; the lane
        // returns the one of its own head
        auto row_score = [&](uint32_t cons_off, int u) -> float {
            Acc2 acc[GT];
#pragma unroll
            for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
            for (int ci = 0; ci < NCH; ++ci) {
                // a slot that was not filled this step holds stale bytes: harmless, nothing is stored for it
                const uint4* src = reinterpret_cast<const uint4*>(ring_g + cons_off + (u * PIECES + ci * TPP) * PIECE_STRIDE);
                float a[8];
                if (TPP == 1) {
                    unpack_bf16x8(src[0], a);
                } else {
                    const uint4 lo = src[0], hi = src[SEARCH_THREADS];
                    a[0] = __uint_as_float(lo.x); a[1] = __uint_as_float(lo.y);
                    a[2] = __uint_as_float(lo.z); a[3] = __uint_as_float(lo.w);
                    a[4] = __uint_as_float(hi.x); a[5] = __uint_as_float(hi.y);
                    a[6] = __uint_as_float(hi.z); a[7] = __uint_as_float(hi.w);
                }
                if (FULLD || (lane + GROUP * ci) * 8 < P.dim) {
#pragma unroll
                    for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);
                }
            }
            float v[GT];
#pragma unroll
            for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
            return HeadReduce<GT>::run(v, lane, 0xffffffffu);  // the whole warp runs every step
        };
        if (s_dense && tile_rows % (SEARCH_GROUPS * RPI) == 0) {
            // Every parent slot of the tile is full and kept for every head (the usual case:
            // the gates prune little): group g owns the rows [g*R, (g+1)*R) of the tile itself,
            // so the source pointer and the score index only step forward and nothing per row
            // needs testing.
            // The CTA's 16 groups take 16 consecutive rows per sub-step, so one step of the CTA
            // reads SEARCH_GROUPS * RPI consecutive rows (8 KB of bf16 at D=128).
            constexpr int STEP_ROWS = SEARCH_GROUPS * RPI;
            const int n_it = tile_rows / STEP_ROWS;
            const char* isrc = gbase + (size_t)grp * row_bytes;
            float* cdst = s_score + (size_t)grp * GT + my_head;
            const size_t sub_bytes = (size_t)SEARCH_GROUPS * row_bytes;
            auto issue_dense = [&](uint32_t stage_off) {
#pragma unroll
                for (int u = 0; u < RPI; ++u) {
#pragma unroll
                    for (int pc = 0; pc < PIECES; ++pc) {
                        const int coff = (pc / TPP) * GROUP * 8 * (int)sizeof(T) + (pc % TPP) * 16;
                        if (FULLD || (lane + GROUP * (pc / TPP)) * 8 < P.dim)
                            cp_async_16s(ring_s + stage_off + (u * PIECES + pc) * PIECE_STRIDE, isrc + u * sub_bytes + coff);
                    }
                }
                isrc += RPI * sub_bytes;
            };
            {
                uint32_t so = 0;
#pragma unroll
                for (int it = 0; it < STAGES - 1; ++it) {
                    if (it < n_it) issue_dense(so);
                    cp_async_commit();
                    so += STAGE_STRIDE;
                }
            }
            if (FULLD && n_it >= STAGES && n_it % STAGES == 0) {
                // Whole rounds of the ring, unrolled: slots, source offsets and score offsets are
                // constants of the instruction stream.  Step k of a round works on slot k and
                // refills slot k-1 with the step STAGES-1 ahead.
                constexpr int RB = 64 * NCH * (int)sizeof(T);          // bytes per row (FULLD)
                constexpr int SUB = SEARCH_GROUPS * RB;                 // bytes per sub-step of the CTA
                auto round = [&](bool last) {
#pragma unroll
                    for (int k = 0; k < STAGES; ++k) {
                        if (!last || k == 0) {
                            const uint32_t slot = (uint32_t)((k + STAGES - 1) % STAGES) * STAGE_STRIDE;
#pragma unroll
                            for (int u = 0; u < RPI; ++u)
#pragma unroll
                                for (int pc = 0; pc < PIECES; ++pc) {
                                    const int coff = (pc / TPP) * GROUP * 8 * (int)sizeof(T) + (pc % TPP) * 16;
                                    cp_async_16s(ring_s + slot + (u * PIECES + pc) * PIECE_STRIDE,
                                                 isrc + (k * RPI + u) * SUB + coff);
                                }
                        }
                        cp_async_commit();
                        cp_async_wait<STAGES - 1>();
#pragma unroll
                        for (int u = 0; u < RPI; ++u) {
                            const float d = row_score((uint32_t)k * STAGE_STRIDE, u);
                            if (writer && (emit_all || d >= leaf_thr)) cdst[(k * RPI + u) * SEARCH_GROUPS * GT] = d;
                        }
                    }
                    isrc += STAGES * RPI * SUB;
                    cdst += STAGES * STEP_ROWS * GT;
                };
                const int n_rounds = n_it / STAGES;
                for (int r = 0; r < n_rounds - 1; ++r) round(false);
                round(true);
            } else {
                uint32_t issue_off = (STAGES - 1) * STAGE_STRIDE, cons_off = 0;
                for (int it = 0; it < n_it; ++it) {
                    if (it + STAGES - 1 < n_it) issue_dense(issue_off);
                    cp_async_commit();
                    issue_off = (issue_off == (STAGES - 1) * STAGE_STRIDE) ? 0 : issue_off + STAGE_STRIDE;
                    cp_async_wait<STAGES - 1>();
#pragma unroll
                    for (int u = 0; u < RPI; ++u) {
                        const float d = row_score(cons_off, u);
                        if (writer && (emit_all || d >= leaf_thr)) cdst[u * SEARCH_GROUPS * GT] = d;
                    }
                    cdst += STEP_ROWS * GT;
                    cons_off = (cons_off == (STAGES - 1) * STAGE_STRIDE) ? 0 : cons_off + STAGE_STRIDE;
                }
            }
        } else {
            const int total = npass * bf;
            int R = (total + SEARCH_GROUPS - 1) / SEARCH_GROUPS;
            R = (R + RPI - 1) / RPI * RPI;
            const int n_it = R / RPI;

            // cursor over the rows of this group: parent-list position k, child c, parent word w
            struct Cursor { int k, c, cnt; uint32_t w; };
            auto load_parent = [&](Cursor& cu) {
                cu.w = cu.k < npass ? s_pl[cu.k] : 0u;
                cu.cnt = (int)(cu.w & 0x7ffu);
            };
            Cursor ic, cc;
            ic.k = div_bf(grp * R, bf, P.bf_magic);
            ic.c = grp * R - ic.k * bf;
            load_parent(ic);
            cc = ic;
            const char* isrc = gbase + (size_t)((ic.w >> 19) * bf + ic.c) * row_bytes;
            float* cdst = s_score + (size_t)((cc.w >> 19) * bf + cc.c) * GT + my_head;
            bool cgate = (cc.w >> (11 + my_head)) & 1u;

            auto issue_rows = [&](uint32_t stage_off) {
    #pragma unroll
                for (int u = 0; u < RPI; ++u) {
                    if (ic.c < ic.cnt) {
    #pragma unroll
                        for (int pc = 0; pc < PIECES; ++pc) {
                            const int coff = (pc / TPP) * GROUP * 8 * (int)sizeof(T) + (pc % TPP) * 16;
                            if (FULLD || (lane + GROUP * (pc / TPP)) * 8 < P.dim)
                                cp_async_16s(ring_s + stage_off + (u * PIECES + pc) * PIECE_STRIDE, isrc + coff);
                        }
                    }
                    ++ic.c;
                    isrc += row_bytes;
                    if (ic.c == bf) {
                        ic.c = 0;
                        ++ic.k;
                        load_parent(ic);
                        isrc = gbase + (size_t)((ic.w >> 19) * bf) * row_bytes;
                    }
                }
            };
            {
                uint32_t so = 0;
    #pragma unroll
                for (int it = 0; it < STAGES - 1; ++it) {
                    if (it < n_it) issue_rows(so);
                    cp_async_commit();
                    so += STAGE_STRIDE;
                }
            }
            uint32_t issue_off = (STAGES - 1) * STAGE_STRIDE, cons_off = 0;
            for (int it = 0; it < n_it; ++it) {
                if (it + STAGES - 1 < n_it) issue_rows(issue_off);
                cp_async_commit();
                issue_off = (issue_off == (STAGES - 1) * STAGE_STRIDE) ? 0 : issue_off + STAGE_STRIDE;
                cp_async_wait<STAGES - 1>();
    #pragma unroll
                for (int u = 0; u < RPI; ++u) {
                    const float d = row_score(cons_off, u);
                    if (writer && cgate && cc.c < cc.cnt && (emit_all || d >= leaf_thr)) *cdst = d;
                    ++cc.c;
                    cdst += GT;
                    if (cc.c == bf) {
                        cc.c = 0;
                        ++cc.k;
                        load_parent(cc);
                        cdst = s_score + (size_t)((cc.w >> 19) * bf) * GT + my_head;
                        cgate = (cc.w >> (11 + my_head)) & 1u;
                    }
                }
                cons_off = (cons_off == (STAGES - 1) * STAGE_STRIDE) ? 0 : cons_off + STAGE_STRIDE;
            }
        }
        cp_async_wait<0>();
        __syncthreads();
    } else {
        __syncthreads();  // the score sentinel must be visible to the compaction warps
    }

    // ---- 6. ordered compaction (one warp per head) + dense output -------------
    if (warp < nq) {
        const int j = warp;
        const int qh = s_qh[j];
        const float scale = s_scale[j];
        const bool want_compact = P.out_idx != nullptr;
        const size_t out_base = (size_t)qh * cap_children + tile_c0;
        const uint32_t* sc = reinterpret_cast<const uint32_t*>(s_score);
        int offset = 0;
        if (P.out_dense) {
            for (int base = 0; base < tile_rows; base += 32) {
                const int i = base + wl;
                const uint32_t bits = (i < tile_rows) ? sc[(size_t)i * GT + j] : NOT_EMITTED;
                const bool k = bits != NOT_EMITTED;
                const float emitted = __fmul_rn(__uint_as_float(bits), scale);
                const uint32_t b = __ballot_sync(0xffffffffu, k);
                if (want_compact && k) {
                    const int pos = offset + __popc(b & ((1u << wl) - 1u));
                    P.out_idx[out_base + pos] = (int32_t)(tile_c0 + i);
                    P.out_score[out_base + pos] = emitted;
                }
                offset += __popc(b);
                if (i < tile_rows && tile_c0 + i < cap_children) P.out_dense[out_base + i] = k ? emitted : 0.f;
            }
        } else {
            // Pass 1: one ballot per 32 rows, all loads independent; lane i keeps the bitmap of
            // rows [32 i, 32 i + 32) (a tile has at most 32 such words).
            static_assert(MAX_TILE_ROWS <= 1024, "one bitmap word per lane");
            uint32_t mybits = 0;
#pragma unroll 8
            for (int it = 0; it < 32; ++it) {
                const int i = it * 32 + wl;
                const uint32_t bits = (i < tile_rows) ? sc[(size_t)i * GT + j] : NOT_EMITTED;
                const uint32_t b = __ballot_sync(0xffffffffu, bits != NOT_EMITTED);
                if (wl == it) mybits = b;
            }
            const int cnt = __popc(mybits);
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, d);
                if (wl >= d) incl += t;
            }
            const int total = __shfl_sync(0xffffffffu, incl, 31);
            if (!want_compact) {
                // only the count is wanted
            } else if (total <= 4 * 32) {
                // few rows emitted: every lane writes out the rows of its own word
                int pos = incl - cnt;
                uint32_t m = mybits;
                while (m) {
                    const int i = wl * 32 + (__ffs((int)m) - 1);
                    m &= m - 1;
                    P.out_idx[out_base + pos] = (int32_t)(tile_c0 + i);
                    P.out_score[out_base + pos] = __fmul_rn(__uint_as_float(sc[(size_t)i * GT + j]), scale);
                    ++pos;
                }
            } else {
                // many rows emitted: word by word, so that the stores of a warp are contiguous
                for (int it = 0; it < 32; ++it) {
                    const uint32_t b = __shfl_sync(0xffffffffu, mybits, it);
                    if (b == 0) continue;
                    if ((b >> wl) & 1u) {
                        const int i = it * 32 + wl;
                        const int pos = offset + __popc(b & ((1u << wl) - 1u));
                        P.out_idx[out_base + pos] = (int32_t)(tile_c0 + i);
                        P.out_score[out_base + pos] = __fmul_rn(__uint_as_float(sc[(size_t)i * GT + j]), scale);
                    }
                    offset += __popc(b);
                }
            }
            offset = total;
        }
        if (wl == 0) {
            if (want_compact) P.out_count[(size_t)qh * P.n_tiles + tile] = offset;
            if (P.stats) {
                uint32_t* st = P.stats + (size_t)qh * HIRA_SEARCH_STATS;
                for (int k = 0; k < 8; ++k)
                    if (k != 5 && s_stat[j][k]) atomicAdd(st + k, s_stat[j][k]);
                if (offset) atomicAdd(st + 5, (uint32_t)offset);
            }
        }
    }
}

template <typename T, int GT, int NCH, int STAGES, int MINB, bool FULLD, int RPI, bool SCAN>
static int launch_search_sc(SearchParams P, int chunks, cudaStream_t stream) {
    constexpr int SEARCH_THREADS = 128;    // 4 warps: one compaction warp per head
    constexpr int BLOCKS = MINB;           // 128-thread CTAs resident per SM
    auto kern = search_kernel<T, GT, NCH, STAGES, BLOCKS, FULLD, SEARCH_THREADS, RPI, SCAN>;
    const size_t tile_rows = (size_t)P.tile_parents * P.bf;
    size_t off = tile_rows * GT * sizeof(float) + (size_t)P.tile_parents * (4 + 2 + 1 + 1);
    off = (off + 15) & ~(size_t)15;
    P.ring_offset = (uint32_t)off;
    const size_t pieces = (size_t)NCH * (sizeof(T) / 2);
    const size_t smem = off + (size_t)STAGES * RPI * pieces * SEARCH_THREADS * 16;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("hira_search: cudaFuncSetAttribute(%zu B smem): %s", smem, cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
    }
    P.n_chunks = chunks;
    HIRA_CHECK_ARG(P.n_tiles <= 65535 && P.n_heads <= 65535, HIRA_ERR_SHAPE,
                   "hira_search: %d tiles x %d heads exceed the grid limits", P.n_tiles, P.n_heads);
    dim3 grid((unsigned)chunks, (unsigned)P.n_tiles_active, (unsigned)P.n_heads);
    kern<<<grid, SEARCH_THREADS, smem, stream>>>(P);
    HIRA_CHECK_LAUNCH("hira_search launch");
    return HIRA_OK;
}

template <typename T, int GT, int NCH, int STAGES, int MINB, bool FULLD, int RPI>
static int launch_search_fd(const SearchParams& P, int chunks, cudaStream_t stream) {
    if (P.scan_out != nullptr) return launch_search_sc<T, GT, NCH, STAGES, MINB, FULLD, RPI, true>(P, chunks, stream);
    return launch_search_sc<T, GT, NCH, STAGES, MINB, FULLD, RPI, false>(P, chunks, stream);
}

// FULLD: every lane's chunks lie inside the row (D == 64 * NCH), so the per-chunk bounds tests drop out
template <typename T, int GT, int NCH, int STAGES, int MINB, int RPI = SEARCH_RPI>
static int launch_search(const SearchParams& P, int chunks, cudaStream_t stream) {
    if (P.dim == 64 * NCH) return launch_search_fd<T, GT, NCH, STAGES, MINB, true, RPI>(P, chunks, stream);
    return launch_search_fd<T, GT, NCH, STAGES, MINB, false, RPI>(P, chunks, stream);
}

template <typename T, int NCH>
static int dispatch_gt(const SearchParams& P, int max_group, cudaStream_t stream) {
    int gt = 1;
    while (gt < max_group && gt < 4) gt <<= 1;   // larger groups run as several 4-head chunks sharing L2
    if (NCH == 4 && gt > 2) gt = 2;  // D > 128: keep the query registers within budget
    const int chunks = (max_group + gt - 1) / gt;
    constexpr bool BF = sizeof(T) == 2;
    constexpr int ST = BF ? (NCH == 2 ? 4 : 2) : 2;  // ring = ST * SEARCH_RPI * pieces * 4 KB
    switch (gt) {
        case 1: return launch_search<T, 1, NCH, ST, 4>(P, chunks, stream);
        case 2: return launch_search<T, 2, NCH, ST, NCH == 4 ? 2 : 4>(P, chunks, stream);
        default: break;
    }
    if constexpr (NCH < 4) {
        if (gt == 4) return launch_search<T, 4, NCH, ST, 4>(P, chunks, stream);
    }
    set_error("hira_search: internal dispatch error");
    return HIRA_ERR_ARG;
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

static int search_impl(const hira_index_t* ix, const float* q, const float* tau,
                       const float* scaling, const float* qnorm, const int32_t* q2kv,
                       int32_t n_qheads, int32_t max_group, int32_t flags,
                       int32_t tile_parents, float* out_dense, int32_t* out_idx,
                       float* out_score, int32_t* out_count, uint32_t* stats,
                       const void* scan_key, int64_t scan_key_stride, unsigned long long* scan_out, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    if (scan_out != nullptr) {
        HIRA_CHECK_ARG(scan_key != nullptr && ix->parent_sqnorm != nullptr, HIRA_ERR_ARG,
                       "hira_search_scan: scan_key and the index's parent_sqnorm cache are required");
        HIRA_CHECK_ARG(q2kv == nullptr, HIRA_ERR_ARG,
                       "hira_search_scan: the fused scan needs the default head grouping (q2kv == NULL), so that "
                       "every kv head is visited");
    }
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
    P.scan_key = scan_key; P.scan_key_stride = scan_key_stride; P.scan_out = scan_out;
    P.parent_sqnorm = ix->parent_sqnorm;
    P.n_heads = ix->n_heads; P.n_qheads = n_qheads; P.group = group; P.depth = ix->depth;
    P.bf = bf; P.dim = ix->dim; P.cap_parents = ix->cap_parents; P.cap_gp = ix->cap_gp;
    P.tile_parents = tile_parents;
    P.n_tiles = (ix->cap_parents + tile_parents - 1) / tile_parents;
    // the dense row is written whole (callers reuse the buffer), the compact output only where keys can be
    P.n_tiles_active = out_dense ? P.n_tiles : active_tiles(ix, tile_parents);
    P.flags = flags;
    P.bf_magic = (uint32_t)((0x100000000ull + (uint64_t)bf - 1) / (uint64_t)bf);
    P.ring_offset = 0;
    P.ng = (tile_parents + bf - 1) / bf;
    if (tile_parents % bf == 0) {
        P.tile_gp_shift = -1;
    } else {
        const int ratio = bf / tile_parents;  // tiles per grandparent (depth 3: bf % tile_parents == 0)
        int sh = 0;
        while ((1 << sh) < ratio) ++sh;
        if (ix->depth == 3 && bf % tile_parents == 0 && (1 << sh) == ratio) {
            P.tile_gp_shift = sh;
        } else {
            P.tile_gp_shift = -2;
            HIRA_CHECK_ARG(ix->cap_parents <= (1 << 20), HIRA_ERR_SHAPE,
                           "hira_search: cap_parents=%d too large for tile_parents=%d with bf=%d", ix->cap_parents, tile_parents, bf);
        }
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // int8 pre-filter on the tensor cores when the index carries the side copy and the call allows it
    if (search_q8_applicable(ix, P)) return launch_search_q8(P, ix, max_group, s);
    const bool wide = ix->dim > 128;
    if (ix->dtype == HIRA_BF16)
        return wide ? dispatch_gt<__nv_bfloat16, 4>(P, max_group, s) : dispatch_gt<__nv_bfloat16, 2>(P, max_group, s);
    return wide ? dispatch_gt<float, 4>(P, max_group, s) : dispatch_gt<float, 2>(P, max_group, s);
}

extern "C" int hira_search(const hira_index_t* ix, const float* q, const float* tau,
                           const float* scaling, const float* qnorm, const int32_t* q2kv,
                           int32_t n_qheads, int32_t max_group, int32_t flags,
                           int32_t tile_parents, float* out_dense, int32_t* out_idx,
                           float* out_score, int32_t* out_count, uint32_t* stats, void* stream) {
    return search_impl(ix, q, tau, scaling, qnorm, q2kv, n_qheads, max_group, flags, tile_parents, out_dense,
                       out_idx, out_score, out_count, stats, nullptr, 0, nullptr, stream);
}

extern "C" int hira_search_scan(const hira_index_t* ix, const float* q, const float* tau,
                                const float* scaling, const float* qnorm, int32_t n_qheads, int32_t flags,
                                int32_t tile_parents, float* out_dense, int32_t* out_idx,
                                float* out_score, int32_t* out_count, uint32_t* stats,
                                const void* scan_key, int64_t scan_key_stride, uint64_t* scan_out, void* stream) {
    HIRA_CHECK_ARG(scan_out != nullptr, HIRA_ERR_ARG, "hira_search_scan: scan_out must not be NULL");
    return search_impl(ix, q, tau, scaling, qnorm, nullptr, n_qheads, 0, flags, tile_parents, out_dense,
                       out_idx, out_score, out_count, stats, scan_key, scan_key_stride,
                       reinterpret_cast<unsigned long long*>(scan_out), stream);
}
