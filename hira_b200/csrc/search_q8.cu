// Halfspace search with an int8 pre-filter on the tensor cores (D = 128, leaf rules >= / >).
//
// The streaming search kernel (search.cu) reads every child row of a kept parent in the
// index dtype (256 B per bf16 key) and is instruction-issue bound on the dot products.  This
// kernel reads a SIDE COPY of the children instead -- int8 rows of 128 B, quantised per row
// after a per-channel rescale -- scores 128 rows at a time against the CTA's query heads
// with tcgen05.mma (kind::i8, exact int32 accumulation in TMEM), and keeps as CANDIDATES the
// rows whose score could reach the threshold given a rigorous bound on the quantisation
// error.  Only the candidates (a few per cent) are then read in the index dtype and decided
// by the canonical fp32 dot product, exactly as search.cu decides them: the emitted sets and
// scores are bit-identical, the bytes per key roughly halve.
//
// Side copy (hira_index_t::children_q8, children_q8_meta, q8_chan_scale), per head:
//   s_i   per-channel scale (rms of channel i over the stored keys), k'_i = k_i / s_i
//   row   k~_i = rint(k'_i / step), step = max_i |k'_i| / 127, stored as int8 with the
//         16-byte chunks of the row permuted for the 128-byte shared-memory swizzle
//         (chunk j of slot r sits at chunk j ^ (r & 7)), so that a plain bulk copy of 128
//         consecutive rows lands in the layout tcgen05.mma reads
//   meta  (step, err) with err >= ||k' - step k~||_2 plus a share for the rounding of the
//         canonical dot product
// Query head: q' = q (.) s is split into two int8 terms, q' = c1 a1 + c2 a2 + r2.  Then
//   q.k = step (c1 a1.k~ + c2 a2.k~) + step r2.k~ + q'.(k' - step k~)
// and the last two terms are bounded by  B step + A err  (A = ||q'||, B = 127 ||r2||_1).
//
// Per CTA (one tile of <= 1024 child slots of one kv head, up to 4 query heads): warps 0-3
// compute the gates exactly as search.cu does, then own the 128 TMEM lanes = the 128 rows of
// a stage; lane 0 of warp 4 streams the needed 16 KB stages (+ 1 KB of meta) through a
// 4-slot ring with cp.async.bulk (no multicast) and issues the MMAs.  Every mbarrier wait
// is bounded; if one runs out the CTA falls back to treating every row of a kept parent as a
// candidate, so the result is still exact.
#include "common.cuh"
#include "search_common.cuh"
#include "tc_common.cuh"
#include <math_constants.h>
#include <cuda_fp16.h>

namespace hira {

constexpr int Q8_DIM = 128;
constexpr int Q8_STAGE_ROWS = 128;
constexpr int Q8_STAGE_BYTES = Q8_STAGE_ROWS * Q8_DIM;    // 16 KB of int8 rows
constexpr int Q8_META_BYTES = Q8_STAGE_ROWS * 4;          // (step, err) per row as two fp16
constexpr int Q8_SLOTS = 4;                               // stages in flight per CTA
constexpr int Q8_MAX_STAGES = MAX_TILE_ROWS / Q8_STAGE_ROWS;   // 8
constexpr int Q8_NCOL = 16;                               // accumulator columns per stage (N of the MMA)
constexpr int Q8_TMEM_COLS = Q8_MAX_STAGES * Q8_NCOL;     // 128
constexpr int Q8_THREADS = 160;                           // 4 worker warps + 1 producer/MMA warp
constexpr int Q8_WORKERS = 128;
constexpr int Q8_MAX_TP = 128;                            // parents per tile (bf >= 8)
// Bound of every mbarrier wait of the search kernel: 20 M cycles (about 10 ms), three orders of magnitude
// above the longest legitimate wait (a bulk copy, four MMAs).  A CTA whose wait runs out falls back to the
// exact path, so the bound only limits what such an event costs the step.
constexpr unsigned long long Q8_WAIT_CYCLES = 20ull * 1000 * 1000;
constexpr int Q8_HINT = 132;   // q8_chan_scale[h][132..134] as uint32: stages kept / stages of the last search, stream-all flag
constexpr int Q8_QBYTES = HIRA_Q8_QUERY_BYTES;            // prepared query terms of one (kv head, chunk of 4 heads)
static_assert(Q8_QBYTES == 2048 + 64, "B operand (16 rows x 128 B) + (c1, c2, A, B) of 4 heads");

// All of the kernel's shared memory is dynamic and 1024-byte aligned: 72 KB, three CTAs per SM.
struct Q8Smem {
    static constexpr int RING = 0;                                    // Q8_SLOTS stages of rows; later the candidates' scores
    static constexpr int BQ = Q8_SLOTS * Q8_STAGE_BYTES;              // 16 x 128 int8 query terms (B operand) + constants
    static constexpr int META = BQ + 2176;                            // [Q8_MAX_STAGES][128] (step, err); later the candidate list
    static constexpr int LIST = META;                                 // [1024] uint16 (row | head mask << 10), ascending rows
    static constexpr int SEG = META + Q8_MAX_STAGES * Q8_META_BYTES;  // [32 segments][32] candidates; during the gates: the scanned key
    static constexpr int PCOUNT = SEG + 2 * MAX_TILE_ROWS;            // [Q8_MAX_TP] int
    static constexpr int PMASK = PCOUNT + 4 * Q8_MAX_TP;              // [Q8_MAX_TP] bytes
    static constexpr int GPMASK = PMASK + Q8_MAX_TP;                  // [Q8_MAX_TP] bytes
    static constexpr int SCAN = GPMASK + Q8_MAX_TP;                   // [16] uint64
    static constexpr int STAT = SCAN + 128;                           // [4][8] uint32
    static constexpr int MISC = STAT + 128;                           // small scalars, see the kernel
    static constexpr int BAR = MISC + 256;                            // full[Q8_SLOTS], done[Q8_MAX_STAGES], go, query
    static constexpr int TMEM_SLOT = BAR + 8 * (Q8_SLOTS + Q8_MAX_STAGES + 2);
    static constexpr int TOTAL = TMEM_SLOT + 16;
};
static_assert(2 * MAX_TILE_ROWS <= Q8_MAX_STAGES * Q8_META_BYTES, "the candidate list fits where the meta rows were");
static_assert(Q8Smem::META % 16 == 0 && Q8Smem::BAR % 8 == 0 && Q8Smem::SCAN % 8 == 0, "bulk-copy and mbarrier alignment");

// kind::i8: D = int32, A = B = signed int8, both K-major, M = 128, N = 16
constexpr uint32_t Q8_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(Q8_NCOL >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// plain (non-multicast) bulk copy global -> this CTA's shared memory, completion on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(Q8_WORKERS) : "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// block reductions over the 128 workers of GT values each (sum or max); every worker gets the results
template <int GT, bool MAX>
__device__ __forceinline__ void worker_reduce(float (&v)[GT], float (*s_red)[8], int warp, int wl) {
#pragma unroll
    for (int j = 0; j < GT; ++j) {
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, v[j], s);
            v[j] = MAX ? fmaxf(v[j], o) : v[j] + o;
        }
    }
    worker_sync();   // s_red free again
    if (wl == 0) {
#pragma unroll
        for (int j = 0; j < GT; ++j) s_red[warp][j] = v[j];
    }
    worker_sync();
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        const float a = s_red[0][j], b = s_red[1][j], c = s_red[2][j], d = s_red[3][j];
        v[j] = MAX ? fmaxf(fmaxf(a, b), fmaxf(c, d)) : (a + b) + (c + d);
    }
}

// The query heads of one (kv head, chunk) as the B operand of the MMA, once per search: worker t owns
// channel t.  q' = q (.) s is split into two int8 terms, q' = c1 a1 + c2 a2 + r2; out = 16 rows of
// 128 int8 (row 2j = a1 of head j, row 2j+1 = a2; 16-byte chunks swizzled by the row; absent heads
// zero) followed by (c1, c2, A, B) per head with A >= ||q'||_2, B >= 127 ||r2||_1 + rounding.
__global__ void __launch_bounds__(Q8_WORKERS)
search_q8_prepare_kernel(const float* __restrict__ q, const float* __restrict__ chan_scale, float* chan_scale_rw,
                         int group, int gt, int dim, unsigned char* __restrict__ out) {
    constexpr int GT = 4;
    __shared__ float s_red[4][8];
    // The search kernel behind this one is launched with programmatic stream serialisation: its CTAs may
    // start (barriers, tensor memory, gates) while this grid runs, and wait for it (griddepcontrol.wait)
    // where they first need the query terms or the hint words.
    asm volatile("griddepcontrol.launch_dependents;");
    const int tid = threadIdx.x, warp = tid >> 5, wl = tid & 31;
    const int chunk = blockIdx.x, h = blockIdx.y;
    int nq = group - chunk * gt;
    nq = nq < 0 ? 0 : (nq > gt ? gt : nq);
    const float cs = chan_scale[(size_t)h * HIRA_Q8_CHAN + tid];
    float qp[GT], v[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        qp[j] = j < nq ? q[(size_t)(h * group + chunk * gt + j) * dim + tid] * cs : 0.f;
        v[j] = fabsf(qp[j]);
    }
    worker_reduce<GT, true>(v, s_red, warp, wl);
    float c1[GT], a1[GT], r1[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        c1[j] = v[j] > 0.f ? v[j] / 127.0f : 1.0f;
        a1[j] = fminf(fmaxf(rintf(qp[j] / c1[j]), -127.f), 127.f);
        r1[j] = __fmaf_rn(-a1[j], c1[j], qp[j]);
        v[j] = fabsf(r1[j]);
    }
    worker_reduce<GT, true>(v, s_red, warp, wl);
    float c2[GT], a2[GT], l1[GT], sq[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) {
        c2[j] = v[j] > 0.f ? v[j] / 127.0f : 1.0f;
        a2[j] = fminf(fmaxf(rintf(r1[j] / c2[j]), -127.f), 127.f);
        l1[j] = fabsf(__fmaf_rn(-a2[j], c2[j], r1[j]));
        sq[j] = qp[j] * qp[j];
    }
    worker_reduce<GT, false>(l1, s_red, warp, wl);
    worker_reduce<GT, false>(sq, s_red, warp, wl);
    if (chunk == 0 && tid == 0) {
        // How the previous search of this head went decides how this one streams: if the gates kept
        // at least 3/4 of the stages, every stage of a tile is requested before its gates are known
        // (they overlap the stream); otherwise only the first few are.  Results never depend on it.
        uint32_t* hint = reinterpret_cast<uint32_t*>(chan_scale_rw + (size_t)h * HIRA_Q8_CHAN + Q8_HINT);
        const uint32_t kept = hint[0], total = hint[1];
        if (total != 0) hint[2] = (4ull * kept >= 3ull * total) ? 1u : 0u;
        hint[0] = 0u;
        hint[1] = 0u;
    }
    unsigned char* dst = out + ((size_t)h * gridDim.x + chunk) * Q8_QBYTES;
    const int ch16 = tid >> 4, byte = tid & 15;
#pragma unroll
    for (int n = 0; n < Q8_NCOL; ++n) {
        float val = 0.f;
        if (n < 2 * GT) val = (n & 1) ? a2[n >> 1] : a1[n >> 1];
        const int off = (n >> 3) * 1024 + (n & 7) * 128 + ((ch16 ^ (n & 7)) << 4) + byte;
        reinterpret_cast<signed char*>(dst)[off] = (signed char)(int)val;
    }
    if (tid < GT) {
        const int j = tid;
        float* qc = reinterpret_cast<float*>(dst + 2048) + 4 * j;
        const float A = sqrtf(sq[j]) * 1.001f;
        qc[0] = c1[j];
        qc[1] = c2[j];
        qc[2] = A;
        // |r2 . k~| <= ||r2||_1 * 127, plus the rounding of the split itself
        qc[3] = 127.0f * l1[j] * 1.001f + A * (127.0f * 11.32f * 3.9e-6f);
    }
}

// CTAs of this device that took the exact fallback because a bounded wait ran out (or the shared-memory
// window was misaligned) since the library was loaded: read with hira_q8_fallback_count
__device__ unsigned int g_q8_fallbacks;

#ifdef HIRA_Q8_PROFILE
__device__ unsigned long long g_q8_prof[16384][16];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define Q8_STAMP(slot, who)                                                                       \
    do {                                                                                          \
        const unsigned lin__ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;     \
        if (threadIdx.x == (who) && lin__ < 16384) g_q8_prof[lin__][slot] = gtime();              \
    } while (0)
#else
#define Q8_STAMP(slot, who) do { } while (0)
#endif

template <typename T, int GT, bool SCAN>
__global__ void __launch_bounds__(Q8_THREADS, 3)
search_q8_kernel(const SearchParams P, const int8_t* __restrict__ k8, const uint32_t* __restrict__ k8_meta,
                 const unsigned char* __restrict__ qterms, uint32_t* __restrict__ hints) {
    constexpr int NCH = 2;
    constexpr int SEARCH_GROUPS = Q8_WORKERS / GROUP;  // 16
    constexpr int PRE = 2;
    extern __shared__ __align__(1024) unsigned char sm[];
    const uint32_t s_base = smem_u32(sm);
    // Candidates: the 128 rows of a stage are 4 segments of 32 (one per worker warp); segment
    // s * 4 + warp lists its candidate rows in ascending order as (lane | head mask << 8).
    unsigned short* s_seg = reinterpret_cast<unsigned short*>(sm + Q8Smem::SEG);
    unsigned short* s_list = reinterpret_cast<unsigned short*>(sm + Q8Smem::LIST);   // all segments, concatenated
    const uint32_t* s_meta = reinterpret_cast<const uint32_t*>(sm + Q8Smem::META);
    uint32_t* s_cscore = reinterpret_cast<uint32_t*>(sm + Q8Smem::RING);   // after the last MMA: [candidate][GT]
    const uint32_t bar_full = s_base + Q8Smem::BAR;                   // [Q8_SLOTS] stage landed
    const uint32_t bar_done = bar_full + 8 * Q8_SLOTS;                // [Q8_MAX_STAGES] MMAs of the k-th stage complete
    const uint32_t bar_go = bar_done + 8 * Q8_MAX_STAGES;             // gates known
    const uint32_t bar_q = bar_go + 8;                                // prepared query terms landed
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(sm + Q8Smem::TMEM_SLOT);
    int* s_pcount = reinterpret_cast<int*>(sm + Q8Smem::PCOUNT);
    unsigned char* s_pmask = sm + Q8Smem::PMASK;
    unsigned char* s_gpmask = sm + Q8Smem::GPMASK;
    unsigned long long* s_scan = reinterpret_cast<unsigned long long*>(sm + Q8Smem::SCAN);
    uint32_t (*s_stat)[8] = reinterpret_cast<uint32_t (*)[8]>(sm + Q8Smem::STAT);
    float* s_xkey = reinterpret_cast<float*>(sm + Q8Smem::SEG);          // [lane][chunk][8]; dead before the first candidate is listed
    int* misc = reinterpret_cast<int*>(sm + Q8Smem::MISC);
    int* s_qh = misc;                                         // [4]
    float* s_scale = reinterpret_cast<float*>(misc + 4);      // [4]
    float* s_tau = reinterpret_cast<float*>(misc + 8);        // [4]
    int& s_nq = misc[12];
    int& s_need = misc[13];
    int& s_ncand = misc[14];
    int& s_fail = misc[15];
    int* s_wcount = misc + 16;                                // [Q8_MAX_STAGES * 4] candidates per segment
    int& s_stream_all = misc[48];                             // the head's streaming mode, read once for the whole CTA
    static_assert(GROUP * NCH * 8 * 4 <= 2 * MAX_TILE_ROWS, "the scanned key fits in the candidate segments' place");

    const int TP = P.tile_parents;
    const int bf = P.bf;
    const int tile_rows = TP * bf;
    const int tid = threadIdx.x;
    const int lane = tid & (GROUP - 1);
    const int grp = tid / GROUP;
    const int warp = tid >> 5;
    const int wl = tid & 31;
    const bool worker = warp < 4;
    const int chunk = blockIdx.x;
    const int tile = blockIdx.y;
    const int h = blockIdx.z;
    const bool ge = P.flags & HIRA_GATE_GE;
    const int leaf_mode = P.flags & (HIRA_LEAF_GE | HIRA_LEAF_GT);
    const size_t cap_children = (size_t)P.cap_parents * bf;
    const T* children = reinterpret_cast<const T*>(P.children) + (size_t)h * cap_children * P.dim;
    const T* parents = reinterpret_cast<const T*>(P.parents) + (size_t)h * P.cap_parents * P.dim;

    // ---- 1. query heads of this kv head handled by this CTA (as in search.cu) -------------
    if (tid < GT * 8) (&s_stat[0][0])[tid] = 0;
    if (tid < Q8_MAX_STAGES * 4) s_wcount[tid] = 0;
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
    if (nq == 0) return;  // uniform over the CTA; nothing allocated yet
    Q8_STAMP(0, 0);

    // ---- 0. barriers, tensor memory ----------------------------------------------------------
    // The operand tiles need a 1024-byte aligned base (the kernel has no static shared memory, so the
    // dynamic window starts aligned); should a driver ever place it otherwise, the tensor path is left
    // out and every row of a kept parent is scored exactly.
    const bool aligned = (s_base & 1023u) == 0u;
    if (tid == 0) {
        s_fail = aligned ? 0 : 1;
        s_need = 0;
        s_ncand = 0;
        // One thread reads the streaming mode for the whole CTA: the kernel that prepares the query terms
        // (and may flip the mode word) can still be running when this CTA starts, and the producer and the
        // workers must agree on the stages that are requested up front.
        s_stream_all = (int)*reinterpret_cast<volatile uint32_t*>(hints + (size_t)h * HIRA_Q8_CHAN + Q8_HINT + 2);
        for (int i = 0; i < Q8_SLOTS; ++i) mbar_init(bar_full + 8 * i, 1);
        for (int i = 0; i < Q8_MAX_STAGES; ++i) mbar_init(bar_done + 8 * i, 1);
        mbar_init(bar_go, 1);
        mbar_init(bar_q, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(s_base + Q8Smem::TMEM_SLOT), "r"(Q8_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    Q8_STAMP(1, 0);

    const int tile_p0 = tile * TP;
    const size_t tile_c0 = (size_t)tile_p0 * bf;
    const int n_stage_tile = tile_rows / Q8_STAGE_ROWS;
    // stages requested before the gates are known: none for a tile beyond the slots in use
    const bool tile_in_use = P.depth == 3 ? (P.tile_gp_shift >= 0 ? (tile >> P.tile_gp_shift)
                                             : (P.tile_gp_shift == -1 ? tile * P.ng : div_bf(tile * TP, bf, P.bf_magic))) < P.used[h * 4 + 1]
                                          : tile_p0 < P.used[h * 4 + 0];
    uint32_t* hint = hints + (size_t)h * HIRA_Q8_CHAN + Q8_HINT;
    const bool stream_all = s_stream_all != 0;
    const int spec = tile_in_use ? ((stream_all || n_stage_tile < Q8_SLOTS) ? n_stage_tile : Q8_SLOTS) : 0;

    if (!worker) {
        // ======================= producer + MMA issuer (one thread) =========================
        if (tid == Q8_WORKERS && aligned) {
            // The first stages of a tile that holds keys are requested at once, before the gates are
            // known (they are nearly always needed; at most Q8_SLOTS stages are read for nothing when
            // the gates prune the whole tile); the rest follows the gates.
            // the stage requests first: the query terms come from the kernel launched just before this one
            const int8_t* rows_g = k8 + ((size_t)h * cap_children + tile_c0) * Q8_DIM;
            const uint32_t* meta_g = k8_meta + (size_t)h * cap_children + tile_c0;
            int order[Q8_MAX_STAGES] = {0, 0, 0, 0, 0, 0, 0, 0};
            int n = spec, issued = 0;
            bool failed = false, got_go = false;
            auto issue = [&](int i) {
                const int slot = i % Q8_SLOTS;
                const uint32_t full = bar_full + 8 * slot;
                mbar_expect_tx(full, Q8_STAGE_BYTES + Q8_META_BYTES);
                bulk_load(s_base + Q8Smem::RING + slot * Q8_STAGE_BYTES, rows_g + (size_t)order[i] * Q8_STAGE_BYTES,
                          Q8_STAGE_BYTES, full);
                bulk_load(s_base + Q8Smem::META + i * Q8_META_BYTES, meta_g + (size_t)order[i] * Q8_STAGE_ROWS,
                          Q8_META_BYTES, full);
            };
            for (int i = 0; i < spec; ++i) order[i] = i;
            for (; issued < spec && issued < Q8_SLOTS; ++issued) issue(issued);
            Q8_STAMP(8, Q8_WORKERS);
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the query terms are written
            mbar_expect_tx(bar_q, Q8_QBYTES);
            bulk_load(s_base + Q8Smem::BQ, qterms + ((size_t)h * P.n_chunks + chunk) * Q8_QBYTES, Q8_QBYTES, bar_q);
            for (int k = 0; !failed; ++k) {
                if (!got_go && k >= spec) {
                    if (!mbar_wait(bar_go, 0, Q8_WAIT_CYCLES)) { failed = true; break; }
                    got_go = true;
                    const int need = *reinterpret_cast<volatile int*>(&s_need);
                    for (int s = spec; s < n_stage_tile; ++s)
                        if ((need >> s) & 1) order[n++] = s;
                }
                if (k >= n) break;
                while (issued < n && issued < k + Q8_SLOTS) {
                    // the slot held stage issued - Q8_SLOTS: free once its MMAs are complete
                    if (issued >= Q8_SLOTS && !mbar_wait(bar_done + 8 * (issued - Q8_SLOTS), 0, Q8_WAIT_CYCLES)) { failed = true; break; }
                    issue(issued);
                    ++issued;
                }
                if (failed) break;
                const int slot = k % Q8_SLOTS;
                if (k == 0 && !mbar_wait(bar_q, 0, Q8_WAIT_CYCLES)) { failed = true; break; }
                if (!mbar_wait(bar_full + 8 * slot, (k / Q8_SLOTS) & 1, Q8_WAIT_CYCLES)) { failed = true; break; }
                if (k == 0) Q8_STAMP(9, Q8_WORKERS);
                if (k == 3) Q8_STAMP(11, Q8_WORKERS);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = s_base + Q8Smem::RING + slot * Q8_STAGE_BYTES, b0 = s_base + Q8Smem::BQ;
#pragma unroll
                for (int ks = 0; ks < Q8_DIM / 32; ++ks)
                    umma_i8(tmem + k * Q8_NCOL, umma_desc(a0 + ks * 32), umma_desc(b0 + ks * 32), Q8_IDESC, ks > 0 ? 1u : 0u);
                umma_commit(bar_done + 8 * k);
            }
            Q8_STAMP(10, Q8_WORKERS);
            if (failed) {
                *reinterpret_cast<volatile int*>(&s_fail) = 1;
                // let copies that may still be in flight land before the ring is reused (bounded)
                mbar_wait(bar_q, 0, Q8_WAIT_CYCLES);
                for (int i = 0; i < issued && i < Q8_SLOTS; ++i) mbar_wait(bar_full + 8 * i, ((issued - 1 - i) / Q8_SLOTS) & 1, Q8_WAIT_CYCLES);
            }
        }
    } else {
        // ================================ workers (128 threads) ================================
        const int my_head = HeadReduce<GT>::head_of_lane(lane);
        const bool head_on = my_head < nq;
        const bool has_qn = false;   // this kernel is only launched for unit queries (qnorm == NULL)
        const int used_parents = P.used[h * 4 + 0];
        const int used_gp = P.used[h * 4 + 1];
        const int g0 = P.tile_gp_shift >= 0 ? (tile >> P.tile_gp_shift)
                                            : (P.tile_gp_shift == -1 ? tile * P.ng : div_bf(tile * TP, bf, P.bf_magic));
        const int ng = P.ng;
        int my_qh = qh_of[0];
#pragma unroll
        for (int j = 1; j < GT; ++j)
            if (my_head == j) my_qh = qh_of[j];
        const float my_tau = head_on ? P.tau[my_qh] : 0.f;
        const float my_qn = 1.f;
        if (tid < nq) {
            s_scale[tid] = P.scaling ? P.scaling[s_qh[tid]] : 1.0f;
            s_tau[tid] = P.tau[s_qh[tid]];
        }
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
        // gate inputs, issued together (as in search.cu)
        RawChunk<T> graw[NCH];
        float grad = 0.f;
        const bool gp_mine = P.depth == 3 && grp < ng && (g0 + grp) < P.cap_gp;
        {
            const T* gps = reinterpret_cast<const T*>(P.gps) + (size_t)h * P.cap_gp * P.dim;
            load_row_raw<T, NCH>(graw, gps + (size_t)(g0 + grp) * P.dim, lane, P.dim, gp_mine);
            if (gp_mine) grad = P.gp_radii[(size_t)h * P.cap_gp + g0 + grp];
        }
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
        const bool do_scan = SCAN && chunk == 0;
        float psq[PRE];
        if (do_scan) {
            if constexpr (SCAN) {
                if (tid < GROUP) {
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
        unsigned long long scan_best = ~0ull;

        bool tile_empty;
        if (P.depth == 3) tile_empty = g0 >= used_gp;
        else tile_empty = tile_p0 >= used_parents;
        const uint32_t allmask = (1u << nq) - 1u;

        if (!tile_empty) {
            // ---- 3a. grandparent gate ----------------------------------------------------
            if (P.depth == 3) {
                const T* gps = reinterpret_cast<const T*>(P.gps) + (size_t)h * P.cap_gp * P.dim;
                for (int i0 = 0; i0 < ng; i0 += SEARCH_GROUPS) {
                    const int i = i0 + grp;
                    const int g = g0 + i;
                    const bool valid = (i < ng) && (g < used_gp);
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
                        if (valid && P.stats && tile_p0 == g0 * bf) {
                            for (int jj = 0; jj < nq; ++jj) {
                                atomicAdd(&s_stat[jj][0], 1u);
                                if ((m >> jj) & 1u) atomicAdd(&s_stat[jj][1], 1u);
                            }
                        }
                    }
                }
            }
            worker_sync();

            // ---- 3b. parent gate -----------------------------------------------------------
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
                if (do_scan && valid) {
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
                        atomicAdd(&s_stat[0][7], 1u);
                        if (m != 0) atomicAdd(&s_stat[0][6], (uint32_t)cnt);
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
            auto scan_score = [&](const RawChunk<T> (&raw)[NCH], float sqn) -> float {
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
                    return __fsub_rn(sqn, __fmul_rn(2.0f, d));
                } else {
                    return 0.f;
                }
            };
#pragma unroll
            for (int u = 0; u < PRE; ++u) {
                if (u * SEARCH_GROUPS < TP) {
                    float ss = 0.f;
                    if (do_scan) ss = scan_score(praw[u], psq[u]);
                    gate_parent(u * SEARCH_GROUPS, gate_dot_raw<T, GT, NCH>(praw[u], qreg, lane), prad[u], pcnt[u], pgc[u], ss);
                }
            }
            for (int i0 = PRE * SEARCH_GROUPS; i0 < TP; i0 += SEARCH_GROUPS) {
                const int p = tile_p0 + i0 + grp;
                const bool in = (i0 + grp < TP) && (p < P.cap_parents);
                const float d = gate_dot<T, GT, NCH>(parents + (size_t)p * P.dim, qreg, lane, P.dim, in);
                const float r = in ? P.parent_radii[(size_t)h * P.cap_parents + p] : 0.f;
                const int cnt = in ? P.child_counts[(size_t)h * P.cap_parents + p] : 0;
                const int gc = (in && P.depth == 3) ? P.gp_counts[(size_t)h * P.cap_gp + g0 + div_bf(p - g0 * bf, bf, P.bf_magic)] : 0;
                float ss = 0.f;
                if (do_scan) {
                    RawChunk<T> raw[NCH];
                    load_row_raw<T, NCH>(raw, parents + (size_t)p * P.dim, lane, P.dim, in);
                    ss = scan_score(raw, in ? P.parent_sqnorm[(size_t)h * P.cap_parents + p] : 0.f);
                }
                gate_parent(i0, d, r, cnt, gc, ss);
            }
            if (do_scan && lane == 0) s_scan[grp] = scan_best;
            worker_sync();

            // ---- 4. stages that hold rows of a kept parent; nearest parent of the tile -------
            if (tid < n_stage_tile) {
                const int p_lo = div_bf(tid * Q8_STAGE_ROWS, bf, P.bf_magic);
                int p_hi = div_bf(tid * Q8_STAGE_ROWS + Q8_STAGE_ROWS - 1, bf, P.bf_magic);
                p_hi = p_hi >= TP ? TP - 1 : p_hi;
                bool any = false;
                for (int i = p_lo; i <= p_hi; ++i) {
                    // rows of parent i inside this stage that are filled
                    const int first = i * bf > tid * Q8_STAGE_ROWS ? 0 : tid * Q8_STAGE_ROWS - i * bf;
                    any = any || (s_pmask[i] != 0 && s_pcount[i] > first);
                }
                if (any) atomicOr(&s_need, 1 << tid);
            } else if (warp == 1 && do_scan) {
                unsigned long long best = wl < SEARCH_GROUPS ? s_scan[wl] : ~0ull;
#pragma unroll
                for (int sft = 16; sft >= 1; sft >>= 1) {
                    const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, sft);
                    best = o < best ? o : best;
                }
                if (wl == 0 && best != ~0ull) atomicMin(P.scan_out + h, best);
            }
        }
        worker_sync();   // s_need, s_pmask, s_pcount are complete; the scanned key is no longer needed
        Q8_STAMP(2, 0);
        if (tid == 0) {
            mbar_arrive(bar_go);
            if (chunk == 0 && tile_in_use) {   // what the gates kept, for the next search's streaming mode
                asm volatile("griddepcontrol.wait;" ::: "memory");   // the counters of the last search are consumed
                atomicAdd(hint, (uint32_t)__popc(*reinterpret_cast<volatile int*>(&s_need)));
                atomicAdd(hint + 1, (uint32_t)n_stage_tile);
            }
        }
        const int need = *reinterpret_cast<volatile int*>(&s_need) | ((1 << spec) - 1);   // the stages requested up front come first

        // a stage's candidates into its warp's segment, in row order
        auto list_candidate = [&](int s, uint32_t cm) {
            const uint32_t bal = __ballot_sync(0xffffffffu, cm != 0u);
            if (cm) s_seg[(s * 4 + warp) * 32 + __popc(bal & ((1u << wl) - 1u))] = (unsigned short)(wl | (cm << 8));
            if (wl == 0) s_wcount[s * 4 + warp] = __popc(bal);
        };

        // ---- 5. candidates: approximate scores out of tensor memory ----------------------------
        {
            bool failed = !aligned;
            if (aligned) {   // the prepared query terms and their constants arrive by a bulk copy
                const bool ok = mbar_wait(bar_q, 0, Q8_WAIT_CYCLES);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    if (wl == 0) *reinterpret_cast<volatile int*>(&s_fail) = 1;
                }
            }
            Q8_STAMP(3, 0);
            const float* s_qc = reinterpret_cast<const float*>(sm + Q8Smem::BQ + 2048);
            float qc[GT][4], tauj[GT];
#pragma unroll
            for (int j = 0; j < GT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) qc[j][e] = s_qc[4 * j + e];
                tauj[j] = j < nq ? s_tau[j] : CUDART_INF_F;
            }
            int k = 0;
            for (int s = 0; s < n_stage_tile; ++s) {   // uniform over the workers
                if (failed) break;
                if (!((need >> s) & 1)) continue;
                // warp-uniform outcome: tcgen05.ld below is a warp-wide instruction
                const bool ok = mbar_wait(bar_done + 8 * k, 0, Q8_WAIT_CYCLES) && !*reinterpret_cast<volatile int*>(&s_fail);
                if (!__all_sync(0xffffffffu, ok)) {
                    failed = true;
                    if (wl == 0) *reinterpret_cast<volatile int*>(&s_fail) = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t acc[16];
                tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + k * Q8_NCOL, acc);
                const int r = s * Q8_STAGE_ROWS + tid;
                const int pl = div_bf(r, bf, P.bf_magic);
                const uint32_t pm = s_pmask[pl];
                const bool filled = (r - pl * bf) < s_pcount[pl];
                const uint32_t mw = s_meta[k * Q8_STAGE_ROWS + tid];   // (step, err) as two fp16
                const float step = __half2float(__ushort_as_half((unsigned short)(mw & 0xffffu)));
                const float err = __half2float(__ushort_as_half((unsigned short)(mw >> 16)));
                uint32_t cm = 0;
#pragma unroll
                for (int j = 0; j < GT; ++j) {
                    const float d1 = __int2float_rn((int)acc[2 * j]), d2 = __int2float_rn((int)acc[2 * j + 1]);
                    const float approx = step * __fmaf_rn(qc[j][0], d1, qc[j][1] * d2);
                    const float margin = __fmaf_rn(qc[j][2], err, qc[j][3] * step);
                    const float upper = approx + margin * 1.001f + 1e-6f + 1e-6f * fabsf(approx);
                    if (upper >= tauj[j]) cm |= 1u << j;
                }
                cm = filled ? (cm & pm) : 0u;
                list_candidate(s, cm);
                if (cm) {   // the exact pass reads this row in the index dtype: start it towards L2 now
                    const char* row = reinterpret_cast<const char*>(children + (tile_c0 + r) * P.dim);
                    prefetch_l2(row);
                    if (sizeof(T) * Q8_DIM > 128) prefetch_l2(row + 128);
                    if (sizeof(T) * Q8_DIM > 256) { prefetch_l2(row + 256); prefetch_l2(row + 384); }
                }
                ++k;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            worker_sync();
            Q8_STAMP(4, 0);
            if (*reinterpret_cast<volatile int*>(&s_fail)) {   // the same for every worker after the barrier
                // a bounded wait ran out: every filled row of a kept parent is a candidate (exact, only slower)
                if (tid == 0) atomicAdd(&g_q8_fallbacks, 1u);
                for (int s = 0; s < n_stage_tile; ++s) {
                    const int r = s * Q8_STAGE_ROWS + tid;
                    const int pl = div_bf(r, bf, P.bf_magic);
                    list_candidate(s, ((r - pl * bf) < s_pcount[pl] && !tile_empty) ? (uint32_t)s_pmask[pl] : 0u);
                }
                worker_sync();
            }
        }

        // ---- 6. the segments concatenated into one ascending list (each warp copies 8 segments) ---
        int ncand;
        {
            const int cnt = wl < n_stage_tile * 4 ? s_wcount[wl] : 0;   // lane i: candidates of segment i
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, d);
                if (wl >= d) incl += t;
            }
            ncand = __shfl_sync(0xffffffffu, incl, 31);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int seg = warp * 8 + i;
                const int c = __shfl_sync(0xffffffffu, cnt, seg), off = __shfl_sync(0xffffffffu, incl, seg) - c;
                if (wl < c) {
                    const int e = s_seg[seg * 32 + wl];
                    s_list[off + wl] = (unsigned short)((seg * 32 + (e & 31)) | ((e >> 8) << 10));
                }
            }
        }
        worker_sync();
        Q8_STAMP(5, 0);

        // ---- 7. exact scores of the candidates, canonical arithmetic ---------------------------
        {
            const bool writer = HeadReduce<GT>::is_writer(lane);
            const float leaf_thr = (leaf_mode == HIRA_LEAF_GT) ? nextafterf(my_tau, CUDART_INF_F) : my_tau;
            constexpr int XR = 2;   // candidate rows per group and iteration: their loads are in flight together
            const int iters = (ncand + XR * SEARCH_GROUPS - 1) / (XR * SEARCH_GROUPS);   // uniform over the workers
            for (int it = 0; it < iters; ++it) {
                int e[XR], r[XR];
                RawChunk<T> raw[XR][NCH];
#pragma unroll
                for (int u = 0; u < XR; ++u) {
                    e[u] = (it * XR + u) * SEARCH_GROUPS + grp;
                    r[u] = e[u] < ncand ? s_list[e[u]] : -1;   // row | head mask << 10
#pragma unroll
                    for (int ci = 0; ci < NCH; ++ci)
                        raw[u][ci] = r[u] >= 0 ? load_chunk_stream<T>(children + (tile_c0 + (r[u] & 1023)) * P.dim, lane + GROUP * ci)
                                               : zero_chunk<T>();
                }
#pragma unroll
                for (int u = 0; u < XR; ++u) {
                    const float d = gate_dot_raw<T, GT, NCH>(raw[u], qreg, lane);
                    if (writer && r[u] >= 0) {
                        const bool em = head_on && ((r[u] >> (10 + my_head)) & 1) && d >= leaf_thr;
                        s_cscore[e[u] * GT + my_head] = em ? __float_as_uint(d) : NOT_EMITTED;
                    }
                }
            }
        }
        worker_sync();
        Q8_STAMP(6, 0);

        // ---- 8. ordered compaction, one warp per head -------------------------------------------
        if (warp < nq) {
            const int j = warp;
            const int qh = s_qh[j];
            const float scale = s_scale[j];
            const size_t out_base = (size_t)qh * cap_children + tile_c0;
            int offset = 0;
            for (int base = 0; base < ncand; base += 32) {
                const int e = base + wl;
                const uint32_t bits = e < ncand ? s_cscore[e * GT + j] : NOT_EMITTED;
                const bool k = bits != NOT_EMITTED;
                const uint32_t b = __ballot_sync(0xffffffffu, k);
                if (k) {
                    const int pos = offset + __popc(b & ((1u << wl) - 1u));
                    P.out_idx[out_base + pos] = (int32_t)(tile_c0 + (s_list[e] & 1023));
                    P.out_score[out_base + pos] = __fmul_rn(__uint_as_float(bits), scale);
                }
                offset += __popc(b);
            }
            if (wl == 0) {
                P.out_count[(size_t)qh * P.n_tiles + tile] = offset;
                if (P.stats) {
                    uint32_t* st = P.stats + (size_t)qh * HIRA_SEARCH_STATS;
                    for (int k = 0; k < 8; ++k)
                        if (k != 5 && s_stat[j][k]) atomicAdd(st + k, s_stat[j][k]);
                    if (offset) atomicAdd(st + 5, (uint32_t)offset);
                    if (j == 0) {
                        if (ncand) atomicAdd(st + 8, (uint32_t)ncand);                           // rows re-read in the index dtype
                        // int8 rows scored (none when a bounded wait ran out and the CTA fell back)
                        if (need && !*reinterpret_cast<volatile int*>(&s_fail))
                            atomicAdd(st + 9, (uint32_t)(__popc(need) * Q8_STAGE_ROWS));
                    }
                }
            }
        }
    }

    Q8_STAMP(7, 0);
    // ---- 9. tensor memory back ----------------------------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Q8_TMEM_COLS) : "memory");
    }
}

template <typename T, int GT, bool SCAN>
static int launch_q8(SearchParams P, int chunks, const hira_index_t* ix, cudaStream_t stream) {
    auto kern = search_q8_kernel<T, GT, SCAN>;
    const size_t smem = Q8Smem::TOTAL;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        set_error("hira_search (int8 pre-filter): cudaFuncSetAttribute(%zu B smem): %s", smem, cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    P.n_chunks = chunks;
    HIRA_CHECK_ARG(P.n_tiles <= 65535 && P.n_heads <= 65535, HIRA_ERR_SHAPE,
                   "hira_search: %d tiles x %d heads exceed the grid limits", P.n_tiles, P.n_heads);
    unsigned char* qterms = reinterpret_cast<unsigned char*>(ix->q8_query_scratch);
    search_q8_prepare_kernel<<<dim3((unsigned)chunks, (unsigned)P.n_heads), Q8_WORKERS, 0, stream>>>(
        P.q, ix->q8_chan_scale, ix->q8_chan_scale, P.group, GT, P.dim, qterms);
    HIRA_CHECK_LAUNCH("hira_search (int8 pre-filter, query terms) launch");
    // launched so that its CTAs may start while the query terms are still being prepared (see above)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)chunks, (unsigned)P.n_tiles_active, (unsigned)P.n_heads);
    cfg.blockDim = dim3(Q8_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, P, reinterpret_cast<const int8_t*>(ix->children_q8),
                           reinterpret_cast<const uint32_t*>(ix->children_q8_meta),
                           reinterpret_cast<const unsigned char*>(qterms), reinterpret_cast<uint32_t*>(ix->q8_chan_scale));
    if (e != cudaSuccess) {
        set_error("hira_search (int8 pre-filter) launch: %s", cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    return HIRA_OK;
}

template <typename T, int GT>
static int launch_q8_scan(const SearchParams& P, int chunks, const hira_index_t* ix, cudaStream_t stream) {
    if (P.scan_out != nullptr) return launch_q8<T, GT, true>(P, chunks, ix, stream);
    return launch_q8<T, GT, false>(P, chunks, ix, stream);
}

bool search_q8_applicable(const hira_index_t* ix, const SearchParams& P) {
    if (!ix->children_q8 || !ix->children_q8_meta || !ix->q8_chan_scale || !ix->q8_query_scratch) return false;
    if (ix->dim != Q8_DIM || P.qnorm != nullptr || P.out_dense != nullptr || P.out_idx == nullptr) return false;
    if (P.q2kv != nullptr || P.group > 4 * HIRA_Q8_QUERY_CHUNKS) return false;   // default head grouping, <= 16 heads per kv head
    if ((P.flags & (HIRA_LEAF_GE | HIRA_LEAF_GT)) == 0) return false;           // every child is emitted: nothing to filter
    const int tile_rows = P.tile_parents * P.bf;
    if (P.bf < 8 || P.tile_parents > Q8_MAX_TP || tile_rows % Q8_STAGE_ROWS != 0 || tile_rows > MAX_TILE_ROWS) return false;
    if (P.cap_parents % P.tile_parents != 0) return false;                        // whole tiles only
    return true;
}

int launch_search_q8(const SearchParams& P, const hira_index_t* ix, int max_group, cudaStream_t stream) {
    int gt = 1;
    while (gt < max_group && gt < 4) gt <<= 1;
    const int chunks = (max_group + gt - 1) / gt;
    const bool bf16 = ix->dtype == HIRA_BF16;
    switch (gt) {
        case 1: return bf16 ? launch_q8_scan<__nv_bfloat16, 1>(P, chunks, ix, stream) : launch_q8_scan<float, 1>(P, chunks, ix, stream);
        case 2: return bf16 ? launch_q8_scan<__nv_bfloat16, 2>(P, chunks, ix, stream) : launch_q8_scan<float, 2>(P, chunks, ix, stream);
        default: return bf16 ? launch_q8_scan<__nv_bfloat16, 4>(P, chunks, ix, stream) : launch_q8_scan<float, 4>(P, chunks, ix, stream);
    }
}

// ---------------------------------------------------------------------------
// Building and maintaining the side copy.
// ---------------------------------------------------------------------------
// per head: rms of every channel over a strided sample of the filled child slots -> s_i, min_i s_i.
// Two kernels: slices of the sample summed by many CTAs (atomicAdd into the head's 128 accumulators,
// which are the scale array itself, and a row count at [135]), then one CTA per head finishes.
constexpr int Q8_CHAN_PARTS = 64;
template <typename T>
__global__ void q8_chan_sums_kernel(const hira_index_t ix) {
    const int h = blockIdx.y, part = blockIdx.x;
    const int c = threadIdx.x;   // channel
    const size_t capC = (size_t)ix.cap_parents * ix.bf;
    const T* rows = reinterpret_cast<const T*>(ix.children) + (size_t)h * capC * Q8_DIM;
    const int32_t* s2t = ix.slot2token ? ix.slot2token + (size_t)h * capC : nullptr;
    const int32_t* cc = ix.child_counts + (size_t)h * ix.cap_parents;
    const size_t n_slots = (size_t)(ix.depth == 3 ? ix.used[h * 4 + 1] * ix.bf : ix.used[h * 4 + 0]) * ix.bf;
    const size_t stride = n_slots > 16384 ? n_slots / 8192 : 1;
    const size_t n_samples = (n_slots + stride - 1) / stride;
    const size_t per = (n_samples + Q8_CHAN_PARTS - 1) / Q8_CHAN_PARTS;
    const size_t i0 = part * per, i1 = i0 + per < n_samples ? i0 + per : n_samples;
    float sum = 0.f;
    int cnt = 0;
    for (size_t i = i0; i < i1; ++i) {
        const size_t r = i * stride;
        const bool filled = s2t ? s2t[r] >= 0 : (int)(r % ix.bf) < cc[r / ix.bf];
        if (!filled) continue;
        const float v = sizeof(T) == 2 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rows)[r * Q8_DIM + c])
                                       : reinterpret_cast<const float*>(rows)[r * Q8_DIM + c];
        sum = __fmaf_rn(v, v, sum);
        ++cnt;
    }
    float* out = ix.q8_chan_scale + (size_t)h * HIRA_Q8_CHAN;
    if (cnt) atomicAdd(out + c, sum);
    if (c == 0 && cnt) atomicAdd(out + 135, (float)cnt);
}

__global__ void q8_chan_finish_kernel(const hira_index_t ix) {
    const int h = blockIdx.x;
    const int c = threadIdx.x;
    float* out = ix.q8_chan_scale + (size_t)h * HIRA_Q8_CHAN;
    const float cnt = out[135];
    float s = cnt > 0.f ? sqrtf(out[c] / cnt) : 1.f;
    if (!(s > 1e-20f) || !(s < 1e20f)) s = 1.f;
    __shared__ float s_min[4];
    float m = s;
#pragma unroll
    for (int sft = 16; sft >= 1; sft >>= 1) m = fminf(m, __shfl_xor_sync(0xffffffffu, m, sft));
    if ((c & 31) == 0) s_min[c >> 5] = m;
    __syncthreads();
    out[c] = s;
    if (c == 0) {
        out[Q8_DIM] = fminf(fminf(s_min[0], s_min[1]), fminf(s_min[2], s_min[3]));
        uint32_t* hint = reinterpret_cast<uint32_t*>(out + Q8_HINT);
        hint[0] = 0u;
        hint[1] = 0u;
        hint[2] = 1u;   // stream every stage until a search has shown that the gates prune
    }
}

// one 8-lane group per child slot: quantise the row (see q8_write_row in common.cuh)
template <typename T>
__global__ void q8_quantize_kernel(const hira_index_t ix, const size_t slots_bound) {
    const int lane = threadIdx.x & (GROUP - 1);
    const size_t capC = (size_t)ix.cap_parents * ix.bf;
    const int h = blockIdx.y;
    const size_t slot = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / GROUP;
    if (slot >= slots_bound) return;
    const size_t w = (size_t)h * capC + slot;   // (head, slot)
    // slots beyond the blocks in use hold no keys (and never did since the last clear): nothing to write
    const size_t in_use = (size_t)(ix.depth == 3 ? ix.used[h * 4 + 1] * ix.bf : ix.used[h * 4 + 0]) * ix.bf;
    if (slot >= in_use) return;
    const T* row = reinterpret_cast<const T*>(ix.children) + w * Q8_DIM;
    float x[2][8];
    load_vec<T, 2>(row, x, lane, Q8_DIM);
    q8_write_row(x, ix.q8_chan_scale + (size_t)h * HIRA_Q8_CHAN, reinterpret_cast<int8_t*>(ix.children_q8) + w * Q8_DIM,
                 reinterpret_cast<uint32_t*>(ix.children_q8_meta) + w, (int)(slot & 7), lane);
}

// parents_bound: parent slots that can hold keys (0 = the whole capacity); the grid covers only those
int q8_refresh(const hira_index_t* ix, cudaStream_t s, long long parents_bound) {
    if (!ix->children_q8) return HIRA_OK;
    HIRA_CHECK_ARG(ix->dim == Q8_DIM && ix->children_q8_meta && ix->q8_chan_scale, HIRA_ERR_ARG,
                   "the int8 side copy needs dim == 128 and its meta / channel-scale arrays");
    if (parents_bound <= 0 || parents_bound > ix->cap_parents) parents_bound = ix->cap_parents;
    const size_t slots_bound = (size_t)parents_bound * ix->bf;
    const dim3 blocks((unsigned)((slots_bound * GROUP + 255) / 256), (unsigned)ix->n_heads);
    cudaMemsetAsync(ix->q8_chan_scale, 0, (size_t)ix->n_heads * HIRA_Q8_CHAN * sizeof(float), s);
    const dim3 parts(Q8_CHAN_PARTS, (unsigned)ix->n_heads);
    if (ix->dtype == HIRA_BF16) {
        q8_chan_sums_kernel<__nv_bfloat16><<<parts, Q8_DIM, 0, s>>>(*ix);
        q8_chan_finish_kernel<<<ix->n_heads, Q8_DIM, 0, s>>>(*ix);
        q8_quantize_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(*ix, slots_bound);
    } else {
        q8_chan_sums_kernel<float><<<parts, Q8_DIM, 0, s>>>(*ix);
        q8_chan_finish_kernel<<<ix->n_heads, Q8_DIM, 0, s>>>(*ix);
        q8_quantize_kernel<float><<<blocks, 256, 0, s>>>(*ix, slots_bound);
    }
    HIRA_CHECK_LAUNCH("int8 side copy launch");
    return HIRA_OK;
}

}  // namespace hira

#ifdef HIRA_Q8_PROFILE
extern "C" int hira_q8_profile_read(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, hira::g_q8_prof, sizeof(hira::g_q8_prof)) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" int hira_q8_fallback_count(uint32_t* host_out) {
    HIRA_CHECK_ARG(host_out != nullptr, HIRA_ERR_ARG, "hira_q8_fallback_count: NULL argument");
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, hira::g_q8_fallbacks, sizeof(v));
    if (e != cudaSuccess) {
        hira::set_error("hira_q8_fallback_count: %s", cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    *host_out = v;
    return HIRA_OK;
}

extern "C" int hira_q8_refresh(const hira_index_t* ix, void* stream) {
    int rc = hira::validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(ix->children_q8 != nullptr, HIRA_ERR_ARG, "hira_q8_refresh: the index has no int8 side copy");
    return hira::q8_refresh(ix, reinterpret_cast<cudaStream_t>(stream), ix->active_parents);
}
