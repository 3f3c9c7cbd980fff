// Tensor-core nearest-centroid assignment (the dense contraction of the index build,
// torch.cdist + argmin at indexer/cuda.py:244-245) for bf16 points with D = 128.
//
// Per CTA: one tile of 128 points (A, 32 KB, loaded once by TMA) against all centroids of
// the head in tiles of 128 (B, 32 KB per tile, double-buffered TMA).  One elected thread
// issues tcgen05.mma (M=128, N=128, K=16, bf16 in, fp32 accumulate in TMEM: 128 lanes x 128
// columns), tcgen05.commit signals an mbarrier, then 256 threads read the accumulator with
// tcgen05.ld (two threads per point, 64 columns each, the next 32 columns in flight while 32 are
// reduced) and fold score = ||c||^2 - 2 x.c into a running arg-min, so the (points x centroids)
// matrix never leaves the SM.  The tile's ||c||^2 sit in shared memory, fetched one tile ahead.
// Two TMEM accumulators alternate (the MMAs of the next centroid tile run while the previous one
// is read out) and two CTAs are resident per SM.
//
// Every wait on an mbarrier is bounded; on a timeout the CTA writes index -1 for its points
// and leaves in an orderly way (TMEM freed).  No TMA multicast is used.
#include "common.cuh"
#include "tc_common.cuh"

#include <cuda.h>
#include <math_constants.h>

namespace hira {

constexpr int TC_BM = 128;       // points per CTA
constexpr int TC_BN = 128;       // centroids per tile
constexpr int TC_K = 128;        // D
constexpr int TC_BOX_K = 64;     // elements per 128-byte swizzle row
constexpr int TC_BOX_BYTES = TC_BM * TC_BOX_K * 2;   // 16 KB
constexpr int TC_EPI_THREADS = 256;  // 8 epilogue warps: warp w reads TMEM lanes 32 (w & 3) .. + 31, columns 64 (w >> 2) .. + 63 of a tile
constexpr int TC_THREADS = TC_EPI_THREADS + 32;   // + 1 producer/MMA warp

struct TcSmem {
    // offsets in the 1024-byte aligned dynamic shared memory
    static constexpr int A = 0;                          // 2 boxes
    static constexpr int B = 2 * TC_BOX_BYTES;           // 2 stages x 2 boxes
    static constexpr int CSQ = B + 4 * TC_BOX_BYTES;     // 2 stages x 128 squared centroid norms
    static constexpr int COMB = CSQ + 2 * TC_BN * 4;     // (score, index) of the upper column half, per point
    static constexpr int BAR = COMB + TC_BM * 8;         // bar_a, bar_b[2], bar_bfree[2], bar_full[2], bar_empty[2]
    static constexpr int TMEM_SLOT = BAR + 9 * 8;
    static constexpr int TOTAL = TMEM_SLOT + 16;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// kind::f16, D = fp32, A = B = bf16, both K-major, M = 128, N = 128
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float min3f(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// tcgen05.ld without its wait: the registers are valid only after tmem_ld_wait(r), which names them as
// in/out operands so that no use of them can be scheduled ahead of the wait
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Warps 0-7 (256 threads) run the arg-min epilogue: warp w owns TMEM lanes 32 (w & 3) .. + 31 = 32 of
// the 128 points, over the column half w >> 2 of every centroid tile (a warp may only read the lane
// quarter of its index mod 4, so two warps share each quarter); lane 0 of warp 8 issues the TMA loads
// and the MMAs.  Two accumulators (2 x 128 TMEM columns) alternate, so the MMAs of centroid tile j+1
// run while tile j is being read out.  All hand-offs are mbarriers with bounded waits.
__global__ void __launch_bounds__(TC_THREADS, 2)
assign_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __nv_bfloat16* __restrict__ points, long long p_head_stride,
                 const float* __restrict__ csq, int n, int k, int32_t* __restrict__ out_idx,
                 float* __restrict__ out_d2) {
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t s_base = smem_u32(sm);
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(sm + TcSmem::TMEM_SLOT);
    const uint32_t bar_a = s_base + TcSmem::BAR;
    const uint32_t bar_b = bar_a + 8;        // [2] centroid tile landed
    const uint32_t bar_bfree = bar_a + 24;   // [2] MMAs that read the stage are complete
    const uint32_t bar_full = bar_a + 40;    // [2] accumulator written
    const uint32_t bar_empty = bar_a + 56;   // [2] accumulator read out by all 128 epilogue threads
    __shared__ int s_fail;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int h = blockIdx.y;
    const int m0 = blockIdx.x * TC_BM;
    const int nt = (k + TC_BN - 1) / TC_BN;

    if (tid == 0) {
        s_fail = 0;
        mbar_init(bar_a, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_b + 8 * i, 1);
            mbar_init(bar_bfree + 8 * i, 1);
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, TC_EPI_THREADS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == TC_EPI_THREADS / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(s_base + TcSmem::TMEM_SLOT), "r"(2 * TC_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    bool failed = false;

    if (warp == TC_EPI_THREADS / 32) {
        if (tid == TC_EPI_THREADS) {
            // ---- producer + MMA issuer -------------------------------------------------------
            mbar_expect_tx(bar_a, 2 * TC_BOX_BYTES);
            tma_load_3d(s_base + TcSmem::A, &map_a, 0, m0, h, bar_a);
            tma_load_3d(s_base + TcSmem::A + TC_BOX_BYTES, &map_a, TC_BOX_K, m0, h, bar_a);
            mbar_expect_tx(bar_b, 2 * TC_BOX_BYTES);
            tma_load_3d(s_base + TcSmem::B, &map_b, 0, 0, h, bar_b);
            tma_load_3d(s_base + TcSmem::B + TC_BOX_BYTES, &map_b, TC_BOX_K, 0, h, bar_b);
            for (int j = 0; j < nt && !failed; ++j) {
                const int st = j & 1;
                if (j + 1 < nt) {
                    // the other stage held tile j-1: refill it once those MMAs are complete
                    const int s2 = (j + 1) & 1;
                    if (j >= 1 && !mbar_wait(bar_bfree + 8 * s2, ((j - 1) >> 1) & 1)) { failed = true; break; }
                    const uint32_t dst = s_base + TcSmem::B + s2 * 2 * TC_BOX_BYTES;
                    mbar_expect_tx(bar_b + 8 * s2, 2 * TC_BOX_BYTES);
                    tma_load_3d(dst, &map_b, 0, (j + 1) * TC_BN, h, bar_b + 8 * s2);
                    tma_load_3d(dst + TC_BOX_BYTES, &map_b, TC_BOX_K, (j + 1) * TC_BN, h, bar_b + 8 * s2);
                }
                bool ok = true;
                if (j == 0) ok = mbar_wait(bar_a, 0);
                ok = ok && mbar_wait(bar_b + 8 * st, (j >> 1) & 1);
                if (ok && j >= 2) ok = mbar_wait(bar_empty + 8 * st, ((j - 2) >> 1) & 1);   // accumulator drained
                if (!ok) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = s_base + TcSmem::A, b0 = s_base + TcSmem::B + st * 2 * TC_BOX_BYTES;
#pragma unroll
                for (int ks = 0; ks < TC_K / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * TC_BOX_BYTES + (ks & 3) * 32;
                    umma_f16(tmem + st * TC_BN, umma_desc(a0 + off), umma_desc(b0 + off), TC_IDESC, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar_bfree + 8 * st);
                umma_commit(bar_full + 8 * st);
            }
            if (failed) s_fail = 1;
        }
    } else {
        // ---- arg-min epilogue: thread (w, l) owns point m0 + 32 (w & 3) + l = that TMEM lane, over the
        //      column half w >> 2 of every tile; the two halves of a point are combined at the end ------
        const int pt = (warp & 3) * 32 + (tid & 31);   // point within the CTA
        const int half = warp >> 2;
        float best = CUDART_INF_F;
        int best_i = 0x7fffffff;
        const float* cs = csq + (size_t)h * k;
        // The squared norms of a centroid tile sit in shared memory: every thread fetches one norm of the
        // NEXT tile while it reads the current one out (past the last centroid: +inf, never the minimum),
        // and the 128 epilogue threads meet once per tile, so the fetch is never waited for.
        float* s_csq = reinterpret_cast<float*>(sm + TcSmem::CSQ);
        if (tid < TC_BN) s_csq[tid] = tid < k ? __ldg(cs + tid) : CUDART_INF_F;
        for (int j = 0; j < nt; ++j) {
            const int st = j & 1;
            const int cn = (j + 1) * TC_BN + tid;
            const float cnext = (tid < TC_BN && j + 1 < nt && cn < k) ? __ldg(cs + cn) : CUDART_INF_F;
            // everyone is done with tile j - 1 (whose norms stage st ^ 1 held) and has stored its norm of tile j
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_THREADS) : "memory");
            if (tid < TC_BN) s_csq[(st ^ 1) * TC_BN + tid] = cnext;
            // A thread whose wait ran out keeps walking the tiles (it only meets the others at the barrier
            // above, so nobody is left waiting there) and reports -1 for its point.
            if (failed) continue;
            if (!mbar_wait(bar_full + 8 * st, (j >> 1) & 1) || *reinterpret_cast<volatile int*>(&s_fail)) {
                failed = true;
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t0 = tmem + ((uint32_t)((warp & 3) * 32) << 16) + st * TC_BN + half * (TC_BN / 2);
            uint32_t r[2][32];
            tmem_ld32_nowait(t0, r[0]);
#pragma unroll
            for (int q = 0; q < TC_BN / 64; ++q) {
                // the next 32 columns are on their way while these 32 are reduced
                tmem_ld_wait(r[q & 1]);
                if (q + 1 < TC_BN / 64) tmem_ld32_nowait(t0 + (q + 1) * 32, r[(q + 1) & 1]);
                const int c0 = j * TC_BN + half * (TC_BN / 2) + q * 32;
                const float4* cq4 = reinterpret_cast<const float4*>(s_csq + st * TC_BN + half * (TC_BN / 2) + q * 32);
                float sc[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 v = cq4[i];
                    // 2*x.c is exact: same bits as csq - 2*dot; two scores per packed FMA
                    const float2 m2 = make_float2(-2.0f, -2.0f);
                    const float2 lo = __ffma2_rn(m2, make_float2(__uint_as_float(r[q & 1][4 * i]), __uint_as_float(r[q & 1][4 * i + 1])),
                                                 make_float2(v.x, v.y));
                    const float2 hi = __ffma2_rn(m2, make_float2(__uint_as_float(r[q & 1][4 * i + 2]), __uint_as_float(r[q & 1][4 * i + 3])),
                                                 make_float2(v.z, v.w));
                    sc[4 * i] = lo.x; sc[4 * i + 1] = lo.y; sc[4 * i + 2] = hi.x; sc[4 * i + 3] = hi.y;
                }
                // the minimum of the 32 scores by three-input minima (16 instead of 31 operations); the
                // index is looked up only when the running minimum improves (rare after the first tiles)
                float m1[12];
#pragma unroll
                for (int i = 0; i < 10; ++i) m1[i] = min3f(sc[3 * i], sc[3 * i + 1], sc[3 * i + 2]);
                m1[10] = sc[30];
                m1[11] = sc[31];
                const float cmin = fminf(min3f(min3f(m1[0], m1[1], m1[2]), min3f(m1[3], m1[4], m1[5]), min3f(m1[6], m1[7], m1[8])),
                                         min3f(m1[9], m1[10], m1[11]));
                if (cmin < best) {   // strict: an equal score later in the scan never replaces an earlier centroid
                    best = cmin;
                    int first = 31;
#pragma unroll
                    for (int i = 30; i >= 0; --i)
                        if (sc[i] == cmin) first = i;
                    best_i = c0 + first;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_empty + 8 * st);
        }
        // the two column halves of a point: the smaller score, on a tie the lower centroid (the earlier in the scan)
        float2* s_comb = reinterpret_cast<float2*>(sm + TcSmem::COMB);
        if (half == 1) s_comb[pt] = make_float2(failed ? CUDART_NAN_F : best, __int_as_float(best_i));
        asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_THREADS) : "memory");
        if (half == 0) {
            const float2 o = s_comb[pt];
            const int oi = __float_as_int(o.y);
            if (o.x != o.x) failed = true;   // the other half gave up
            else if (o.x < best || (o.x == best && oi < best_i)) { best = o.x; best_i = oi; }
        }
        const int p = m0 + pt;
        if (half == 0 && p < n) {
            if (failed) {
                out_idx[(size_t)h * n + p] = -1;
                out_d2[(size_t)h * n + p] = 0.f;
            } else {
                const __nv_bfloat16* row = points + (size_t)h * p_head_stride + (size_t)p * TC_K;
                float xsq = 0.f;
#pragma unroll 4
                for (int c = 0; c < TC_K / 8; ++c) {
                    float f[8];
                    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(row) + c), f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) xsq = __fmaf_rn(f[e], f[e], xsq);
                }
                out_idx[(size_t)h * n + p] = best_i;
                out_d2[(size_t)h * n + p] = fmaxf(__fadd_rn(xsq, best), 0.f);
            }
        }
    }
    if (tid == TC_EPI_THREADS && failed) {
        // let copies that may still be in flight land before the shared memory is given back (bounded)
        mbar_wait(bar_b, 0);
        mbar_wait(bar_b + 8, 0);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_EPI_THREADS / 32) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TC_BN) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// rows x 128 bf16 per head, head stride in elements; box = 64 elements x 128 rows, 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long head_stride, int n_heads) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)TC_K, (cuuint64_t)rows, (cuuint64_t)n_heads};
    const cuuint64_t strides[2] = {(cuuint64_t)TC_K * 2, (cuuint64_t)head_stride * 2};
    const cuuint32_t box[3] = {(cuuint32_t)TC_BOX_K, (cuuint32_t)TC_BM, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool assign_tc_supported(int dtype, int n, int k, int dim) {
    return dtype == HIRA_BF16 && dim == TC_K && n >= 1 && k >= 1;
}

int launch_assign_tc(const void* points, long long p_head_stride, const void* cents, const float* csq,
                     int n_heads, int n, int k, int dim, int32_t* out_idx, float* out_d2, cudaStream_t s) {
    HIRA_CHECK_ARG(dim == TC_K, HIRA_ERR_SHAPE, "tensor-core assignment needs dim == %d", TC_K);
    HIRA_CHECK_ARG(((uintptr_t)points & 15) == 0 && ((uintptr_t)cents & 15) == 0 && (p_head_stride % 8) == 0,
                   HIRA_ERR_ARG, "tensor-core assignment needs 16-byte aligned rows");
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, points, n, p_head_stride, n_heads) || !make_map(&map_b, cents, k, (long long)k * TC_K, n_heads)) {
        set_error("tensor-core assignment: cuTensorMapEncodeTiled failed or is unavailable");
        return HIRA_ERR_CUDA;
    }
    const size_t smem = TcSmem::TOTAL + 1024;
    cudaError_t e = cudaFuncSetAttribute(assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("assign_tc: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return HIRA_ERR_CUDA; }
    dim3 grid((unsigned)((n + TC_BM - 1) / TC_BM), (unsigned)n_heads);
    assign_tc_kernel<<<grid, TC_THREADS, smem, s>>>(map_a, map_b, reinterpret_cast<const __nv_bfloat16*>(points),
                                                    p_head_stride, csq, n, k, out_idx, out_d2);
    HIRA_CHECK_LAUNCH("assign_tc launch");
    return HIRA_OK;
}

}  // namespace hira
