// Gather-sparse flash-decode attention over the compacted search output, plus
// the log-sum-exp merge used for split-KV partials and for sequence shards.
//
// The reference names this step (attention/hira_attention.py:1-3) but ships no
// implementation; the contract here follows its searcher API: emitted scores
// already are the logits (scaling * q.k, searcher/cpu.py:58-63), the value rows
// sit in the same slots as the keys (indexer/cuda.py:397-423), and the keys not
// yet indexed arrive as a dense queue (cache/hira_cache.py:121-140).
//
// One CTA per (query head, split of the tile range).  8-lane groups each
// gather one value row (256 B for V=128 bf16) with two 128-bit loads per lane,
// four rows in flight per thread; softmax is online in fp32.
#include "common.cuh"
#include "merge_row.cuh"
#include <math_constants.h>
#include <atomic>

namespace hira {

constexpr int ATTN_THREADS = 128;
constexpr int ATTN_HW = ATTN_THREADS / GROUP;  // 8-lane groups: one value row per group per step
constexpr int ATTN_LIST = 1024;   // (slot, logit) entries per staging list; there are two lists
constexpr int ATTN_TB = 32;       // tiles whose counts are fetched and prefix-summed together
constexpr int QUEUE_FLAG = 0x40000000;

struct AttnParams {
    const void* values;
    const float* q;
    const float* scaling;
    const int32_t* q2kv;
    const int32_t* idx;
    const float* score;
    const int32_t* count;
    const void* queued_k;
    const void* queued_v;
    float* ws;
    float* out;     // with one split the kernel writes the normalised output (and out_ml) itself
    float* out_ml;
    int n_heads, n_qheads, group, dim, vdim, n_tiles, tile_rows, n_splits, n_queued;
    int n_tiles_active;  // tiles that can hold keys (<= n_tiles, the stride of `count`)
    long long cap_children;
    long long queued_head_stride;
    long long out_stride, ml_stride;  // elements between the heads' rows of out / out_ml
};

__device__ __forceinline__ void attn_cp_async_16(uint32_t smem_addr, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void attn_cp_async_4(uint32_t smem_addr, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void attn_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void attn_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// value rows in flight per 8-lane group: the ring of one CTA is ATTN_THREADS * 16 B * pieces * depth
template <typename TV, int NVCH>
struct GatherRing {
    static constexpr int TPP = (int)(sizeof(TV) / 2);       // 16-byte pieces per 8-element chunk
    static constexpr int PIECES = NVCH * TPP;               // 16-byte pieces per thread per row
    static constexpr int STAGE_BYTES = ATTN_THREADS * 16 * PIECES;
    static constexpr int DEPTH = STAGE_BYTES <= 4096 ? 6 : (STAGE_BYTES <= 8192 ? 3 : 2);  // 24 KB: five CTAs per SM
    static constexpr int BYTES = STAGE_BYTES * DEPTH;
};

template <typename TV, int NVCH>
__device__ __forceinline__ void accumulate_row(float (&acc)[NVCH][8], const RawChunk<TV> (&raw)[NVCH], float p) {
#pragma unroll
    for (int i = 0; i < NVCH; ++i) {
        float v[8];
        to_float(raw[i], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = __fmaf_rn(p, v[e], acc[i][e]);
    }
}

template <typename TK, typename TV, int NCH, int NVCH>
__global__ void __launch_bounds__(ATTN_THREADS)
sparse_attn_kernel(const AttnParams P) {
    __shared__ int s_idx[2][ATTN_LIST];
    __shared__ float s_logit[2][ATTN_LIST];
    __shared__ int s_cnt[2][ATTN_TB];
    __shared__ int s_off[2][ATTN_TB + 1];
    __shared__ float s_red[ATTN_HW];
    __shared__ float s_bcast;
    extern __shared__ __align__(16) float s_out[];  // [ATTN_HW][vdim] at the end; the gather ring before
    using Ring = GatherRing<TV, NVCH>;

    const int tid = threadIdx.x;
    const int lane = tid & (GROUP - 1);
    const int hw = tid / GROUP;
    const int warp = tid >> 5, wl = tid & 31;
    const int qh = blockIdx.y;
    const int split = blockIdx.x;
    const int h = P.q2kv ? P.q2kv[qh] : qh / P.group;
    const TV* values = reinterpret_cast<const TV*>(P.values) + (size_t)h * P.cap_children * P.vdim;
    const int t0 = (int)(((long long)split * P.n_tiles_active) / P.n_splits);
    const int t1 = (int)(((long long)(split + 1) * P.n_tiles_active) / P.n_splits);

    float m = -CUDART_INF_F;
    float l = 0.f;  // this group's share of the denominator
    float acc[NVCH][8];
#pragma unroll
    for (int i = 0; i < NVCH; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;

    // online-softmax step over one staged list: block maximum, rescale, gather + accumulate
    auto flush = [&](const int* s_idx, const float* s_logit, int fill) {
        __syncthreads();
        // block max of the staged logits
        float mx = -CUDART_INF_F;
        for (int i = tid; i < fill; i += ATTN_THREADS) mx = fmaxf(mx, s_logit[i]);
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        if (wl == 0) s_red[warp] = mx;
        __syncthreads();
        if (tid == 0) {
            float v = s_red[0];
            for (int w = 1; w < ATTN_THREADS / 32; ++w) v = fmaxf(v, s_red[w]);
            s_bcast = v;
        }
        __syncthreads();
        const float new_m = fmaxf(m, s_bcast);
        if (new_m > -CUDART_INF_F) {
            const float alpha = (m > -CUDART_INF_F) ? __expf(m - new_m) : 0.f;
            l *= alpha;
#pragma unroll
            for (int i = 0; i < NVCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] *= alpha;
            m = new_m;
            // Value rows through a private ring of asynchronous 16-byte copies: each thread keeps
            // DEPTH-1 rows of its group in flight ahead of the one it accumulates, and only reads
            // the pieces it copied itself, so the gather is a continuous stream without barriers.
            const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(s_out) + tid * 16;
            const unsigned char* ring_g = reinterpret_cast<const unsigned char*>(s_out) + tid * 16;
            const int n_rounds = (fill + ATTN_HW - 1) / ATTN_HW;  // uniform over the CTA
            auto issue = [&](int k) {
                const int e = k * ATTN_HW + hw;
                if (k < n_rounds && e < fill) {
                    const int id = s_idx[e];
                    const TV* row = (id & QUEUE_FLAG)
                        ? reinterpret_cast<const TV*>(P.queued_v) + (size_t)h * P.queued_head_stride + (size_t)(id & ~QUEUE_FLAG) * P.vdim
                        : values + (size_t)id * P.vdim;
                    const uint32_t dst = ring_s + (uint32_t)(k % Ring::DEPTH) * Ring::STAGE_BYTES;
#pragma unroll
                    for (int pc = 0; pc < Ring::PIECES; ++pc) {
                        const int c = lane + GROUP * (pc / Ring::TPP);
                        if (c * 8 < P.vdim)
                            attn_cp_async_16(dst + pc * (ATTN_THREADS * 16),
                                             reinterpret_cast<const char*>(row) + (size_t)c * 8 * sizeof(TV) + (pc % Ring::TPP) * 16);
                    }
                }
                attn_cp_async_commit();
            };
#pragma unroll
            for (int k = 0; k < Ring::DEPTH - 1; ++k) issue(k);
            for (int k = 0; k < n_rounds; ++k) {
                issue(k + Ring::DEPTH - 1);
                attn_cp_async_wait<Ring::DEPTH - 1>();
                const int e = k * ATTN_HW + hw;
                if (e < fill) {  // uniform inside the group
                    const float p = __expf(s_logit[e] - m);
                    const unsigned char* src = ring_g + (size_t)(k % Ring::DEPTH) * Ring::STAGE_BYTES;
                    RawChunk<TV> raw[NVCH];
#pragma unroll
                    for (int i = 0; i < NVCH; ++i) {
                        if ((lane + GROUP * i) * 8 < P.vdim) {
                            if constexpr (sizeof(TV) == 2) {
                                raw[i].a = *reinterpret_cast<const uint4*>(src + i * (ATTN_THREADS * 16));
                            } else {
                                raw[i].a = *reinterpret_cast<const float4*>(src + (2 * i) * (ATTN_THREADS * 16));
                                raw[i].b = *reinterpret_cast<const float4*>(src + (2 * i + 1) * (ATTN_THREADS * 16));
                            }
                        } else {
                            raw[i] = zero_chunk<TV>();
                        }
                    }
                    accumulate_row<TV, NVCH>(acc, raw, p);
                    l += p;
                }
            }
        }
        // The prefetches of the next list and of the next counts were issued without a group of
        // their own: they ride in the ring's groups above.  When the ring did not run (every staged
        // logit -inf or NaN) nothing has committed them yet, and wait_group only covers committed
        // groups -- so commit here, unconditionally (an empty group costs nothing).
        attn_cp_async_commit();
        attn_cp_async_wait<0>();
        __syncthreads();
    };

    // ---- emitted children of this split's tiles -------------------------------
    // A three-stage software pipeline over blocks of ATTN_TB tiles, all by asynchronous copies
    // into shared memory: (A) the tile counts of block b+2, (B) the (slot, logit) entries of
    // the next list (block b+1, or the next ATTN_LIST entries of a block that emitted more),
    // (C) maximum + gather of the current list.  A and B ride in the copy groups of C's value
    // ring, so while the value rows of one list stream in, the next list arrives as well.
    const int nblk = (t1 - t0 + ATTN_TB - 1) / ATTN_TB;
    auto fetch_counts = [&](int b) {  // A
        if (b < nblk && tid < ATTN_TB) {
            const int t = t0 + b * ATTN_TB + tid;
            if (t < t1) attn_cp_async_4((uint32_t)__cvta_generic_to_shared(&s_cnt[b & 1][tid]), P.count + (size_t)qh * P.n_tiles + t);
            else s_cnt[b & 1][tid] = 0;
        }
    };
    auto scan_counts = [&](int b) {   // prefix sums of a block whose counts have landed (warp 0)
        if (warp == 0) {
            const int c = s_cnt[b & 1][wl];
            int v = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, v, d);
                if (wl >= d) v += o;
            }
            s_off[b & 1][wl + 1] = v;
            if (wl == 0) s_off[b & 1][0] = 0;
        }
    };
    auto fetch_entries = [&](int b, int sub, int buf) {  // B
        const int* off = s_off[b & 1];
        const int v0 = sub * ATTN_LIST;
        const int n = min(ATTN_LIST, off[ATTN_TB] - v0);
        for (int i = tid; i < n; i += ATTN_THREADS) {
            const int v = v0 + i;
            int lo = 0;  // the tile of entry v: the last one whose prefix is <= v
#pragma unroll
            for (int step = ATTN_TB / 2; step >= 1; step >>= 1)
                if (off[lo + step] <= v) lo += step;
            const size_t at = (size_t)qh * P.cap_children + (size_t)(t0 + b * ATTN_TB + lo) * P.tile_rows + (size_t)(v - off[lo]);
            attn_cp_async_4((uint32_t)__cvta_generic_to_shared(&s_idx[buf][i]), P.idx + at);
            attn_cp_async_4((uint32_t)__cvta_generic_to_shared(&s_logit[buf][i]), P.score + at);
        }
    };
    if (nblk > 0) {
        fetch_counts(0);
        attn_cp_async_commit();
        attn_cp_async_wait<0>();
        __syncthreads();
        scan_counts(0);
        fetch_counts(1);
        __syncthreads();
        fetch_entries(0, 0, 0);
        attn_cp_async_commit();
        attn_cp_async_wait<0>();
        __syncthreads();
        int blk = 0, sub = 0, buf = 0;
        while (blk < nblk) {  // every test below is uniform over the CTA
            const int total = s_off[blk & 1][ATTN_TB];
            const int n = min(ATTN_LIST, total - sub * ATTN_LIST);
            int next_blk = blk, next_sub = sub + 1;
            if ((sub + 1) * ATTN_LIST >= total) {
                next_blk = blk + 1;
                next_sub = 0;
            }
            if (next_blk != blk && next_blk < nblk) {
                scan_counts(next_blk);       // its counts landed before the last barrier
                __syncthreads();
                fetch_counts(next_blk + 1);  // into the buffer of block `blk`, whose prefix sums exist
            }
            if (next_blk < nblk) fetch_entries(next_blk, next_sub, buf ^ 1);
            if (n > 0) {
                flush(s_idx[buf], s_logit[buf], n);
            } else {
                attn_cp_async_commit();
                attn_cp_async_wait<0>();
                __syncthreads();
            }
            blk = next_blk;
            sub = next_sub;
            buf ^= 1;
        }
    }

    // ---- queued (not yet indexed) keys: split 0 only ---------------------------
    if (split == 0 && P.n_queued > 0) {
        float qreg[NCH][8];
        load_vec_f32<NCH>(P.q + (size_t)qh * P.dim, qreg, lane, P.dim);
        const float scale = P.scaling ? P.scaling[qh] : 1.0f;
        const TK* qk = reinterpret_cast<const TK*>(P.queued_k) + (size_t)h * P.queued_head_stride;
        int j0 = 0;
        while (j0 < P.n_queued) {
            const int fill = 0;
            const int n = min(P.n_queued - j0, ATTN_LIST);
            for (int b = 0; b < n; b += ATTN_HW) {  // uniform trip count
                const int j = b + hw;
                Acc2 a2{0.f, 0.f};
                if (j < n) {
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const int c = lane + GROUP * i;
                        if (c * 8 < P.dim) {
                            float a[8];
                            to_float(load_chunk<TK>(qk + (size_t)(j0 + j) * P.dim, c), a);
                            chunk_fma(a2, a, qreg[i]);
                        }
                    }
                }
                const float d = group_sum(__fadd_rn(a2.e, a2.o));
                if (lane == 0 && j < n) {
                    s_idx[0][fill + j] = QUEUE_FLAG | (j0 + j);
                    s_logit[0][fill + j] = __fmul_rn(d, scale);
                }
            }
            flush(s_idx[0], s_logit[0], n);
            j0 += n;
        }
    }

    // ---- combine the groups ----------------------------------------------------
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NVCH; ++i) {
        const int c = lane + GROUP * i;
        if (c * 8 < P.vdim) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s_out[(size_t)hw * P.vdim + c * 8 + e] = acc[i][e];
        }
    }
    if (lane == 0) s_red[hw] = l;
    __syncthreads();
    if (P.n_splits == 1) {
        // the only partial of this head: what the merge would compute, written directly
        float L = 0.f;
        for (int w = 0; w < ATTN_HW; ++w) L += s_red[w];
        for (int d = tid; d < P.vdim; d += ATTN_THREADS) {
            float s = 0.f;
            for (int w = 0; w < ATTN_HW; ++w) s += s_out[(size_t)w * P.vdim + d];
            P.out[(size_t)qh * P.out_stride + d] = L > 0.f ? s / L : 0.f;
        }
        if (tid == 0 && P.out_ml) {
            P.out_ml[(size_t)qh * P.ml_stride] = m;
            P.out_ml[(size_t)qh * P.ml_stride + 1] = L;
        }
        return;
    }
    float* ws = P.ws + ((size_t)qh * P.n_splits + split) * (P.vdim + 2);
    for (int d = tid; d < P.vdim; d += ATTN_THREADS) {
        float s = 0.f;
        for (int w = 0; w < ATTN_HW; ++w) s += s_out[(size_t)w * P.vdim + d];
        ws[2 + d] = s;
    }
    if (tid == 0) {
        float s = 0.f;
        for (int w = 0; w < ATTN_HW; ++w) s += s_red[w];
        ws[0] = m;
        ws[1] = s;
    }
}

// out = sum_s w_s * o_s / sum_s w_s * (normalised ? 1 : l_s-free) ... see below.
// Partials are (m_s, l_s, o_s).  With unnormalised o_s (split-KV workspace):
//   out = sum_s e^{m_s-M} o_s / sum_s e^{m_s-M} l_s.
// With normalised o_s (sequence shards): o_s is first scaled back by l_s.
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             long long o_part_stride, long long o_head_stride,
                             long long ml_part_stride, long long ml_head_stride,
                             int n_parts, int vdim, int normalised, float* __restrict__ out,
                             float* __restrict__ out_ml, long long out_stride, long long out_ml_stride) {
    const int qh = blockIdx.x;
    merge_row(part_o + qh * o_head_stride, part_ml + qh * ml_head_stride, o_part_stride, ml_part_stride, n_parts, vdim,
              normalised, out + (size_t)qh * out_stride, out_ml ? out_ml + (size_t)qh * out_ml_stride : nullptr);
}

template <typename TK, typename TV, int NCH, int NVCH>
static int launch_attn_n(const AttnParams& P, cudaStream_t s) {
    auto kern = sparse_attn_kernel<TK, TV, NCH, NVCH>;
    dim3 grid((unsigned)P.n_splits, (unsigned)P.n_qheads);
    size_t smem = (size_t)ATTN_HW * P.vdim * sizeof(float);   // the final combine, in the ring's place
    if (smem < (size_t)GatherRing<TV, NVCH>::BYTES) smem = GatherRing<TV, NVCH>::BYTES;
    if (smem + 20 * 1024 > 48 * 1024) {   // static shared memory (lists, counts) comes on top
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("hira_sparse_attn: cudaFuncSetAttribute(%zu B smem): %s", smem, cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
    }
    kern<<<grid, ATTN_THREADS, smem, s>>>(P);
    HIRA_CHECK_LAUNCH("hira_sparse_attn launch");
    return HIRA_OK;
}

template <typename TK, typename TV>
static int launch_attn(const AttnParams& P, cudaStream_t s) {
    const bool k2 = P.dim > 128, v2 = P.vdim > 128;   // chunks per lane: 2 up to 128 elements, else 4
    if (!k2 && !v2) return launch_attn_n<TK, TV, 2, 2>(P, s);
    if (k2 && !v2) return launch_attn_n<TK, TV, 4, 2>(P, s);
    if (!k2 && v2) return launch_attn_n<TK, TV, 2, 4>(P, s);
    return launch_attn_n<TK, TV, 4, 4>(P, s);
}

}  // namespace hira

using namespace hira;

extern "C" int hira_attn_default_splits(int32_t n_qheads, int32_t n_tiles) {
    if (n_qheads < 1 || n_tiles < 1) return 1;
    // One wave of CTAs: five 128-thread CTAs fit per SM (96 registers), and a launch that is a
    // little over a whole number of waves pays for a nearly empty last one.  Measured: 64 query
    // heads 41 -> 34 us against the former 16 CTAs/SM target, 512 query heads unchanged.
    const int factor = 5;   // CTAs per SM aimed for
    int s = (factor * 148) / n_qheads;
    if (s > n_tiles) s = n_tiles;
    if (s > 64) s = 64;
    return s < 1 ? 1 : s;
}

extern "C" int hira_sparse_attn(const hira_index_t* ix, const float* q, const float* scaling,
                                const int32_t* q2kv, int32_t n_qheads, int32_t tile_parents,
                                const int32_t* idx, const float* score, const int32_t* count,
                                const void* queued_k, const void* queued_v, int32_t n_queued,
                                int64_t queued_head_stride, int32_t n_splits, float* workspace,
                                float* out, float* out_ml, int64_t out_head_stride, int64_t ml_head_stride,
                                void* stream) {
    int rc = validate_index(ix, true);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(idx && score && count && workspace && out, HIRA_ERR_ARG,
                   "hira_sparse_attn: idx, score, count, workspace and out must not be NULL");
    HIRA_CHECK_ARG(n_qheads >= 1 && n_splits >= 1, HIRA_ERR_SHAPE, "hira_sparse_attn: n_qheads=%d n_splits=%d",
                   n_qheads, n_splits);
    HIRA_CHECK_ARG(q2kv || n_qheads % ix->n_heads == 0, HIRA_ERR_SHAPE,
                   "hira_sparse_attn: n_qheads=%d not divisible by n_heads=%d and no q2kv given", n_qheads, ix->n_heads);
    HIRA_CHECK_ARG(tile_parents >= 1, HIRA_ERR_SHAPE, "hira_sparse_attn: tile_parents=%d", tile_parents);
    HIRA_CHECK_ARG(n_queued >= 0, HIRA_ERR_SHAPE, "hira_sparse_attn: n_queued=%d", n_queued);
    if (n_queued > 0) {
        HIRA_CHECK_ARG(q && queued_k && queued_v, HIRA_ERR_ARG,
                       "hira_sparse_attn: q, queued_k and queued_v are required when n_queued > 0");
        HIRA_CHECK_ARG(n_queued < QUEUE_FLAG, HIRA_ERR_SHAPE, "hira_sparse_attn: n_queued too large");
        // one head stride serves queued_k (rows of dim) and queued_v (rows of vdim)
        HIRA_CHECK_ARG(ix->dim == ix->vdim, HIRA_ERR_SHAPE,
                       "hira_sparse_attn: queued keys/values need dim == vdim (got %d and %d): the single "
                       "queued_head_stride applies to both arrays", ix->dim, ix->vdim);
    }
    AttnParams P;
    P.values = ix->values; P.q = q; P.scaling = scaling; P.q2kv = q2kv;
    P.idx = idx; P.score = score; P.count = count;
    P.queued_k = queued_k; P.queued_v = queued_v; P.ws = workspace;
    P.out = out; P.out_ml = out_ml;
    P.n_heads = ix->n_heads; P.n_qheads = n_qheads;
    P.group = q2kv ? 1 : n_qheads / ix->n_heads;
    P.dim = ix->dim; P.vdim = ix->vdim;
    P.n_tiles = (ix->cap_parents + tile_parents - 1) / tile_parents;
    P.n_tiles_active = active_tiles(ix, tile_parents);
    P.tile_rows = tile_parents * ix->bf;
    P.n_splits = n_splits; P.n_queued = n_queued;
    P.cap_children = (long long)ix->cap_parents * ix->bf;
    P.queued_head_stride = queued_head_stride;
    HIRA_CHECK_ARG((out_head_stride == 0 || out_head_stride >= ix->vdim) && (ml_head_stride == 0 || ml_head_stride >= 2),
                   HIRA_ERR_SHAPE, "hira_sparse_attn: out_head_stride=%lld / ml_head_stride=%lld too small",
                   (long long)out_head_stride, (long long)ml_head_stride);
    P.out_stride = out_head_stride ? out_head_stride : ix->vdim;
    P.ml_stride = ml_head_stride ? ml_head_stride : 2;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (ix->dtype == HIRA_BF16 && ix->vdtype == HIRA_BF16) rc = launch_attn<__nv_bfloat16, __nv_bfloat16>(P, s);
    else if (ix->dtype == HIRA_F32 && ix->vdtype == HIRA_F32) rc = launch_attn<float, float>(P, s);
    else if (ix->dtype == HIRA_F32 && ix->vdtype == HIRA_BF16) rc = launch_attn<float, __nv_bfloat16>(P, s);
    else rc = launch_attn<__nv_bfloat16, float>(P, s);
    if (rc != HIRA_OK) return rc;
    if (n_splits == 1) return HIRA_OK;  // the attention kernel wrote `out` itself
    const long long pstride = ix->vdim + 2;
    merge_kernel<<<n_qheads, 128, 0, s>>>(workspace + 2, workspace, pstride, pstride * n_splits, pstride,
                                          pstride * n_splits, n_splits, ix->vdim, 0, out, out_ml, P.out_stride,
                                          P.ml_stride);
    HIRA_CHECK_LAUNCH("hira_sparse_attn merge launch");
    return HIRA_OK;
}

extern "C" int hira_merge_partials(const float* part_o, const float* part_ml, int32_t n_parts,
                                   int32_t n_qheads, int32_t vdim, int64_t o_part_stride, int64_t o_head_stride,
                                   int64_t ml_part_stride, int64_t ml_head_stride, float* out, float* out_ml,
                                   void* stream) {
    HIRA_CHECK_ARG(part_o && part_ml && out, HIRA_ERR_ARG, "hira_merge_partials: NULL argument");
    HIRA_CHECK_ARG(n_parts >= 1 && n_qheads >= 1 && vdim >= 1, HIRA_ERR_SHAPE,
                   "hira_merge_partials: n_parts=%d n_qheads=%d vdim=%d", n_parts, n_qheads, vdim);
    if (o_head_stride == 0) o_head_stride = vdim;
    if (o_part_stride == 0) o_part_stride = (int64_t)n_qheads * o_head_stride;
    if (ml_head_stride == 0) ml_head_stride = 2;
    if (ml_part_stride == 0) ml_part_stride = (int64_t)n_qheads * ml_head_stride;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    merge_kernel<<<n_qheads, 128, 0, s>>>(part_o, part_ml, o_part_stride, o_head_stride, ml_part_stride,
                                          ml_head_stride, n_parts, vdim, 1, out, out_ml, vdim, 2);
    HIRA_CHECK_LAUNCH("hira_merge_partials launch");
    return HIRA_OK;
}

// ---------------------------------------------------------------------------
// Sparse attention for callers that must not allocate.
//
// Some hosts of this library cannot give hira_sparse_attn a workspace: a decode
// loop that has promised "no cudaMalloc after warm-up" (an allocation can stall
// every stream of the device), a plugin that only receives input and output
// buffers from its framework, or a C caller without any device allocator of its
// own.  For them the split-KV partials live in a fixed array inside the library
// image.  Every GPU that loads the library carries the array until the process
// exits, so it is kept modest: HIRA_NOALLOC_SCRATCH_FLOATS floats (4 MiB).
// ---------------------------------------------------------------------------
static __device__ __align__(256) float g_attn_scratch[HIRA_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
// device address of g_attn_scratch per device, null = not looked up yet.  Threads that race on
// the first call of a device all store the same address; the atomics make that race benign.
std::atomic<float*> g_scratch_ptr[kMaxDevices];

// In host code `g_attn_scratch` names a host-side shadow of the symbol, not device
// memory, so the address a kernel can use has to be asked for -- once per device,
// with that device current.
int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        hira::set_error("hira_sparse_attn_noalloc: cudaGetDevice failed or device index %d is out of range", dev);
        return HIRA_ERR_CUDA;
    }
    float* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_scratch);
        if (e != cudaSuccess || p == nullptr) {
            hira::set_error("hira_sparse_attn_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return HIRA_OK;
}
}  // namespace

extern "C" int hira_sparse_attn_noalloc(const hira_index_t* ix, const float* q, const float* scaling,
                                        const int32_t* q2kv, int32_t n_qheads, int32_t tile_parents,
                                        const int32_t* idx, const float* score, const int32_t* count,
                                        const void* queued_k, const void* queued_v, int32_t n_queued,
                                        int64_t queued_head_stride, int32_t n_splits, float* out, float* out_ml,
                                        int64_t out_head_stride, int64_t ml_head_stride, void* stream) {
    HIRA_CHECK_ARG(ix != nullptr, HIRA_ERR_ARG, "hira_sparse_attn_noalloc: index is NULL");
    HIRA_CHECK_ARG(n_qheads >= 1 && n_splits >= 1 && ix->vdim >= 1, HIRA_ERR_SHAPE,
                   "hira_sparse_attn_noalloc: n_qheads=%d n_splits=%d vdim=%d", n_qheads, n_splits, ix->vdim);
    const long long need = (long long)n_qheads * n_splits * (ix->vdim + 2);
    HIRA_CHECK_ARG(need <= (long long)HIRA_NOALLOC_SCRATCH_FLOATS, HIRA_ERR_CAPACITY,
                   "hira_sparse_attn_noalloc: n_qheads (%d) x n_splits (%d) x (vdim + 2) (%d) = %lld floats of "
                   "partials exceed the built-in scratch of %d floats; lower n_splits or call hira_sparse_attn "
                   "with a workspace of your own",
                   n_qheads, n_splits, ix->vdim + 2, need, (int)HIRA_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != HIRA_OK) return rc;
    // every (query head, split) slot of the scratch that the merge reads is written by the
    // attention kernel of this same call first, so nothing has to be cleared
    return hira_sparse_attn(ix, q, scaling, q2kv, n_qheads, tile_parents, idx, score, count, queued_k, queued_v,
                            n_queued, queued_head_stride, n_splits, scratch, out, out_ml, out_head_stride,
                            ml_head_stride, stream);
}
