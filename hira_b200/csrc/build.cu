// Index build: per head, per level, nearest-centroid assignment, capacity-bf
// grouping closest-first with overflow into free slots, blocked layout, radii.
//
// Follows CUDAIndexer.build (indexer/cuda.py:56-108):
//   _build_random_bf_level_batched (:200-336): K = ceil(n/bf) centres taken from
//     the points themselves, one nearest-centre assignment (cdist + argmin,
//     :244-245), each centre keeps its bf closest points in distance order
//     (:252-303), the overflow goes to the free slots (:309-334);
//   _build_parents_children_from_keys (:338-426) and
//   _build_grandparents_parents_children_from_keys (:428-538): blocked layout,
//     second level over the parent centres, child blocks move with their parent;
//   _compute_parent_radii_from_layout / _compute_grandparent_radii_from_layout
//     (:114-198).
// Differences by design: the (n, K) distance matrix is never materialised (the
// arg-min runs inside the contraction), the overflow fill is deterministic
// (ascending free slot <- overflow in (centre, distance) order) instead of a
// per-head randperm, optional Lloyd mean updates precede the final assignment,
// and counts/validity are written as explicit state.
#include "common.cuh"
#include <cub/cub.cuh>
#include <math_constants.h>

namespace hira {

int q8_refresh(const hira_index_t* ix, cudaStream_t s, long long parents_bound);
int launch_assign_tc(const void* points, long long p_head_stride, const void* cents, const float* csq,
                     int n_heads, int n, int k, int dim, int32_t* out_idx, float* out_d2, cudaStream_t s);
bool assign_tc_supported(int dtype, int n, int k, int dim);

// ---------------------------------------------------------------------------
// Sequential-chain helpers (the assignment's arithmetic: one fp32 FMA chain
// over d = 0..D-1 starting from 0).
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f(float v) { return v; }
template <> __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void sqnorm_seq_kernel(const T* __restrict__ rows, long long n_rows, int dim, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows) return;
    const T* r = rows + i * dim;
    float acc = 0.f;
    for (int d = 0; d < dim; ++d) {
        const float v = to_f(r[d]);
        acc = __fmaf_rn(v, v, acc);
    }
    out[i] = acc;
}

// ---------------------------------------------------------------------------
// CUDA-core assignment: 64 points x 64 centres per step, 4x4 per thread.
// ---------------------------------------------------------------------------
constexpr int AS_PTS = 64, AS_CTS = 64, AS_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(AS_THREADS)
assign_kernel(const T* __restrict__ points, long long p_head_stride, const T* __restrict__ cents,
              const float* __restrict__ csq, int n, int k, int dim, int32_t* __restrict__ out_idx,
              float* __restrict__ out_d2) {
    extern __shared__ __align__(16) float sm[];
    const int ld = dim + 1;
    float* xs = sm;                  // [AS_PTS][ld]
    float* cs = sm + AS_PTS * ld;    // [AS_CTS][ld]
    const int h = blockIdx.y;
    const int p0 = blockIdx.x * AS_PTS;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const T* P = points + (size_t)h * p_head_stride;
    const T* C = cents + (size_t)h * k * dim;
    const float* CS = csq + (size_t)h * k;

    for (int e = tid; e < AS_PTS * dim; e += AS_THREADS) {
        const int r = e / dim, d = e - r * dim;
        xs[r * ld + d] = (p0 + r < n) ? to_f(P[(size_t)(p0 + r) * dim + d]) : 0.f;
    }
    float best_s[4];
    int best_i[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { best_s[i] = CUDART_INF_F; best_i[i] = 0x7fffffff; }

    for (int c0 = 0; c0 < k; c0 += AS_CTS) {
        __syncthreads();
        for (int e = tid; e < AS_CTS * dim; e += AS_THREADS) {
            const int r = e / dim, d = e - r * dim;
            cs[r * ld + d] = (c0 + r < k) ? to_f(C[(size_t)(c0 + r) * dim + d]) : 0.f;
        }
        __syncthreads();
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int d = 0; d < dim; ++d) {
            float xv[4], cv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[(ty + 16 * i) * ld + d];
#pragma unroll
            for (int j = 0; j < 4; ++j) cv[j] = cs[(tx + 16 * j) * ld + d];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(xv[i], cv[j], acc[i][j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tx + 16 * j;
            if (c < k) {
                const float cq = CS[c];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float s = __fsub_rn(cq, __fmul_rn(2.0f, acc[i][j]));
                    if (s < best_s[i] || (s == best_s[i] && c < best_i[i])) { best_s[i] = s; best_i[i] = c; }
                }
            }
        }
    }
    __syncthreads();
    // reduce over the 16 threads (tx) that share a point; reuse cs
    float* rs = cs;                                   // [AS_PTS][16]
    int* ri = reinterpret_cast<int*>(cs + AS_PTS * 16);  // [AS_PTS][16]
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        rs[(ty + 16 * i) * 16 + tx] = best_s[i];
        ri[(ty + 16 * i) * 16 + tx] = best_i[i];
    }
    __syncthreads();
    if (tid < AS_PTS && p0 + tid < n) {
        float bs = rs[tid * 16];
        int bi = ri[tid * 16];
        for (int t = 1; t < 16; ++t) {
            const float s = rs[tid * 16 + t];
            const int c = ri[tid * 16 + t];
            if (s < bs || (s == bs && c < bi)) { bs = s; bi = c; }
        }
        float xsq = 0.f;
        for (int d = 0; d < dim; ++d) xsq = __fmaf_rn(xs[tid * ld + d], xs[tid * ld + d], xsq);
        out_idx[(size_t)h * n + p0 + tid] = bi;
        out_d2[(size_t)h * n + p0 + tid] = fmaxf(__fadd_rn(xsq, bs), 0.f);
    }
}

template <typename T>
static int launch_assign_cc(const T* points, long long p_head_stride, const T* cents, const float* csq,
                            int n_heads, int n, int k, int dim, int32_t* out_idx, float* out_d2, cudaStream_t s) {
    // points tile + the larger of (centre tile, the 2 x [AS_PTS][16] reduction arrays that reuse it)
    const size_t cs_floats = (size_t)AS_CTS * (dim + 1) > (size_t)2 * AS_PTS * 16 ? (size_t)AS_CTS * (dim + 1)
                                                                                  : (size_t)2 * AS_PTS * 16;
    const size_t smem = ((size_t)AS_PTS * (dim + 1) + cs_floats) * sizeof(float);
    auto kern = assign_kernel<T>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("assign: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return HIRA_ERR_CUDA; }
    }
    dim3 grid((unsigned)((n + AS_PTS - 1) / AS_PTS), (unsigned)n_heads);
    kern<<<grid, AS_THREADS, smem, s>>>(points, p_head_stride, cents, csq, n, k, dim, out_idx, out_d2);
    HIRA_CHECK_LAUNCH("assign launch");
    return HIRA_OK;
}

static int run_assign(int dtype, const void* points, long long p_head_stride, const void* cents, float* csq,
                      int n_heads, int n, int k, int dim, int use_tc, int32_t* out_idx, float* out_d2,
                      cudaStream_t s, bool csq_ready = false) {
    const long long rows = (long long)n_heads * k;
    const int blocks = (int)((rows + 255) / 256);
    if (!csq_ready) {
        if (dtype == HIRA_BF16)
            sqnorm_seq_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(cents), rows, dim, csq);
        else
            sqnorm_seq_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const float*>(cents), rows, dim, csq);
        HIRA_CHECK_LAUNCH("sqnorm launch");
    }
    if (use_tc && assign_tc_supported(dtype, n, k, dim))
        return launch_assign_tc(points, p_head_stride, cents, csq, n_heads, n, k, dim, out_idx, out_d2, s);
    if (dtype == HIRA_BF16)
        return launch_assign_cc(reinterpret_cast<const __nv_bfloat16*>(points), p_head_stride,
                                reinterpret_cast<const __nv_bfloat16*>(cents), csq, n_heads, n, k, dim, out_idx, out_d2, s);
    return launch_assign_cc(reinterpret_cast<const float*>(points), p_head_stride,
                            reinterpret_cast<const float*>(cents), csq, n_heads, n, k, dim, out_idx, out_d2, s);
}

// ---------------------------------------------------------------------------
// Level build pieces.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_centres_kernel(const T* __restrict__ points, long long p_head_stride, int n,
                                      const int32_t* __restrict__ cent_idx, int k, int dim, T* __restrict__ cents) {
    // one thread per (head, centre, 8-element chunk)
    const int chunks = dim / 8;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= (long long)k * chunks) return;
    const int c = (int)(t / chunks), ch = (int)(t % chunks);
    int src;
    if (cent_idx) {
        src = cent_idx[(size_t)h * k + c];
        src = src < 0 ? 0 : (src >= n ? n - 1 : src);
    } else {
        src = (int)(((long long)c * n) / k);  // evenly strided
    }
    const T* r = points + (size_t)h * p_head_stride + (size_t)src * dim + ch * 8;
    T* w = cents + ((size_t)h * k + c) * dim + ch * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = r[e];
}

// An assignment outside [0, k) -- the tensor-core kernel writes -1 for the points of a CTA whose
// bounded barrier wait ran out -- must not reach the segment arithmetic below: the point goes to
// centre 0 at distance 0 (so that every later index stays in range) and the caller is told through
// the status word.
// `placed` (balanced rounds): points that already have a slot sort behind every real segment.
__global__ void make_sort_keys_kernel(const int32_t* __restrict__ idx, const float* __restrict__ d2, int n, int k,
                                      long long total, long long n_seg, const int32_t* __restrict__ placed,
                                      uint64_t* __restrict__ keys, uint32_t* __restrict__ vals,
                                      int32_t* __restrict__ status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int h = (int)(i / n);
    if (placed && placed[i] >= 0) {
        keys[i] = (uint64_t)n_seg << 32;
        vals[i] = (uint32_t)(i - (long long)h * n);
        return;
    }
    int c = idx[i];
    float d = d2[i];
    if (c < 0 || c >= k || !(d >= 0.f)) {
        if (status) atomicOr(status, HIRA_STATUS_ASSIGN_FAILED);
        c = 0;
        d = 0.f;
    }
    const uint64_t seg = (uint64_t)h * k + (uint32_t)c;
    keys[i] = (seg << 32) | (uint64_t)__float_as_uint(d);  // d >= 0: bits order like values
    vals[i] = (uint32_t)(i - (long long)h * n);
}

// start[s] = first sorted position whose segment id >= s, for s in [0, n_seg]
__global__ void segment_starts_kernel(const uint64_t* __restrict__ keys, long long total, long long n_seg,
                                      int32_t* __restrict__ start) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i > total) return;
    long long cur = (i < total) ? (long long)(keys[i] >> 32) : n_seg;
    long long prev = (i == 0) ? -1 : (long long)(keys[i - 1] >> 32);
    cur = cur > n_seg ? n_seg : cur;     // `start` has n_seg + 1 entries
    prev = prev > n_seg ? n_seg : prev;
    for (long long s = prev + 1; s <= cur; ++s) start[s] = (int32_t)i;
}

// Lloyd mean update: one 8-lane group per centre, members added in sorted order
template <typename T, int NCH>
__global__ void means_kernel(const T* __restrict__ points, long long p_head_stride, int n,
                             const uint32_t* __restrict__ sorted_ids, const int32_t* __restrict__ start, int k,
                             int dim, long long n_seg, T* __restrict__ cents) {
    const int lane = threadIdx.x & (GROUP - 1);
    const long long seg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / GROUP;
    if (seg >= n_seg) return;
    const int h = (int)(seg / k);
    const int b = start[seg], e = start[seg + 1];
    if (e <= b) return;  // empty cluster keeps its centre
    float sum[NCH][8];
#pragma unroll
    for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[i][j] = 0.f;
    const T* P = points + (size_t)h * p_head_stride;
    for (int m = b; m < e; ++m) {
        const uint32_t id = sorted_ids[m];
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int c = lane + GROUP * i;
            if (c * 8 < dim) {
                float a[8];
                to_float(load_chunk<T>(P + (size_t)id * dim, c), a);
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[i][j] = __fadd_rn(sum[i][j], a[j]);
            }
        }
    }
    const float cnt = (float)(e - b);
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + GROUP * i;
        if (c * 8 < dim) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __fdiv_rn(sum[i][j], cnt);
            store_chunk(cents + (size_t)seg * dim, c, o);
        }
    }
}

// Balanced rounds: centres that are full drop out of the next assignment (score +inf).
__global__ void mask_full_centres_kernel(const float* __restrict__ csq, const int32_t* __restrict__ filled, int bf,
                                         long long n_seg, float* __restrict__ csq_masked) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_seg) return;
    csq_masked[c] = filled[c] < bf ? csq[c] : CUDART_INF_F;
}

// An intermediate balanced round: every centre accepts, closest first, as many of the points that
// chose it as it still has room for; the rest stay unplaced for the next round.
__global__ void accept_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ sorted_ids,
                              const int32_t* __restrict__ start, const int32_t* __restrict__ filled, int n, int k,
                              int bf, long long total, long long n_seg, int32_t* __restrict__ slot) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= total) return;
    const long long seg = (long long)(keys[j] >> 32);
    if (seg >= n_seg) return;   // placed earlier
    const int h = (int)(seg / k);
    const int c = (int)(seg - (long long)h * k);
    const int rank = (int)(j - start[seg]);
    const int have = filled[seg];
    if (rank < bf - have) slot[(size_t)h * n + sorted_ids[j]] = c * bf + have + rank;
}
__global__ void accept_counts_kernel(const int32_t* __restrict__ start, int bf, long long n_seg,
                                     int32_t* __restrict__ filled) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_seg) return;
    const int cnt = start[c + 1] - start[c], room = bf - filled[c];
    filled[c] += cnt < room ? cnt : room;
}

// per head: exclusive scans of free slots and overflow counts over the centres; `filled` = slots
// taken in earlier balanced rounds (all zero without them)
__global__ void __launch_bounds__(1024)
capacity_scan_kernel(const int32_t* __restrict__ start, const int32_t* __restrict__ filled, int k, int bf,
                     int32_t* __restrict__ free_base, int32_t* __restrict__ left_base, int32_t* __restrict__ fill_cnt) {
    typedef cub::BlockScan<int, 1024> Scan;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int s_total_left;
    const int h = blockIdx.x;
    const int32_t* st = start + (size_t)h * k;
    const int32_t* fl = filled + (size_t)h * k;
    int32_t* fb = free_base + (size_t)h * (k + 1);
    int32_t* lb = left_base + (size_t)h * (k + 1);
    int carry_f = 0, carry_l = 0;
    for (int c0 = 0; c0 < k; c0 += 1024) {
        const int c = c0 + threadIdx.x;
        int cnt = 0, room = 0;
        if (c < k) { cnt = st[c + 1] - st[c]; room = bf - fl[c]; }
        const int fr = (c < k) ? max(room - cnt, 0) : 0;
        const int lf = (c < k) ? max(cnt - room, 0) : 0;
        int ef, el, tf, tl;
        Scan(tmp).ExclusiveSum(fr, ef, tf);
        __syncthreads();
        Scan(tmp).ExclusiveSum(lf, el, tl);
        __syncthreads();
        if (c < k) { fb[c] = carry_f + ef; lb[c] = carry_l + el; }
        carry_f += tf; carry_l += tl;
    }
    if (threadIdx.x == 0) { fb[k] = carry_f; lb[k] = carry_l; s_total_left = carry_l; }
    __syncthreads();
    const int total_left = s_total_left;
    for (int c = threadIdx.x; c < k; c += 1024) {
        const int cnt = st[c + 1] - st[c], room = bf - fl[c];
        const int fr = max(room - cnt, 0);
        int recv = total_left - fb[c];
        recv = recv < 0 ? 0 : (recv > fr ? fr : recv);
        fill_cnt[(size_t)h * k + c] = fl[c] + min(cnt, room) + recv;
    }
}

// slot (centre*bf + rank) of every point inside its level (the last round: everything is placed)
__global__ void placement_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ sorted_ids,
                                 const int32_t* __restrict__ start, const int32_t* __restrict__ filled,
                                 const int32_t* __restrict__ free_base, const int32_t* __restrict__ left_base, int n,
                                 int k, int bf, long long total, long long n_seg, int32_t* __restrict__ slot) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= total) return;
    const long long seg = (long long)(keys[j] >> 32);
    if (seg >= n_seg) return;   // placed in an earlier balanced round
    const int h = (int)(seg / k);
    const int c = (int)(seg - (long long)h * k);
    const int rank = (int)(j - start[seg]);
    const int32_t* fl = filled + (size_t)h * k;
    const int room = bf - fl[c];
    int s;
    if (rank < room) {
        s = c * bf + fl[c] + rank;
    } else {
        const int32_t* fb = free_base + (size_t)h * (k + 1);
        const int32_t* st = start + (size_t)h * k;
        const int L = left_base[(size_t)h * (k + 1) + c] + (rank - room);
        // largest c2 with fb[c2] <= L and a free slot there: upper_bound(fb, L) - 1
        int lo = 0, hi = k;  // search in fb[0..k]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (fb[mid] <= L) lo = mid; else hi = mid - 1;
        }
        // skip centres without free slots (fb equal runs): lo is the last index with fb[lo] <= L,
        // which has fb[lo+1] > L, hence at least one free slot
        const int cnt2 = st[lo + 1] - st[lo];
        s = lo * bf + fl[lo] + min(cnt2, bf - fl[lo]) + (L - fb[lo]);
    }
    slot[(size_t)h * n + sorted_ids[j]] = s;
}

template <typename T>
__global__ void scatter_rows_kernel(const T* __restrict__ src, long long src_head_stride, int n, int dim,
                                    const int32_t* __restrict__ slot1, const int32_t* __restrict__ slot2, int k1,
                                    int bf, T* __restrict__ dst, long long dst_head_rows,
                                    int32_t* __restrict__ slot2token, int token_base) {
    // one thread per (head, point, chunk)
    const int chunks = dim / 8;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= (long long)n * chunks) return;
    const int i = (int)(t / chunks), ch = (int)(t % chunks);
    int s = slot1[(size_t)h * n + i];
    if (slot2) {
        const int c = s / bf, r = s - c * bf;
        s = slot2[(size_t)h * k1 + c] * bf + r;
    }
    const T* r8 = src + (size_t)h * src_head_stride + (size_t)i * dim + ch * 8;
    T* w8 = dst + ((size_t)h * dst_head_rows + s) * dim + ch * 8;
    if (sizeof(T) == 2) {
        *reinterpret_cast<uint4*>(w8) = *reinterpret_cast<const uint4*>(r8);
    } else {
        reinterpret_cast<float4*>(w8)[0] = reinterpret_cast<const float4*>(r8)[0];
        reinterpret_cast<float4*>(w8)[1] = reinterpret_cast<const float4*>(r8)[1];
    }
    if (slot2token && ch == 0) slot2token[(size_t)h * dst_head_rows + s] = token_base + i;
}

// parents (and their counts) into their final slots
template <typename T>
__global__ void scatter_parents_kernel(const T* __restrict__ cents1, const int32_t* __restrict__ fill1,
                                       const int32_t* __restrict__ slot2, int k1, int dim, T* __restrict__ parents,
                                       int32_t* __restrict__ child_counts, int cap_parents) {
    const int chunks = dim / 8;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= (long long)k1 * chunks) return;
    const int c = (int)(t / chunks), ch = (int)(t % chunks);
    const int s = slot2 ? slot2[(size_t)h * k1 + c] : c;
    const T* r8 = cents1 + ((size_t)h * k1 + c) * dim + ch * 8;
    T* w8 = parents + ((size_t)h * cap_parents + s) * dim + ch * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = r8[e];
    if (ch == 0) child_counts[(size_t)h * cap_parents + s] = fill1[(size_t)h * k1 + c];
}

template <typename T>
__global__ void scatter_gps_kernel(const T* __restrict__ cents2, const int32_t* __restrict__ fill2, int k2, int dim,
                                   T* __restrict__ gps, int32_t* __restrict__ gp_counts, int cap_gp) {
    const int chunks = dim / 8;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= (long long)k2 * chunks) return;
    const int g = (int)(t / chunks), ch = (int)(t % chunks);
    const T* r8 = cents2 + ((size_t)h * k2 + g) * dim + ch * 8;
    T* w8 = gps + ((size_t)h * cap_gp + g) * dim + ch * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = r8[e];
    if (ch == 0) gp_counts[(size_t)h * cap_gp + g] = fill2[(size_t)h * k2 + g];
}

__global__ void set_used_kernel(int32_t* used, int n_heads, int used_p, int used_g, int n_keys) {
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= n_heads) return;
    used[h * 4 + 0] = used_p; used[h * 4 + 1] = used_g; used[h * 4 + 2] = n_keys; used[h * 4 + 3] = 0;
}

// ---------------------------------------------------------------------------
// Radii from the layout.
// ---------------------------------------------------------------------------
template <typename T, int NCH>
__global__ void parent_radii_kernel(const hira_index_t ix) {
    const int lane = threadIdx.x & (GROUP - 1);
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / GROUP;  // (head, parent)
    if (w >= (long long)ix.n_heads * ix.cap_parents) return;
    const int h = (int)(w / ix.cap_parents), p = (int)(w % ix.cap_parents);
    const int bf = ix.bf, dim = ix.dim;
    bool valid;
    if (ix.depth == 3) {
        const int g = p / bf;
        valid = g < ix.used[h * 4 + 1] && (p - g * bf) < ix.gp_counts[(size_t)h * ix.cap_gp + g];
    } else {
        valid = p < ix.used[h * 4 + 0];
    }
    float r = 0.f, sq = 0.f;
    if (valid) {
        const T* par = reinterpret_cast<const T*>(ix.parents) + ((size_t)h * ix.cap_parents + p) * dim;
        const T* ch = reinterpret_cast<const T*>(ix.children) + ((size_t)h * ix.cap_parents + p) * bf * dim;
        int cnt = ix.child_counts[(size_t)h * ix.cap_parents + p];
        cnt = cnt > bf ? bf : cnt;
        float px[NCH][8];
        load_vec<T, NCH>(par, px, lane, dim);
        sq = reg_sqnorm<NCH>(px);
        for (int c = 0; c < cnt; ++c) {
            const float d2 = row_dist2_reg<T, NCH>(ch + (size_t)c * dim, px, lane, dim);
            r = fmaxf(r, __fsqrt_rn(d2));
        }
    }
    if (lane == 0) {
        ix.parent_radii[(size_t)h * ix.cap_parents + p] = r;
        if (ix.parent_sqnorm) ix.parent_sqnorm[(size_t)h * ix.cap_parents + p] = sq;
    }
}

template <typename T, int NCH>
__global__ void gp_radii_kernel(const hira_index_t ix) {
    const int lane = threadIdx.x & (GROUP - 1);
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / GROUP;  // (head, gp)
    if (w >= (long long)ix.n_heads * ix.cap_gp) return;
    const int h = (int)(w / ix.cap_gp), g = (int)(w % ix.cap_gp);
    const int bf = ix.bf, dim = ix.dim;
    const bool valid = g < ix.used[h * 4 + 1];
    float r = 0.f, sq = 0.f;
    if (valid) {
        const T* gp = reinterpret_cast<const T*>(ix.grand_parents) + ((size_t)h * ix.cap_gp + g) * dim;
        const T* par = reinterpret_cast<const T*>(ix.parents) + ((size_t)h * ix.cap_parents + (size_t)g * bf) * dim;
        const float* pr = ix.parent_radii + (size_t)h * ix.cap_parents + (size_t)g * bf;
        int cnt = ix.gp_counts[(size_t)h * ix.cap_gp + g];
        cnt = cnt > bf ? bf : cnt;
        float gx[NCH][8];
        load_vec<T, NCH>(gp, gx, lane, dim);
        sq = reg_sqnorm<NCH>(gx);
        for (int c = 0; c < cnt; ++c) {
            const float d2 = row_dist2_reg<T, NCH>(par + (size_t)c * dim, gx, lane, dim);
            r = fmaxf(r, __fadd_rn(__fsqrt_rn(d2), pr[c]));
        }
    }
    if (lane == 0) {
        ix.gp_radii[(size_t)h * ix.cap_gp + g] = r;
        if (ix.gp_sqnorm) ix.gp_sqnorm[(size_t)h * ix.cap_gp + g] = sq;
    }
}

template <typename T>
static int launch_radii(const hira_index_t* ix, cudaStream_t s) {
    const long long hw_p = (long long)ix->n_heads * ix->cap_parents;
    const int blocks_p = (int)((hw_p * GROUP + 255) / 256);
    if (ix->dim > 128) parent_radii_kernel<T, 4><<<blocks_p, 256, 0, s>>>(*ix);
    else parent_radii_kernel<T, 2><<<blocks_p, 256, 0, s>>>(*ix);
    HIRA_CHECK_LAUNCH("parent radii launch");
    if (ix->depth == 3) {
        const long long hw_g = (long long)ix->n_heads * ix->cap_gp;
        const int blocks_g = (int)((hw_g * GROUP + 255) / 256);
        if (ix->dim > 128) gp_radii_kernel<T, 4><<<blocks_g, 256, 0, s>>>(*ix);
        else gp_radii_kernel<T, 2><<<blocks_g, 256, 0, s>>>(*ix);
        HIRA_CHECK_LAUNCH("grandparent radii launch");
    }
    return HIRA_OK;
}

// ---------------------------------------------------------------------------
// Export (slot order -> token order).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void export_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ slot2token,
                                   long long head_rows, long long visit_rows, int dim, int token_base, int n_out,
                                   T* __restrict__ dst) {
    const int chunks = dim / 8;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= visit_rows * chunks) return;
    const long long s = t / chunks;
    const int ch = (int)(t % chunks);
    const int tok = slot2token[(size_t)h * head_rows + s];
    if (tok < 0) return;
    const int o = tok - token_base;
    if (o < 0 || o >= n_out) return;
    const T* r8 = src + ((size_t)h * head_rows + s) * dim + ch * 8;
    T* w8 = dst + ((size_t)h * n_out + o) * dim + ch * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) w8[e] = r8[e];
}

// ---------------------------------------------------------------------------
// Workspace carving.
// ---------------------------------------------------------------------------
struct BuildWs {
    size_t total = 0;
    size_t cents1, cents2, csq, csq_masked, filled, a_idx, a_d2, keys_in, keys_out, vals_in, vals_out, start, fill1,
        fill2, fbase, lbase, slot1, slot2, cub;
    size_t cub_bytes = 0;
};

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

static BuildWs carve(const hira_index_t* ix, int n_keys) {
    BuildWs w;
    const size_t H = ix->n_heads, n = n_keys, bf = ix->bf, D = ix->dim, es = elem_size(ix->dtype);
    const size_t k1 = (n + bf - 1) / bf, k2 = (k1 + bf - 1) / bf;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return o; };
    w.cents1 = take(H * k1 * D * es);
    w.cents2 = take(H * k2 * D * es);
    w.csq = take(H * k1 * 4);
    w.csq_masked = take(H * k1 * 4);
    w.filled = take(H * k1 * 4);
    w.a_idx = take(H * n * 4);
    w.a_d2 = take(H * n * 4);
    w.keys_in = take(H * n * 8);
    w.keys_out = take(H * n * 8);
    w.vals_in = take(H * n * 4);
    w.vals_out = take(H * n * 4);
    w.start = take((H * k1 + 2) * 4);
    w.fill1 = take(H * k1 * 4);
    w.fill2 = take(H * k2 * 4);
    w.fbase = take(H * (k1 + 1) * 4);
    w.lbase = take(H * (k1 + 1) * 4);
    w.slot1 = take(H * n * 4);
    w.slot2 = take(H * k1 * 4);
    size_t cub_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const uint64_t*)nullptr, (uint64_t*)nullptr,
                                    (const uint32_t*)nullptr, (uint32_t*)nullptr, (long long)(H * n));
    w.cub_bytes = cub_bytes;
    w.cub = take(cub_bytes);
    w.total = off;
    return w;
}

// One level: points -> K centres (in `cents`), per-point slot (centre*bf+rank)
// and per-centre filled count.
template <typename T>
static int build_level(int dtype, const T* points, long long p_head_stride, int n_heads, int n, int k, int bf,
                       int dim, const int32_t* cent_idx, int n_iters, int balance_rounds, int use_tc, T* cents, char* base,
                       const BuildWs& w, int32_t* slot, int32_t* fill, int32_t* status, cudaStream_t s) {
    const long long total = (long long)n_heads * n;
    const long long n_seg = (long long)n_heads * k;
    float* csq = reinterpret_cast<float*>(base + w.csq);
    int32_t* a_idx = reinterpret_cast<int32_t*>(base + w.a_idx);
    float* a_d2 = reinterpret_cast<float*>(base + w.a_d2);
    uint64_t* keys_in = reinterpret_cast<uint64_t*>(base + w.keys_in);
    uint64_t* keys_out = reinterpret_cast<uint64_t*>(base + w.keys_out);
    uint32_t* vals_in = reinterpret_cast<uint32_t*>(base + w.vals_in);
    uint32_t* vals_out = reinterpret_cast<uint32_t*>(base + w.vals_out);
    int32_t* start = reinterpret_cast<int32_t*>(base + w.start);
    int32_t* fbase = reinterpret_cast<int32_t*>(base + w.fbase);
    int32_t* lbase = reinterpret_cast<int32_t*>(base + w.lbase);
    const int chunks = dim / 8;
    {
        dim3 grid((unsigned)(((long long)k * chunks + 255) / 256), (unsigned)n_heads);
        gather_centres_kernel<T><<<grid, 256, 0, s>>>(points, p_head_stride, n, cent_idx, k, dim, cents);
        HIRA_CHECK_LAUNCH("gather centres launch");
    }
    int seg_bits = 1;
    while ((1ll << seg_bits) < n_seg) ++seg_bits;
    const int iters = n_iters < 1 ? 1 : n_iters;
    for (int it = 0; it < iters; ++it) {
        int rc = run_assign(dtype, points, p_head_stride, cents, csq, n_heads, n, k, dim, use_tc, a_idx, a_d2, s);
        if (rc != HIRA_OK) return rc;
        const int blocks = (int)((total + 255) / 256);
        make_sort_keys_kernel<<<blocks, 256, 0, s>>>(a_idx, a_d2, n, k, total, n_seg, nullptr, keys_in, vals_in, status);
        HIRA_CHECK_LAUNCH("sort keys launch");
        size_t cub_bytes = w.cub_bytes;
        cudaError_t e = cub::DeviceRadixSort::SortPairs(base + w.cub, cub_bytes, keys_in, keys_out, vals_in, vals_out,
                                                        total, 0, 32 + seg_bits, s);
        if (e != cudaSuccess) { set_error("radix sort: %s", cudaGetErrorString(e)); return HIRA_ERR_CUDA; }
        const int blocks1 = (int)((total + 1 + 255) / 256);
        segment_starts_kernel<<<blocks1, 256, 0, s>>>(keys_out, total, n_seg, start);
        HIRA_CHECK_LAUNCH("segment starts launch");
        if (it + 1 < iters) {
            const int mblocks = (int)((n_seg * GROUP + 255) / 256);
            if (dim > 128) means_kernel<T, 4><<<mblocks, 256, 0, s>>>(points, p_head_stride, n, vals_out, start, k, dim, n_seg, cents);
            else means_kernel<T, 2><<<mblocks, 256, 0, s>>>(points, p_head_stride, n, vals_out, start, k, dim, n_seg, cents);
            HIRA_CHECK_LAUNCH("means launch");
        }
    }
    // ---- capacity-aware rounds: points that did not fit under their nearest centre choose again
    // among the centres that still have room, closest first, `balance_rounds` times; what is left
    // after that (and everything beyond the bf closest when balance_rounds == 0, the reference's
    // rule, indexer/cuda.py:252-334) goes to the free slots in (centre, distance) order.
    int32_t* filled = reinterpret_cast<int32_t*>(base + w.filled);
    float* csq_masked = reinterpret_cast<float*>(base + w.csq_masked);
    cudaMemsetAsync(filled, 0, (size_t)n_seg * 4, s);
    const int blocks = (int)((total + 255) / 256);
    const int seg_blocks = (int)((n_seg + 255) / 256);
    if (balance_rounds > 0) cudaMemsetAsync(slot, 0xff, (size_t)total * 4, s);
    for (int r = 0; r < balance_rounds; ++r) {
        accept_kernel<<<blocks, 256, 0, s>>>(keys_out, vals_out, start, filled, n, k, bf, total, n_seg, slot);
        accept_counts_kernel<<<seg_blocks, 256, 0, s>>>(start, bf, n_seg, filled);
        mask_full_centres_kernel<<<seg_blocks, 256, 0, s>>>(csq, filled, bf, n_seg, csq_masked);
        HIRA_CHECK_LAUNCH("balanced round launch");
        int rc = run_assign(dtype, points, p_head_stride, cents, csq_masked, n_heads, n, k, dim, use_tc, a_idx, a_d2, s, true);
        if (rc != HIRA_OK) return rc;
        make_sort_keys_kernel<<<blocks, 256, 0, s>>>(a_idx, a_d2, n, k, total, n_seg, slot, keys_in, vals_in, status);
        HIRA_CHECK_LAUNCH("sort keys launch");
        size_t cub_bytes = w.cub_bytes;
        int bits = 1;
        while ((1ll << bits) <= n_seg) ++bits;   // the sentinel segment n_seg needs one more value
        cudaError_t e = cub::DeviceRadixSort::SortPairs(base + w.cub, cub_bytes, keys_in, keys_out, vals_in, vals_out,
                                                        total, 0, 32 + bits, s);
        if (e != cudaSuccess) { set_error("radix sort: %s", cudaGetErrorString(e)); return HIRA_ERR_CUDA; }
        segment_starts_kernel<<<(int)((total + 1 + 255) / 256), 256, 0, s>>>(keys_out, total, n_seg, start);
        HIRA_CHECK_LAUNCH("segment starts launch");
    }
    capacity_scan_kernel<<<n_heads, 1024, 0, s>>>(start, filled, k, bf, fbase, lbase, fill);
    HIRA_CHECK_LAUNCH("capacity scan launch");
    placement_kernel<<<blocks, 256, 0, s>>>(keys_out, vals_out, start, filled, fbase, lbase, n, k, bf, total, n_seg, slot);
    HIRA_CHECK_LAUNCH("placement launch");
    return HIRA_OK;
}

template <typename T>
static int build_impl(const hira_index_t* ix, const void* keys_v, const void* values, int n_keys,
                      long long k_head_stride, long long v_head_stride, int token_base, const int32_t* cent_idx1,
                      const int32_t* cent_idx2, int n_iters, int balance_rounds, int use_tc, char* base, const BuildWs& w,
                      int32_t* status, cudaStream_t s) {
    const T* keys = reinterpret_cast<const T*>(keys_v);
    const int H = ix->n_heads, bf = ix->bf, dim = ix->dim;
    const int k1 = (n_keys + bf - 1) / bf;
    const int k2 = (k1 + bf - 1) / bf;
    const size_t es = elem_size(ix->dtype);
    const size_t capP = ix->cap_parents, capC = capP * bf;
    // ---- clear the index -----------------------------------------------------
    // Everything, or -- when the host vouches through active_parents that no slot beyond that bound
    // was ever used -- the slots up to the larger of that bound and what this build fills.
    {
        size_t clearP = capP;
        if (ix->active_parents > 0) {
            const size_t fills = ix->depth == 3 ? (size_t)k2 * bf : (size_t)k1;
            clearP = (size_t)ix->active_parents > fills ? (size_t)ix->active_parents : fills;
            if (clearP > capP) clearP = capP;
        }
        const size_t clearC = clearP * bf, clearG = ix->depth == 3 ? (clearP + bf - 1) / bf : 0;
        auto clear = [&](void* ptr, int value, size_t row_bytes, size_t rows_cap, size_t rows_clear) {
            if (ptr) cudaMemset2DAsync(ptr, rows_cap * row_bytes, value, rows_clear * row_bytes, (size_t)H, s);
        };
        clear(ix->children, 0, dim * es, capC, clearC);
        clear(ix->values, 0, ix->values ? ix->vdim * elem_size(ix->vdtype) : 0, capC, clearC);
        clear(ix->slot2token, 0xff, 4, capC, clearC);
        clear(ix->parents, 0, dim * es, capP, clearP);
        clear(ix->parent_radii, 0, 4, capP, clearP);
        clear(ix->parent_sqnorm, 0, 4, capP, clearP);
        clear(ix->child_counts, 0, 4, capP, clearP);
        if (ix->depth == 3) {
            clear(ix->grand_parents, 0, dim * es, ix->cap_gp, clearG);
            clear(ix->gp_radii, 0, 4, ix->cap_gp, clearG);
            clear(ix->gp_sqnorm, 0, 4, ix->cap_gp, clearG);
            clear(ix->gp_counts, 0, 4, ix->cap_gp, clearG);
        }
    }
    HIRA_CHECK_LAUNCH("index clear");
    if (n_keys == 0) {
        set_used_kernel<<<(H + 127) / 128, 128, 0, s>>>(ix->used, H, 0, 0, 0);
        HIRA_CHECK_LAUNCH("set used launch");
        return HIRA_OK;
    }
    T* cents1 = reinterpret_cast<T*>(base + w.cents1);
    T* cents2 = reinterpret_cast<T*>(base + w.cents2);
    int32_t* slot1 = reinterpret_cast<int32_t*>(base + w.slot1);
    int32_t* slot2 = reinterpret_cast<int32_t*>(base + w.slot2);
    int32_t* fill1 = reinterpret_cast<int32_t*>(base + w.fill1);
    int32_t* fill2 = reinterpret_cast<int32_t*>(base + w.fill2);
    int rc = build_level<T>(ix->dtype, keys, k_head_stride, H, n_keys, k1, bf, dim, cent_idx1, n_iters, balance_rounds, use_tc,
                            cents1, base, w, slot1, fill1, status, s);
    if (rc != HIRA_OK) return rc;
    const int32_t* slot2_used = nullptr;
    if (ix->depth == 3) {
        rc = build_level<T>(ix->dtype, cents1, (long long)k1 * dim, H, k1, k2, bf, dim, cent_idx2, n_iters, balance_rounds, use_tc,
                            cents2, base, w, slot2, fill2, status, s);
        if (rc != HIRA_OK) return rc;
        slot2_used = slot2;
        const int chunks = dim / 8;
        dim3 grid((unsigned)(((long long)k2 * chunks + 255) / 256), (unsigned)H);
        scatter_gps_kernel<T><<<grid, 256, 0, s>>>(cents2, fill2, k2, dim, reinterpret_cast<T*>(ix->grand_parents),
                                                   ix->gp_counts, ix->cap_gp);
        HIRA_CHECK_LAUNCH("scatter gps launch");
    }
    {
        const int chunks = dim / 8;
        dim3 grid((unsigned)(((long long)k1 * chunks + 255) / 256), (unsigned)H);
        scatter_parents_kernel<T><<<grid, 256, 0, s>>>(cents1, fill1, slot2_used, k1, dim,
                                                       reinterpret_cast<T*>(ix->parents), ix->child_counts,
                                                       ix->cap_parents);
        HIRA_CHECK_LAUNCH("scatter parents launch");
        dim3 gridc((unsigned)(((long long)n_keys * chunks + 255) / 256), (unsigned)H);
        scatter_rows_kernel<T><<<gridc, 256, 0, s>>>(keys, k_head_stride, n_keys, dim, slot1, slot2_used, k1, bf,
                                                     reinterpret_cast<T*>(ix->children), (long long)capC,
                                                     ix->slot2token, token_base);
        HIRA_CHECK_LAUNCH("scatter children launch");
    }
    if (ix->values) {
        const int vchunks = ix->vdim / 8;
        dim3 gridv((unsigned)(((long long)n_keys * vchunks + 255) / 256), (unsigned)H);
        if (ix->vdtype == HIRA_BF16)
            scatter_rows_kernel<__nv_bfloat16><<<gridv, 256, 0, s>>>(
                reinterpret_cast<const __nv_bfloat16*>(values), v_head_stride, n_keys, ix->vdim, slot1, slot2_used, k1,
                bf, reinterpret_cast<__nv_bfloat16*>(ix->values), (long long)capC, nullptr, 0);
        else
            scatter_rows_kernel<float><<<gridv, 256, 0, s>>>(reinterpret_cast<const float*>(values), v_head_stride,
                                                             n_keys, ix->vdim, slot1, slot2_used, k1, bf,
                                                             reinterpret_cast<float*>(ix->values), (long long)capC,
                                                             nullptr, 0);
        HIRA_CHECK_LAUNCH("scatter values launch");
    }
    set_used_kernel<<<(H + 127) / 128, 128, 0, s>>>(ix->used, H, ix->depth == 3 ? k2 * bf : k1,
                                                     ix->depth == 3 ? k2 : 0, n_keys);
    HIRA_CHECK_LAUNCH("set used launch");
    rc = launch_radii<T>(ix, s);
    if (rc != HIRA_OK) return rc;
    // the int8 side copy of the children, when the index carries one: over the slots this build filled
    return q8_refresh(ix, s, ix->depth == 3 ? (long long)k2 * bf : (long long)k1);
}

}  // namespace hira

using namespace hira;

extern "C" size_t hira_build_workspace_bytes(const hira_index_t* ix, int32_t n_keys) {
    if (validate_index(ix, false) != HIRA_OK || n_keys < 0) return 0;
    return carve(ix, n_keys > 0 ? n_keys : 1).total;
}

extern "C" int hira_build(const hira_index_t* ix, const void* keys, const void* values, int32_t n_keys,
                          int64_t k_head_stride, int64_t v_head_stride, int32_t token_base,
                          const int32_t* cent_idx1, const int32_t* cent_idx2, int32_t n_iters,
                          int32_t balance_rounds, int32_t use_tensor_cores, int32_t* status, void* workspace,
                          size_t workspace_bytes, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(n_keys >= 0, HIRA_ERR_SHAPE, "hira_build: n_keys=%d", n_keys);
    HIRA_CHECK_ARG(balance_rounds >= 0 && balance_rounds <= 64, HIRA_ERR_ARG, "hira_build: balance_rounds=%d", balance_rounds);
    HIRA_CHECK_ARG(n_keys == 0 || keys, HIRA_ERR_ARG, "hira_build: keys is NULL");
    HIRA_CHECK_ARG((ix->values == nullptr) == (values == nullptr) || n_keys == 0, HIRA_ERR_ARG,
                   "hira_build: values must be given iff the index stores values");
    const long long bf = ix->bf;
    const long long k1 = (n_keys + bf - 1) / bf, k2 = (k1 + bf - 1) / bf;
    if (ix->depth == 3)
        HIRA_CHECK_ARG(k2 <= ix->cap_gp, HIRA_ERR_CAPACITY, "hira_build: %d keys need %lld grandparents, capacity %d",
                       n_keys, k2, ix->cap_gp);
    else
        HIRA_CHECK_ARG(k1 <= ix->cap_parents, HIRA_ERR_CAPACITY, "hira_build: %d keys need %lld parents, capacity %d",
                       n_keys, k1, ix->cap_parents);
    const BuildWs w = carve(ix, n_keys > 0 ? n_keys : 1);
    HIRA_CHECK_ARG(n_keys == 0 || (workspace && workspace_bytes >= w.total), HIRA_ERR_CAPACITY,
                   "hira_build: workspace of %zu bytes given, %zu needed", workspace_bytes, w.total);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    char* base = reinterpret_cast<char*>(workspace);
    if (ix->dtype == HIRA_BF16)
        return build_impl<__nv_bfloat16>(ix, keys, values, n_keys, k_head_stride, v_head_stride, token_base, cent_idx1,
                                         cent_idx2, n_iters, balance_rounds, use_tensor_cores, base, w, status, s);
    return build_impl<float>(ix, keys, values, n_keys, k_head_stride, v_head_stride, token_base, cent_idx1, cent_idx2,
                             n_iters, balance_rounds, use_tensor_cores, base, w, status, s);
}

extern "C" int hira_recompute_radii(const hira_index_t* ix, void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    return ix->dtype == HIRA_BF16 ? launch_radii<__nv_bfloat16>(ix, s) : launch_radii<float>(ix, s);
}

extern "C" int hira_export(const hira_index_t* ix, int32_t token_base, int32_t n_out, void* out_k, void* out_v,
                           void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(ix->slot2token, HIRA_ERR_ARG, "hira_export: the index has no slot2token map");
    HIRA_CHECK_ARG(out_k && n_out >= 1, HIRA_ERR_ARG, "hira_export: out_k is NULL or n_out < 1");
    HIRA_CHECK_ARG(!out_v || ix->values, HIRA_ERR_ARG, "hira_export: out_v given but the index stores no values");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long rows = (long long)ix->cap_parents * ix->bf;
    // only the slots that can hold keys are visited (the host's bound, hira_index_t::active_parents)
    const long long visit = (ix->active_parents > 0 ? (long long)ix->active_parents : (long long)ix->cap_parents) * ix->bf;
    {
        const int chunks = ix->dim / 8;
        dim3 grid((unsigned)((visit * chunks + 255) / 256), (unsigned)ix->n_heads);
        if (ix->dtype == HIRA_BF16)
            export_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(ix->children),
                                                                   ix->slot2token, rows, visit, ix->dim, token_base, n_out,
                                                                   reinterpret_cast<__nv_bfloat16*>(out_k));
        else
            export_rows_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<const float*>(ix->children), ix->slot2token,
                                                           rows, visit, ix->dim, token_base, n_out,
                                                           reinterpret_cast<float*>(out_k));
        HIRA_CHECK_LAUNCH("export keys launch");
    }
    if (out_v) {
        const int chunks = ix->vdim / 8;
        dim3 grid((unsigned)((visit * chunks + 255) / 256), (unsigned)ix->n_heads);
        if (ix->vdtype == HIRA_BF16)
            export_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(ix->values),
                                                                   ix->slot2token, rows, visit, ix->vdim, token_base, n_out,
                                                                   reinterpret_cast<__nv_bfloat16*>(out_v));
        else
            export_rows_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<const float*>(ix->values), ix->slot2token,
                                                           rows, visit, ix->vdim, token_base, n_out,
                                                           reinterpret_cast<float*>(out_v));
        HIRA_CHECK_LAUNCH("export values launch");
    }
    return HIRA_OK;
}

extern "C" int hira_assign(const void* points, const void* cents, int32_t dtype, int32_t n_heads, int32_t n,
                           int32_t k, int32_t dim, int32_t use_tensor_cores, float* csq_scratch, int32_t* out_idx,
                           float* out_dist2, void* stream) {
    HIRA_CHECK_ARG(points && cents && csq_scratch && out_idx && out_dist2, HIRA_ERR_ARG, "hira_assign: NULL argument");
    HIRA_CHECK_ARG(dtype == HIRA_F32 || dtype == HIRA_BF16, HIRA_ERR_DTYPE, "hira_assign: dtype %d", dtype);
    HIRA_CHECK_ARG(n_heads >= 1 && n >= 1 && k >= 1, HIRA_ERR_SHAPE, "hira_assign: n_heads=%d n=%d k=%d", n_heads, n, k);
    HIRA_CHECK_ARG(dim >= 8 && dim <= 256 && dim % 8 == 0, HIRA_ERR_SHAPE, "hira_assign: dim=%d", dim);
    return run_assign(dtype, points, (long long)n * dim, cents, csq_scratch, n_heads, n, k, dim, use_tensor_cores,
                      out_idx, out_dist2, reinterpret_cast<cudaStream_t>(stream));
}
