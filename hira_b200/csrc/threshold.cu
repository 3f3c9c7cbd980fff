// Threshold (tau) finders, on device.
//
// The reference declares sample_max(samples, query) and
// sample_mean_topk(samples, query, k) (cache/threshold_finder.py:1-14, selected
// by HiraConfig.threshold_method / sample_size, cache/hira_config.py:22-23) but
// both raise NotImplementedError; the meaning implemented here is the one the
// names state: score a sample of keys against the query, then take the maximum
// or the mean of the k largest scores.  hira_kth_score gives the exact k-th
// largest score over a whole head (used to set tau so that a given number of
// keys survives).
#include "common.cuh"
#include <math_constants.h>

namespace hira {

constexpr int TAU_THREADS = 256;
constexpr int TAU_HW = TAU_THREADS / GROUP;
constexpr int TAU_MAX_SAMPLES = 4096;

template <typename T, int NCH>
__global__ void __launch_bounds__(TAU_THREADS)
threshold_kernel(const T* __restrict__ samples, long long head_stride, int n_samples, int dim,
                 const float* __restrict__ q, const int32_t* __restrict__ q2kv, int group, int method, int k,
                 float* __restrict__ tau_out) {
    __shared__ float s[TAU_MAX_SAMPLES];
    const int tid = threadIdx.x, lane = tid & (GROUP - 1), hw = tid / GROUP;
    const int qh = blockIdx.x;
    const int h = q2kv ? q2kv[qh] : qh / group;
    const T* rows = samples + (size_t)h * head_stride;
    float qreg[NCH][8];
    load_vec_f32<NCH>(q + (size_t)qh * dim, qreg, lane, dim);
    int n2 = 1;
    while (n2 < n_samples) n2 <<= 1;
    for (int b = 0; b < n2; b += TAU_HW) {  // uniform trip count
        const int i = b + hw;
        Acc2 acc{0.f, 0.f};
        if (i < n_samples) {
#pragma unroll
            for (int ci = 0; ci < NCH; ++ci) {
                const int c = lane + GROUP * ci;
                if (c * 8 < dim) {
                    float a[8];
                    to_float(load_chunk<T>(rows + (size_t)i * dim, c), a);
                    chunk_fma(acc, a, qreg[ci]);
                }
            }
        }
        const float r = group_sum(__fadd_rn(acc.e, acc.o));
        const float d = (i < n_samples) ? r : -CUDART_INF_F;  // padding sorts last
        if (lane == 0 && i < n2) s[i] = d;
    }
    __syncthreads();
    // bitonic sort, descending
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n2; i += TAU_THREADS) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const float a = s[i], b = s[j];
                    if (desc ? (a < b) : (a > b)) { s[i] = b; s[j] = a; }
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        float t;
        if (method == HIRA_TAU_SAMPLE_MAX) {
            t = s[0];
        } else if (method == HIRA_TAU_SAMPLE_KTH) {
            t = s[k - 1];
        } else {
            float sum = 0.f;
            for (int i = 0; i < k; ++i) sum = __fadd_rn(sum, s[i]);
            t = __fdiv_rn(sum, (float)k);
        }
        tau_out[qh] = t;
    }
}

// radix select, 8 bits per pass, over the compacted scores of one query head
__global__ void __launch_bounds__(1024)
kth_kernel(const float* __restrict__ score, const int32_t* __restrict__ count, long long cap_children,
           int n_tiles, int n_tiles_active, int tile_rows, const int32_t* __restrict__ kk,
           float* __restrict__ tau_out) {
    __shared__ unsigned int hist[256];
    __shared__ unsigned int s_prefix, s_remaining;
    const int qh = blockIdx.x;
    const int tid = threadIdx.x;
    const float* sc = score + (size_t)qh * cap_children;
    const int32_t* cnt = count + (size_t)qh * n_tiles;
    uint32_t prefix = 0, prefix_mask = 0;
    uint32_t remaining = (uint32_t)kk[qh];
    bool fail = kk[qh] < 1;
    for (int pass = 0; pass < 4 && !fail; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int t = 0; t < n_tiles_active; ++t) {
            const int c = cnt[t];
            for (int i = tid; i < c; i += blockDim.x) {
                const uint32_t key = order_key(sc[(size_t)t * tile_rows + i]);
                if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
            }
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t acc = 0;
            int d = 255;
            for (; d >= 0; --d) {
                if (acc + hist[d] >= remaining) break;
                acc += hist[d];
            }
            if (d < 0) {
                s_prefix = 0xffffffffu; s_remaining = 0;  // fewer than k scores
            } else {
                s_prefix = (uint32_t)d; s_remaining = remaining - acc;
            }
        }
        __syncthreads();
        if (s_remaining == 0) { fail = true; }
        else {
            prefix |= s_prefix << shift;
            prefix_mask |= 0xffu << shift;
            remaining = s_remaining;
        }
        __syncthreads();
    }
    if (tid == 0) tau_out[qh] = fail ? -CUDART_INF_F : key_to_float(prefix);
}

// q_hat = q / ||q|| (fp32) and the per-head logit scale ||q|| * softmax_scale: the unit query
// and `scaling` the reference's searchers expect (searcher/cpu.py:58-63), in one launch.
template <typename T>
__global__ void __launch_bounds__(128)
prepare_query_kernel(const T* __restrict__ q, int dim, float sm_scale, float* __restrict__ q_hat,
                     float* __restrict__ logit_scale) {
    __shared__ float s_part[4];
    const int qh = blockIdx.x, tid = threadIdx.x;
    const T* row = q + (size_t)qh * dim;
    float acc = 0.f;
    for (int d = tid; d < dim; d += 128) {
        const float v = (float)row[d];
        acc = __fmaf_rn(v, v, acc);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((tid & 31) == 0) s_part[tid >> 5] = acc;
    __syncthreads();
    const float nrm = fmaxf(__fsqrt_rn(s_part[0] + s_part[1] + s_part[2] + s_part[3]), 1e-20f);
    for (int d = tid; d < dim; d += 128) q_hat[(size_t)qh * dim + d] = __fdiv_rn((float)row[d], nrm);
    if (tid == 0) logit_scale[qh] = nrm * sm_scale;
}

}  // namespace hira

using namespace hira;

extern "C" int hira_prepare_query(const void* q, int32_t dtype, int32_t n_qheads, int32_t dim, float sm_scale,
                                  float* q_hat, float* logit_scale, void* stream) {
    HIRA_CHECK_ARG(q && q_hat && logit_scale, HIRA_ERR_ARG, "hira_prepare_query: NULL argument");
    HIRA_CHECK_ARG(dtype == HIRA_F32 || dtype == HIRA_BF16, HIRA_ERR_DTYPE, "hira_prepare_query: dtype %d", dtype);
    HIRA_CHECK_ARG(n_qheads >= 1 && dim >= 1, HIRA_ERR_SHAPE, "hira_prepare_query: n_qheads=%d dim=%d", n_qheads, dim);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == HIRA_BF16)
        prepare_query_kernel<<<n_qheads, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(q), dim, sm_scale, q_hat, logit_scale);
    else
        prepare_query_kernel<<<n_qheads, 128, 0, s>>>(reinterpret_cast<const float*>(q), dim, sm_scale, q_hat, logit_scale);
    HIRA_CHECK_LAUNCH("hira_prepare_query launch");
    return HIRA_OK;
}


extern "C" int hira_threshold(const void* samples, int32_t dtype, int32_t n_heads, int32_t n_samples,
                              int32_t dim, int64_t head_stride, const float* q, const int32_t* q2kv,
                              int32_t n_qheads, int32_t method, int32_t k, float* tau_out, void* stream) {
    HIRA_CHECK_ARG(samples && q && tau_out, HIRA_ERR_ARG, "hira_threshold: NULL argument");
    HIRA_CHECK_ARG(dtype == HIRA_F32 || dtype == HIRA_BF16, HIRA_ERR_DTYPE, "hira_threshold: dtype %d", dtype);
    HIRA_CHECK_ARG(n_samples >= 1 && n_samples <= TAU_MAX_SAMPLES, HIRA_ERR_CAPACITY,
                   "hira_threshold: n_samples=%d outside 1..%d", n_samples, TAU_MAX_SAMPLES);
    HIRA_CHECK_ARG(dim >= 8 && dim <= 256 && dim % 8 == 0, HIRA_ERR_SHAPE, "hira_threshold: dim=%d", dim);
    HIRA_CHECK_ARG(n_heads >= 1 && n_qheads >= 1 && (q2kv || n_qheads % n_heads == 0), HIRA_ERR_SHAPE,
                   "hira_threshold: n_heads=%d n_qheads=%d", n_heads, n_qheads);
    HIRA_CHECK_ARG(method >= 0 && method <= 2, HIRA_ERR_ARG, "hira_threshold: unknown method %d", method);
    HIRA_CHECK_ARG(method == HIRA_TAU_SAMPLE_MAX || (k >= 1 && k <= n_samples), HIRA_ERR_ARG,
                   "hira_threshold: k=%d outside 1..n_samples=%d", k, n_samples);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int group = q2kv ? 1 : n_qheads / n_heads;
    const bool wide = dim > 128;  // chunks per lane: 2 up to 128 elements, else 4
    if (dtype == HIRA_BF16) {
        auto* p = reinterpret_cast<const __nv_bfloat16*>(samples);
        if (wide) threshold_kernel<__nv_bfloat16, 4><<<n_qheads, TAU_THREADS, 0, s>>>(p, head_stride, n_samples, dim, q, q2kv, group, method, k, tau_out);
        else threshold_kernel<__nv_bfloat16, 2><<<n_qheads, TAU_THREADS, 0, s>>>(p, head_stride, n_samples, dim, q, q2kv, group, method, k, tau_out);
    } else {
        auto* p = reinterpret_cast<const float*>(samples);
        if (wide) threshold_kernel<float, 4><<<n_qheads, TAU_THREADS, 0, s>>>(p, head_stride, n_samples, dim, q, q2kv, group, method, k, tau_out);
        else threshold_kernel<float, 2><<<n_qheads, TAU_THREADS, 0, s>>>(p, head_stride, n_samples, dim, q, q2kv, group, method, k, tau_out);
    }
    HIRA_CHECK_LAUNCH("hira_threshold launch");
    return HIRA_OK;
}

extern "C" int hira_kth_score(const hira_index_t* ix, int32_t n_qheads, int32_t tile_parents,
                              const float* score, const int32_t* count, const int32_t* k, float* tau_out,
                              void* stream) {
    int rc = validate_index(ix, false);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(score && count && k && tau_out, HIRA_ERR_ARG, "hira_kth_score: NULL argument");
    HIRA_CHECK_ARG(n_qheads >= 1 && tile_parents >= 1, HIRA_ERR_SHAPE, "hira_kth_score: n_qheads=%d tile_parents=%d",
                   n_qheads, tile_parents);
    const int n_tiles = (ix->cap_parents + tile_parents - 1) / tile_parents;
    kth_kernel<<<n_qheads, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        score, count, (long long)ix->cap_parents * ix->bf, n_tiles, active_tiles(ix, tile_parents), tile_parents * ix->bf, k,
        tau_out);
    HIRA_CHECK_LAUNCH("hira_kth_score launch");
    return HIRA_OK;
}
