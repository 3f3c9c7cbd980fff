// Shared device helpers for libhira_b200: error plumbing, row loads and the
// canonical fp32 dot product that defines the library's bit-exact results.
//
// Canonical dot product of two D-vectors (D a multiple of 8, D <= 256),
// evaluated by a group of 8 lanes (a quarter of a warp):
//   lane l owns the 8-element chunks c with c % 8 == l  (elements 8c .. 8c+7);
//   inside a lane two accumulators run over its chunks in increasing order:
//     e = fma(a[8c+2j],   b[8c+2j],   e)      j = 0..3   (even elements)
//     o = fma(a[8c+2j+1], b[8c+2j+1], o)                 (odd elements)
//   the lane partial is p_l = e + o (lanes owning no chunk contribute +0);
//   the 8 partials are summed by a butterfly: for s in 4,2,1: p_l += p_{l^s}.
// All adds are IEEE fp32 round-to-nearest; the butterfly is symmetric, so every
// lane ends with the same bits.  The CPU oracle evaluates the identical tree,
// which is what makes selected-key sets bit-exact at the threshold boundary.
// Eight lanes per row keep the shuffle count per row low (the search kernel is
// close to instruction-issue bound) while every 16-byte load still sits in a
// fully used 128-byte line: lanes 0..7 read bytes [0,128) of a bf16 row with
// their first chunk and [128,256) with their second.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hira_b200.h"

namespace hira {

void set_error(const char* fmt, ...);

#define HIRA_CHECK_ARG(cond, code, ...)      \
    do {                                     \
        if (!(cond)) {                       \
            ::hira::set_error(__VA_ARGS__);  \
            return (code);                   \
        }                                    \
    } while (0)

#define HIRA_CHECK_LAUNCH(what)                                               \
    do {                                                                      \
        cudaError_t e__ = cudaGetLastError();                                 \
        if (e__ != cudaSuccess) {                                             \
            ::hira::set_error("%s: %s", (what), cudaGetErrorString(e__));     \
            return HIRA_ERR_CUDA;                                             \
        }                                                                     \
    } while (0)

int validate_index(const hira_index_t* ix, bool need_values);
// tiles of `tile_parents` parent slots that can hold keys (hira_index_t::active_parents)
int active_tiles(const hira_index_t* ix, int tile_parents);

// order-preserving map float -> uint32 (a < b  <=>  order_key(a) < order_key(b), -0 before +0) and back
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
    const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}


// chunks (of 8 elements) each of the 8 lanes owns: 1 for D <= 64, 2 for D <= 128, 4 for D <= 256
__host__ __device__ inline int chunks_per_lane(int dim) { return dim <= 64 ? 1 : (dim <= 128 ? 2 : 4); }

__host__ __device__ inline size_t elem_size(int dtype) { return dtype == HIRA_BF16 ? 2 : 4; }

// ---------------------------------------------------------------------------
// Loads of one 8-element chunk of a row into fp32 registers.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void unpack_bf16x8(const uint4& r, float (&f)[8]) {
    f[0] = __uint_as_float(r.x << 16);
    f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16);
    f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16);
    f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16);
    f[7] = __uint_as_float(r.w & 0xffff0000u);
}

// Raw chunk as it sits in memory: 16 B for bf16, 32 B for fp32.
template <typename T> struct RawChunk;
template <> struct RawChunk<__nv_bfloat16> { uint4 a; };
template <> struct RawChunk<float> { float4 a, b; };

// streaming (read-once) load of chunk c of the row at `row`
template <typename T>
__device__ __forceinline__ RawChunk<T> load_chunk_stream(const T* row, int c);
template <>
__device__ __forceinline__ RawChunk<__nv_bfloat16> load_chunk_stream(const __nv_bfloat16* row, int c) {
    RawChunk<__nv_bfloat16> r;
    r.a = __ldcs(reinterpret_cast<const uint4*>(row) + c);
    return r;
}
template <>
__device__ __forceinline__ RawChunk<float> load_chunk_stream(const float* row, int c) {
    RawChunk<float> r;
    const float4* p = reinterpret_cast<const float4*>(row) + 2 * c;
    r.a = __ldcs(p);
    r.b = __ldcs(p + 1);
    return r;
}
// cached load (rows that other CTAs re-read: centres, queries)
template <typename T>
__device__ __forceinline__ RawChunk<T> load_chunk(const T* row, int c);
template <>
__device__ __forceinline__ RawChunk<__nv_bfloat16> load_chunk(const __nv_bfloat16* row, int c) {
    RawChunk<__nv_bfloat16> r;
    r.a = __ldg(reinterpret_cast<const uint4*>(row) + c);
    return r;
}
template <>
__device__ __forceinline__ RawChunk<float> load_chunk(const float* row, int c) {
    RawChunk<float> r;
    const float4* p = reinterpret_cast<const float4*>(row) + 2 * c;
    r.a = __ldg(p);
    r.b = __ldg(p + 1);
    return r;
}
// coherent load (rows written earlier by the same kernel must not go through
// the read-only path)
template <typename T>
__device__ __forceinline__ RawChunk<T> load_chunk_coherent(const T* row, int c);
template <>
__device__ __forceinline__ RawChunk<__nv_bfloat16> load_chunk_coherent(const __nv_bfloat16* row, int c) {
    RawChunk<__nv_bfloat16> r;
    r.a = *(reinterpret_cast<const uint4*>(row) + c);
    return r;
}
template <>
__device__ __forceinline__ RawChunk<float> load_chunk_coherent(const float* row, int c) {
    RawChunk<float> r;
    const float4* p = reinterpret_cast<const float4*>(row) + 2 * c;
    r.a = p[0];
    r.b = p[1];
    return r;
}
__device__ __forceinline__ void to_float(const RawChunk<__nv_bfloat16>& r, float (&f)[8]) {
    unpack_bf16x8(r.a, f);
}
__device__ __forceinline__ void to_float(const RawChunk<float>& r, float (&f)[8]) {
    f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w;
    f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
}
template <typename T>
__device__ __forceinline__ RawChunk<T> zero_chunk();
template <>
__device__ __forceinline__ RawChunk<__nv_bfloat16> zero_chunk() {
    RawChunk<__nv_bfloat16> r; r.a = make_uint4(0, 0, 0, 0); return r;
}
template <>
__device__ __forceinline__ RawChunk<float> zero_chunk() {
    RawChunk<float> r; r.a = make_float4(0, 0, 0, 0); r.b = r.a; return r;
}

// store 8 fp32 values as one chunk of a row of type T (round to nearest even)
__device__ __forceinline__ void store_chunk(__nv_bfloat16* row, int c, const float (&f)[8]) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(f[2], f[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(f[4], f[5]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(f[6], f[7]);
    uint4 r;
    r.x = *reinterpret_cast<uint32_t*>(&p0);
    r.y = *reinterpret_cast<uint32_t*>(&p1);
    r.z = *reinterpret_cast<uint32_t*>(&p2);
    r.w = *reinterpret_cast<uint32_t*>(&p3);
    reinterpret_cast<uint4*>(row)[c] = r;
}
__device__ __forceinline__ void store_chunk(float* row, int c, const float (&f)[8]) {
    float4* p = reinterpret_cast<float4*>(row) + 2 * c;
    p[0] = make_float4(f[0], f[1], f[2], f[3]);
    p[1] = make_float4(f[4], f[5], f[6], f[7]);
}

// ---------------------------------------------------------------------------
// Canonical dot product pieces.
// ---------------------------------------------------------------------------
struct Acc2 { float e, o; };

// one chunk into the (even, odd) accumulator pair; packed FFMA2 on sm_100
__device__ __forceinline__ void chunk_fma(Acc2& acc, const float (&a)[8], const float (&b)[8]) {
#if __CUDA_ARCH__ >= 1000
    float2 s = make_float2(acc.e, acc.o);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        s = __ffma2_rn(make_float2(a[2 * j], a[2 * j + 1]), make_float2(b[2 * j], b[2 * j + 1]), s);
    acc.e = s.x; acc.o = s.y;
#else
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        acc.e = __fmaf_rn(a[2 * j], b[2 * j], acc.e);
        acc.o = __fmaf_rn(a[2 * j + 1], b[2 * j + 1], acc.o);
    }
#endif
}

// butterfly over the 16 lanes of a half-warp; every lane gets the sum
// Shuffles name only the 8 lanes of the caller's own group, so the groups of a
// warp may diverge (different trip counts, early exit).
constexpr int GROUP = 8;  // lanes per row
__device__ __forceinline__ unsigned group_mask() { return 0xffu << (threadIdx.x & 24); }

__device__ __forceinline__ float group_sum(float p) {
    const unsigned gm = group_mask();
    p = __fadd_rn(p, __shfl_xor_sync(gm, p, 4));
    p = __fadd_rn(p, __shfl_xor_sync(gm, p, 2));
    p = __fadd_rn(p, __shfl_xor_sync(gm, p, 1));
    return p;
}

// Same butterfly for G values at once with fewer shuffles (a reduce-scatter:
// at each step a lane keeps half of its values and sends the other half).
// On return the canonical sum of head head_of_lane(lane) is in the result; adds
// are commutative so the bits equal group_sum() of each value.  `gm` is the
// shuffle mask: group_mask() where the groups of a warp may have diverged, the
// full mask where the whole warp is known to be converged (cheaper: a variable
// mask makes the compiler emit a membership check).
template <int G> struct HeadReduce;
template <> struct HeadReduce<1> {
    static __device__ __forceinline__ float run(const float (&v)[1], int /*lane*/, unsigned gm) {
        float p = v[0];
        p = __fadd_rn(p, __shfl_xor_sync(gm, p, 4));
        p = __fadd_rn(p, __shfl_xor_sync(gm, p, 2));
        p = __fadd_rn(p, __shfl_xor_sync(gm, p, 1));
        return p;
    }
    static __device__ __forceinline__ int head_of_lane(int /*lane*/) { return 0; }
    static __device__ __forceinline__ bool is_writer(int lane) { return lane == 0; }
    static __device__ __forceinline__ int first_lane(int /*j*/) { return 0; }
};
template <> struct HeadReduce<2> {
    static __device__ __forceinline__ float run(const float (&v)[2], int lane, unsigned gm) {
        const bool hi = lane & 4;
        float r = __fadd_rn(hi ? v[1] : v[0], __shfl_xor_sync(gm, hi ? v[0] : v[1], 4));
        r = __fadd_rn(r, __shfl_xor_sync(gm, r, 2));
        r = __fadd_rn(r, __shfl_xor_sync(gm, r, 1));
        return r;
    }
    static __device__ __forceinline__ int head_of_lane(int lane) { return (lane >> 2) & 1; }
    static __device__ __forceinline__ bool is_writer(int lane) { return (lane & 3) == 0; }
    static __device__ __forceinline__ int first_lane(int j) { return j * 4; }
};
template <> struct HeadReduce<4> {
    static __device__ __forceinline__ float run(const float (&v)[4], int lane, unsigned gm) {
        const bool b2 = lane & 4, b1 = lane & 2;
        float a = __fadd_rn(b2 ? v[2] : v[0], __shfl_xor_sync(gm, b2 ? v[0] : v[2], 4));
        float b = __fadd_rn(b2 ? v[3] : v[1], __shfl_xor_sync(gm, b2 ? v[1] : v[3], 4));
        float r = __fadd_rn(b1 ? b : a, __shfl_xor_sync(gm, b1 ? a : b, 2));
        r = __fadd_rn(r, __shfl_xor_sync(gm, r, 1));
        return r;
    }
    static __device__ __forceinline__ int head_of_lane(int lane) { return (lane >> 1) & 3; }
    static __device__ __forceinline__ bool is_writer(int lane) { return (lane & 1) == 0; }
    static __device__ __forceinline__ int first_lane(int j) { return j * 2; }
};
template <> struct HeadReduce<8> {
    static __device__ __forceinline__ float run(const float (&v)[8], int lane, unsigned gm) {
        const bool b2 = lane & 4, b1 = lane & 2, b0 = lane & 1;
        float w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            w[j] = __fadd_rn(b2 ? v[4 + j] : v[j], __shfl_xor_sync(gm, b2 ? v[j] : v[4 + j], 4));
        float x[2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
            x[j] = __fadd_rn(b1 ? w[2 + j] : w[j], __shfl_xor_sync(gm, b1 ? w[j] : w[2 + j], 2));
        return __fadd_rn(b0 ? x[1] : x[0], __shfl_xor_sync(gm, b0 ? x[0] : x[1], 1));
    }
    static __device__ __forceinline__ int head_of_lane(int lane) { return lane & 7; }
    static __device__ __forceinline__ bool is_writer(int /*lane*/) { return true; }
    static __device__ __forceinline__ int first_lane(int j) { return j; }
};

// canonical dot of a global row with a per-lane register copy of the other
// operand (b[c][8] = the lane's chunks of b).  NCH = chunks per lane.
template <typename T, int NCH>
__device__ __forceinline__ float row_dot(const T* row, const float (&b)[NCH][8], int lane, int dim) {
    Acc2 acc{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            float a[8];
            to_float(load_chunk<T>(row, c), a);
            chunk_fma(acc, a, b[i]);
        }
    }
    return group_sum(__fadd_rn(acc.e, acc.o));
}

// canonical ||a - b||^2 for two global rows (fp32 difference, then the tree)
template <typename TA, typename TB, int NCH>
__device__ __forceinline__ float row_dist2(const TA* ra, const TB* rb, int lane, int dim) {
    Acc2 acc{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            float a[8], b[8], d[8];
            to_float(load_chunk<TA>(ra, c), a);
            to_float(load_chunk<TB>(rb, c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] = __fsub_rn(a[j], b[j]);
            chunk_fma(acc, d, d);
        }
    }
    return group_sum(__fadd_rn(acc.e, acc.o));
}

// the same with coherent loads, and against a register copy of one operand
template <typename T, int NCH>
__device__ __forceinline__ float row_dist2_reg(const T* row, const float (&x)[NCH][8], int lane, int dim) {
    Acc2 acc{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            float a[8], d[8];
            to_float(load_chunk_coherent<T>(row, c), a);
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] = __fsub_rn(x[i][j], a[j]);
            chunk_fma(acc, d, d);
        }
    }
    return group_sum(__fadd_rn(acc.e, acc.o));
}
template <typename TA, typename TB, int NCH>
__device__ __forceinline__ float row_dist2_coherent(const TA* ra, const TB* rb, int lane, int dim) {
    Acc2 acc{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            float a[8], b[8], d[8];
            to_float(load_chunk_coherent<TA>(ra, c), a);
            to_float(load_chunk_coherent<TB>(rb, c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] = __fsub_rn(a[j], b[j]);
            chunk_fma(acc, d, d);
        }
    }
    return group_sum(__fadd_rn(acc.e, acc.o));
}
// canonical ||x||^2 of a register vector
template <int NCH>
__device__ __forceinline__ float reg_sqnorm(const float (&x)[NCH][8]) {
    Acc2 acc{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) chunk_fma(acc, x[i], x[i]);
    return group_sum(__fadd_rn(acc.e, acc.o));
}

// load the lane's chunks of an fp32 vector (query) into registers
template <int NCH>
__device__ __forceinline__ void load_vec_f32(const float* v, float (&b)[NCH][8], int lane, int dim) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            to_float(load_chunk<float>(v, c), b[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) b[i][j] = 0.f;
        }
    }
}
template <typename T, int NCH>
__device__ __forceinline__ void load_vec(const T* v, float (&b)[NCH][8], int lane, int dim) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = lane + 8 * i;
        if (c * 8 < dim) {
            to_float(load_chunk<T>(v, c), b[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) b[i][j] = 0.f;
        }
    }
}

// ---------------------------------------------------------------------------
// int8 side copy of a child row (D = 128), written by the 8 lanes of a group; see search_q8.cu.
//   x        the lane's two chunks of the row in fp32 (values exactly as stored in the index)
//   chan     per-channel scales s_i [128] followed by min_i s_i at [128]
//   dst      the row's 128 bytes;  swz = slot & 7 permutes its 16-byte chunks
//   meta     (step, err) as two fp16: k'_i = x_i / s_i, step = max |k'_i| / 127 rounded up, k~_i = rint(k'_i / step),
//            err >= ||k' - step k~||_2 + 2^-15 ||x||_2 / min_i s_i  (the second term covers the
//            rounding of the canonical fp32 dot product for any query: ||q (.) s|| >= min s ||q||)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void q8_write_row(const float (&x)[2][8], const float* __restrict__ chan, int8_t* dst,
                                             uint32_t* meta, int swz, int lane) {
    float kp[2][8];
    float amax = 0.f;
    Acc2 nx{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = lane + GROUP * i;
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(chan) + 2 * c);
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(chan) + 2 * c + 1);
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            kp[i][e] = __fdiv_rn(x[i][e], sc[e]);
            amax = fmaxf(amax, fabsf(kp[i][e]));
        }
        chunk_fma(nx, x[i], x[i]);
    }
    const unsigned gm = group_mask();
    amax = fmaxf(amax, __shfl_xor_sync(gm, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(gm, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(gm, amax, 1));
    // the step is stored as fp16, so it is rounded (up) to one first and the row quantised with that
    bool ok = amax > 0.f && amax < 3.0e38f;
    float step = ok ? __half2float(__float2half_ru(__fdiv_rn(amax, 127.0f))) : 1.0f;
    if (!(step > 0.f) || !(step < 6.0e4f)) { ok = false; step = 1.0f; }
    Acc2 ne{0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float dlt[8];
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float kq = ok ? rintf(__fdiv_rn(kp[i][e], step)) : 0.f;
            kq = fminf(fmaxf(kq, -127.f), 127.f);
            dlt[e] = __fmaf_rn(-kq, step, kp[i][e]);
            w[e >> 2] |= ((uint32_t)(int)kq & 0xffu) << (8 * (e & 3));
        }
        chunk_fma(ne, dlt, dlt);
        const int c = lane + GROUP * i;        // 8-element chunk of the row: half (c & 1) of 16-byte chunk c >> 1
        const int off = (((c >> 1) ^ swz) << 4) + ((c & 1) << 3);
        *reinterpret_cast<uint2*>(dst + off) = make_uint2(w[0], w[1]);
    }
    const float err2 = group_sum(__fadd_rn(ne.e, ne.o));
    const float xsq = group_sum(__fadd_rn(nx.e, nx.o));
    if (lane == 0) {
        const float min_s = __ldg(chan + 128);
        const float err = ok ? sqrtf(err2) * 1.001f + 3.1e-5f * sqrtf(xsq) / min_s
                             : (amax > 0.f ? 3.0e38f : 0.f);    // a row that cannot be quantised is always a candidate
        // rounded up; beyond the fp16 range it becomes +inf, which keeps the row a candidate
        *meta = (uint32_t)__half_as_ushort(__float2half_ru(step)) | ((uint32_t)__half_as_ushort(__float2half_ru(err)) << 16);
    }
}

// non-negative floats order like their bit patterns
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

}  // namespace hira
