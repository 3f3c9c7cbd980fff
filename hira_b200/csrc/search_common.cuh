// Pieces shared by the two search kernels (the streaming one and the one with the int8
// pre-filter): launch parameters, asynchronous-copy helpers and the canonical gate arithmetic.
#pragma once

#include "common.cuh"

namespace hira {

constexpr int MAX_TILE_ROWS = 1024;
constexpr int SEARCH_RPI = 2;  // rows per 8-lane group per pipeline step
constexpr uint32_t NOT_EMITTED = 0xffffffffu;  // score-buffer sentinel (a NaN no arithmetic produces)

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_16s(uint32_t smem_addr, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

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
    // optional by-product for the append that follows: nearest valid parent of one new key per head
    const void* scan_key;              // [n_heads] rows of `dim` elements in the index dtype, or NULL
    long long scan_key_stride;         // elements between the heads' keys
    const float* parent_sqnorm;        // [n_heads][cap_parents]
    unsigned long long* scan_out;      // [n_heads] packed (order_key(score) << 32 | parent slot), atomicMin
    int n_heads, n_qheads, group, depth, bf, dim;
    int cap_parents, cap_gp, tile_parents, n_tiles, n_chunks, flags;
    int n_tiles_active;       // tiles launched (<= n_tiles, which stays the stride of out_count)
    uint32_t ring_offset;     // byte offset of the per-thread prefetch ring in dynamic shared memory
    int ng;                   // grandparents touched by one tile
    int tile_gp_shift;        // first grandparent of tile t: t >> shift (TP * 2^shift == bf), t * ng (-1: TP % bf == 0), t * TP / bf (-2)
    uint32_t bf_magic;        // ceil(2^32 / bf): x / bf == __umulhi(x, bf_magic) for x < 2^20, bf <= 1024
};

__device__ __forceinline__ int div_bf(int x, int bf, uint32_t magic) {
    return bf == 1 ? x : (int)__umulhi((uint32_t)x, magic);
}

__device__ __forceinline__ bool gate_keep(float dot, float r, float qn, bool has_qn, float tau, bool ge) {
    const float rr = has_qn ? __fmul_rn(qn, r) : r;
    const float s = __fadd_rn(dot, rr);
    return ge ? (s >= tau) : (s > tau);
}

// bit j of the result = predicate of the first lane that owns head j in this 8-lane group
template <int GT>
__device__ __forceinline__ uint32_t head_mask_from_ballot(uint32_t ballot, int tid) {
    const int base = tid & 24;
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < GT; ++j) m |= ((ballot >> (base + HeadReduce<GT>::first_lane(j))) & 1u) << j;
    return m;
}

// canonical q.row for the GT heads held in qreg; result for head_of_lane(lane)
template <typename T, int GT, int NCH>
__device__ __forceinline__ float gate_dot(const T* row, const float (&qreg)[GT][NCH][8], int lane, int dim, bool load) {
    float v[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) v[j] = 0.f;
    if (load) {
        Acc2 acc[GT];
#pragma unroll
        for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
            const int c = lane + GROUP * ci;
            if (c * 8 < dim) {
                float a[8];
                to_float(load_chunk<T>(row, c), a);
#pragma unroll
                for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);
            }
        }
#pragma unroll
        for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
    }
    return HeadReduce<GT>::run(v, lane, 0xffffffffu);  // callers keep the warp converged
}

// the same from chunks already loaded into registers
template <typename T, int GT, int NCH>
__device__ __forceinline__ float gate_dot_raw(const RawChunk<T> (&raw)[NCH], const float (&qreg)[GT][NCH][8], int lane) {
    Acc2 acc[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) acc[j] = Acc2{0.f, 0.f};
#pragma unroll
    for (int ci = 0; ci < NCH; ++ci) {
        float a[8];
        to_float(raw[ci], a);
#pragma unroll
        for (int j = 0; j < GT; ++j) chunk_fma(acc[j], a, qreg[j][ci]);   // chunks outside the row were loaded as zeros
    }
    float v[GT];
#pragma unroll
    for (int j = 0; j < GT; ++j) v[j] = __fadd_rn(acc[j].e, acc[j].o);
    return HeadReduce<GT>::run(v, lane, 0xffffffffu);  // callers keep the warp converged
}

template <typename T, int NCH>
__device__ __forceinline__ void load_row_raw(RawChunk<T> (&raw)[NCH], const T* row, int lane, int dim, bool doit) {
#pragma unroll
    for (int ci = 0; ci < NCH; ++ci) {
        const int c = lane + GROUP * ci;
        if (doit && c * 8 < dim) raw[ci] = load_chunk<T>(row, c);
        else raw[ci] = zero_chunk<T>();
    }
}


// set by search.cu's host code, consumed by the kernel launchers of both files
int launch_search_q8(const SearchParams& P, const hira_index_t* ix, int max_group, cudaStream_t stream);
int q8_refresh(const hira_index_t* ix, cudaStream_t s, long long parents_bound);
bool search_q8_applicable(const hira_index_t* ix, const SearchParams& P);

}  // namespace hira
