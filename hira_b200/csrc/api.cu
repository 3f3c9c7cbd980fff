// Error plumbing and argument validation shared by every entry point.
#include "common.cuh"

#include <stdarg.h>
#include <string.h>

namespace hira {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int active_tiles(const hira_index_t* ix, int tile_parents) {
    const int active = ix->active_parents > 0 ? ix->active_parents : ix->cap_parents;
    return (active + tile_parents - 1) / tile_parents;
}

int validate_index(const hira_index_t* ix, bool need_values) {
    HIRA_CHECK_ARG(ix != nullptr, HIRA_ERR_ARG, "index is NULL");
    HIRA_CHECK_ARG(ix->dtype == HIRA_F32 || ix->dtype == HIRA_BF16, HIRA_ERR_DTYPE,
                   "index dtype %d is neither HIRA_F32 nor HIRA_BF16", ix->dtype);
    HIRA_CHECK_ARG(ix->depth == 2 || ix->depth == 3, HIRA_ERR_ARG,
                   "Unsupported index depth: %d (2 or 3 levels)", ix->depth);
    HIRA_CHECK_ARG(ix->bf >= 1 && ix->bf <= 1024, HIRA_ERR_SHAPE, "branching factor %d outside 1..1024", ix->bf);
    HIRA_CHECK_ARG(ix->dim >= 8 && ix->dim <= 256 && ix->dim % 8 == 0, HIRA_ERR_SHAPE,
                   "dim=%d must be a multiple of 8 in 8..256", ix->dim);
    HIRA_CHECK_ARG(ix->n_heads >= 1, HIRA_ERR_SHAPE, "n_heads=%d must be >= 1", ix->n_heads);
    HIRA_CHECK_ARG(ix->cap_parents >= 1, HIRA_ERR_SHAPE, "cap_parents=%d must be >= 1", ix->cap_parents);
    HIRA_CHECK_ARG((long long)ix->cap_parents * ix->bf < (1ll << 30), HIRA_ERR_SHAPE,
                   "cap_parents*bf = %lld child slots per head exceeds 2^30",
                   (long long)ix->cap_parents * ix->bf);
    HIRA_CHECK_ARG(ix->active_parents >= 0 && ix->active_parents <= ix->cap_parents, HIRA_ERR_SHAPE,
                   "active_parents=%d outside 0..cap_parents (%d)", ix->active_parents, ix->cap_parents);
    HIRA_CHECK_ARG(ix->children && ix->parents && ix->parent_radii && ix->child_counts && ix->used,
                   HIRA_ERR_ARG, "index has a NULL children/parents/parent_radii/child_counts/used pointer");
    if (ix->depth == 3) {
        HIRA_CHECK_ARG(ix->cap_gp >= 1 && ix->cap_parents == ix->cap_gp * ix->bf, HIRA_ERR_SHAPE,
                       "depth 3 needs cap_parents (%d) == cap_gp (%d) * bf (%d)", ix->cap_parents, ix->cap_gp, ix->bf);
        HIRA_CHECK_ARG(ix->grand_parents && ix->gp_radii && ix->gp_counts, HIRA_ERR_ARG,
                       "depth-3 index has a NULL grand_parents/gp_radii/gp_counts pointer");
    }
    if (need_values || ix->values) {
        HIRA_CHECK_ARG(ix->values != nullptr, HIRA_ERR_ARG, "index has no values");
        HIRA_CHECK_ARG(ix->vdtype == HIRA_F32 || ix->vdtype == HIRA_BF16, HIRA_ERR_DTYPE,
                       "values dtype %d is neither HIRA_F32 nor HIRA_BF16", ix->vdtype);
        HIRA_CHECK_ARG(ix->vdim >= 8 && ix->vdim <= 256 && ix->vdim % 8 == 0, HIRA_ERR_SHAPE,
                       "vdim=%d must be a multiple of 8 in 8..256", ix->vdim);
    }
    return HIRA_OK;
}

}  // namespace hira

extern "C" const char* hira_last_error(void) { return hira::g_err; }
extern "C" const char* hira_version(void) { return "hira_b200 0.1 (sm_100a)"; }

extern "C" int hira_decode_attention(const hira_index_t* index, const void* q, int32_t q_dtype, float sm_scale,
                                     const float* tau, const int32_t* q2kv, int32_t n_qheads, int32_t max_group,
                                     int32_t flags, int32_t tile_parents, float* q_hat, float* logit_scale,
                                     int32_t* idx, float* score, int32_t* count,
                                     const void* queued_k, const void* queued_v, int32_t n_queued,
                                     int64_t queued_head_stride, int32_t n_splits, float* workspace,
                                     float* out, float* out_ml,
                                     const void* scan_key, int64_t scan_key_stride, uint64_t* scan_out,
                                     void* searched, void* stream) {
    HIRA_CHECK_ARG(index != nullptr, HIRA_ERR_ARG, "hira_decode_attention: index is NULL");
    HIRA_CHECK_ARG(q && q_hat && logit_scale, HIRA_ERR_ARG, "hira_decode_attention: q, q_hat and logit_scale must not be NULL");
    int rc = hira_prepare_query(q, q_dtype, n_qheads, index->dim, sm_scale, q_hat, logit_scale, stream);
    if (rc != HIRA_OK) return rc;
    if (scan_out != nullptr) {
        HIRA_CHECK_ARG(q2kv == nullptr, HIRA_ERR_ARG, "hira_decode_attention: the fused parent scan needs q2kv == NULL");
        rc = hira_search_scan(index, q_hat, tau, logit_scale, nullptr, n_qheads, flags, tile_parents, nullptr, idx,
                              score, count, nullptr, scan_key, scan_key_stride, scan_out, stream);
    } else {
        rc = hira_search(index, q_hat, tau, logit_scale, nullptr, q2kv, n_qheads, max_group, flags, tile_parents,
                         nullptr, idx, score, count, nullptr, stream);
    }
    if (rc != HIRA_OK) return rc;
    if (searched != nullptr) {
        cudaError_t e = cudaEventRecord(reinterpret_cast<cudaEvent_t>(searched), reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) {
            hira::set_error("hira_decode_attention: cudaEventRecord: %s", cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
    }
    return hira_sparse_attn(index, q_hat, logit_scale, q2kv, n_qheads, tile_parents, idx, score, count,
                            queued_k, queued_v, n_queued, queued_head_stride, n_splits, workspace, out, out_ml,
                            stream);
}
