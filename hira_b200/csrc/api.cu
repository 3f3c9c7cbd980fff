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
    if (ix->children_q8 || ix->children_q8_meta || ix->q8_chan_scale || ix->q8_query_scratch) {
        HIRA_CHECK_ARG(ix->children_q8 && ix->children_q8_meta && ix->q8_chan_scale && ix->q8_query_scratch, HIRA_ERR_ARG,
                       "the int8 side copy needs children_q8, children_q8_meta, q8_chan_scale and q8_query_scratch together");
        HIRA_CHECK_ARG(ix->dim == 128, HIRA_ERR_SHAPE, "the int8 side copy needs dim == 128 (got %d)", ix->dim);
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
                                     float* out, float* out_ml, int64_t out_head_stride, int64_t ml_head_stride,
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
                            out_head_stride, ml_head_stride, stream);
}

// ---------------------------------------------------------------------------
// One decode step from host buffers.
// ---------------------------------------------------------------------------
#define HIRA_CUDA_OK(call, what)                                                        \
    do {                                                                                \
        cudaError_t e__ = (call);                                                       \
        if (e__ != cudaSuccess) {                                                       \
            hira::set_error("hira_decode_step: %s: %s", (what), cudaGetErrorString(e__)); \
            return HIRA_ERR_CUDA;                                                       \
        }                                                                               \
    } while (0)

extern "C" int hira_step_events_create(hira_step_t* step) {
    HIRA_CHECK_ARG(step != nullptr, HIRA_ERR_ARG, "hira_step_events_create: step is NULL");
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < 3; ++i) {
        cudaError_t e = cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
            hira::set_error("hira_step_events_create: %s", cudaGetErrorString(e));
            return HIRA_ERR_CUDA;
        }
    }
    step->ev_copied = ev[0]; step->ev_searched = ev[1]; step->ev_appended = ev[2];
    return HIRA_OK;
}

extern "C" int hira_step_events_destroy(hira_step_t* step) {
    HIRA_CHECK_ARG(step != nullptr, HIRA_ERR_ARG, "hira_step_events_destroy: step is NULL");
    void** ev[3] = {&step->ev_copied, &step->ev_searched, &step->ev_appended};
    for (int i = 0; i < 3; ++i) {
        if (*ev[i]) cudaEventDestroy(reinterpret_cast<cudaEvent_t>(*ev[i]));
        *ev[i] = nullptr;
    }
    return HIRA_OK;
}

extern "C" int hira_decode_step(const hira_index_t* index, const hira_step_t* st, const void* q_host,
                                int32_t q_dtype, float sm_scale, int32_t n_qheads, const float* tau_dev,
                                const void* k_host, const void* v_host, float* out_host, void* stream,
                                void* side_stream) {
    int rc = hira::validate_index(index, true);
    if (rc != HIRA_OK) return rc;
    HIRA_CHECK_ARG(st && q_host && out_host, HIRA_ERR_ARG, "hira_decode_step: step, q_host and out_host must not be NULL");
    HIRA_CHECK_ARG(st->q_dev && st->q_hat && st->logit_scale && st->idx && st->score && st->count && st->workspace &&
                   st->out_dev, HIRA_ERR_ARG, "hira_decode_step: the step's device buffers are incomplete");
    HIRA_CHECK_ARG(st->ev_copied && st->ev_searched && st->ev_appended, HIRA_ERR_ARG,
                   "hira_decode_step: call hira_step_events_create first");
    HIRA_CHECK_ARG(q_dtype == HIRA_F32 || q_dtype == HIRA_BF16, HIRA_ERR_DTYPE, "hira_decode_step: q_dtype %d", q_dtype);
    HIRA_CHECK_ARG(tau_dev != nullptr || (st->tau && st->tau_samples && st->n_samples >= 1), HIRA_ERR_ARG,
                   "hira_decode_step: give tau_dev, or tau scratch and threshold samples in the step");
    const bool append = k_host != nullptr;
    HIRA_CHECK_ARG(!append || (st->k_dev && st->status && (v_host != nullptr) == (index->values != nullptr)),
                   HIRA_ERR_ARG, "hira_decode_step: an append needs k_dev, status and values iff the index stores them");
    HIRA_CHECK_ARG(!append || !v_host || st->v_dev, HIRA_ERR_ARG, "hira_decode_step: v_dev is NULL");
    cudaStream_t main_s = reinterpret_cast<cudaStream_t>(stream);
    cudaStream_t side_s = side_stream ? reinterpret_cast<cudaStream_t>(side_stream) : main_s;
    cudaEvent_t copied = reinterpret_cast<cudaEvent_t>(st->ev_copied);
    cudaEvent_t searched = reinterpret_cast<cudaEvent_t>(st->ev_searched);
    cudaEvent_t appended = reinterpret_cast<cudaEvent_t>(st->ev_appended);
    const size_t qe = hira::elem_size(q_dtype), ke = hira::elem_size(index->dtype), ve = hira::elem_size(index->vdtype);
    const bool fused = append && st->scan != nullptr;

    // The second stream joins the step here: it starts behind whatever precedes the step on `stream` (under
    // stream capture this is what makes its work part of the recorded graph).
    if (append && side_s != main_s) {
        HIRA_CUDA_OK(cudaEventRecord(copied, main_s), "event record");
        HIRA_CUDA_OK(cudaStreamWaitEvent(side_s, copied, 0), "stream wait");
    }
    HIRA_CUDA_OK(cudaMemcpyAsync(st->q_dev, q_host, (size_t)n_qheads * index->dim * qe, cudaMemcpyHostToDevice, main_s),
                 "query copy");
    if (append) {
        // the new key / value rows travel on the side stream, beside the query copy and the search
        HIRA_CUDA_OK(cudaMemcpyAsync(st->k_dev, k_host, (size_t)index->n_heads * index->dim * ke,
                                     cudaMemcpyHostToDevice, side_s), "key copy");
        if (v_host)
            HIRA_CUDA_OK(cudaMemcpyAsync(st->v_dev, v_host, (size_t)index->n_heads * index->vdim * ve,
                                         cudaMemcpyHostToDevice, side_s), "value copy");
        if (fused && side_s != main_s) {   // the search reads the key
            HIRA_CUDA_OK(cudaEventRecord(copied, side_s), "event record");
            HIRA_CUDA_OK(cudaStreamWaitEvent(main_s, copied, 0), "stream wait");
        }
    }
    rc = hira_prepare_query(st->q_dev, q_dtype, n_qheads, index->dim, sm_scale, st->q_hat, st->logit_scale, stream);
    if (rc != HIRA_OK) return rc;
    const float* tau = tau_dev;
    if (tau == nullptr) {
        rc = hira_threshold(st->tau_samples, index->dtype, index->n_heads, st->n_samples, index->dim,
                            st->samples_head_stride, st->q_hat, nullptr, n_qheads, st->tau_method, st->tau_k, st->tau,
                            stream);
        if (rc != HIRA_OK) return rc;
        tau = st->tau;
    }
    if (fused)
        rc = hira_search_scan(index, st->q_hat, tau, st->logit_scale, nullptr, n_qheads, st->flags, st->tile_parents,
                              nullptr, st->idx, st->score, st->count, nullptr, st->k_dev, index->dim, st->scan, stream);
    else
        rc = hira_search(index, st->q_hat, tau, st->logit_scale, nullptr, nullptr, n_qheads, 0, st->flags,
                         st->tile_parents, nullptr, st->idx, st->score, st->count, nullptr, stream);
    if (rc != HIRA_OK) return rc;
    if (append) {
        // the attention reads nothing the append writes: the append only waits for the search
        if (side_s != main_s) {
            HIRA_CUDA_OK(cudaEventRecord(searched, main_s), "event record");
            HIRA_CUDA_OK(cudaStreamWaitEvent(side_s, searched, 0), "stream wait");
        }
        if (fused)
            rc = hira_append_scanned(index, st->k_dev, v_host ? st->v_dev : nullptr, index->dim, index->vdim, -1,
                                     st->status, st->scan, side_s);
        else
            rc = hira_append(index, st->k_dev, v_host ? st->v_dev : nullptr, 1, index->dim, index->vdim, -1,
                             st->status, st->append_ws, st->append_ws_bytes, side_s);
        if (rc != HIRA_OK) return rc;
        if (side_s != main_s) HIRA_CUDA_OK(cudaEventRecord(appended, side_s), "event record");
    }
    rc = hira_sparse_attn(index, st->q_hat, st->logit_scale, nullptr, n_qheads, st->tile_parents, st->idx, st->score,
                          st->count, nullptr, nullptr, 0, 0, st->n_splits, st->workspace, st->out_dev, nullptr, 0, 0,
                          stream);
    if (rc != HIRA_OK) return rc;
    HIRA_CUDA_OK(cudaMemcpyAsync(out_host, st->out_dev, (size_t)n_qheads * index->vdim * sizeof(float),
                                 cudaMemcpyDeviceToHost, main_s), "output copy");
    if (append && side_s != main_s) HIRA_CUDA_OK(cudaStreamWaitEvent(main_s, appended, 0), "stream wait");
    return HIRA_OK;
}
