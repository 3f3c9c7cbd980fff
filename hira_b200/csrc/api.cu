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
