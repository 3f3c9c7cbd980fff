/*
 * hira_b200.h -- C ABI of libhira_b200.so: the decode-time hot path of HIRA
 * ("Louver" hierarchical range-searching sparse attention) as hand-written
 * CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions (all entry points unless stated otherwise)
 *   - Every pointer inside hira_index_t and every data argument is a DEVICE
 *     pointer; the hira_index_t struct itself lives in host memory.
 *   - Nothing is allocated, freed or synchronised: the caller owns all memory
 *     (including workspaces) and all work is enqueued on `stream`.
 *   - Return value: HIRA_OK, or a negative HIRA_ERR_* detected on the host
 *     before any launch; hira_last_error() gives the message for the calling
 *     thread.  Problems only the device can see (index capacity exhausted
 *     during an append) are reported through a caller-provided `int32_t*
 *     status` word in device memory (0 = ok), never by a trap.
 *   - Heads: the batch is folded into the head axis.  `n_heads` counts
 *     (batch, kv_head) pairs, `n_qheads` counts (batch, query_head) pairs.
 *
 * Blocked index layout (same as the reference's CUDAIndexer tensors,
 * indexer/cuda.py:40-54, 350-356, 440-446):
 *   parent p owns child slots [p*bf, (p+1)*bf); with depth 3 grandparent g owns
 *   parent slots [g*bf, (g+1)*bf).  Unlike the reference, which infers
 *   validity from "row is all pad_value" on every call
 *   (indexer/cuda.py:1241-1298), validity is explicit persistent state:
 *   child_counts / gp_counts / used.
 */
#ifndef HIRA_B200_H
#define HIRA_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HIRA_OK 0
#define HIRA_ERR_ARG (-1)      /* null pointer / bad enum / bad flag            */
#define HIRA_ERR_SHAPE (-2)    /* sizes inconsistent with the index             */
#define HIRA_ERR_DTYPE (-3)    /* unsupported element type                      */
#define HIRA_ERR_CAPACITY (-4) /* workspace or fixed scratch too small          */
#define HIRA_ERR_CUDA (-5)     /* a CUDA runtime call or launch failed          */

/* element types */
#define HIRA_F32 0
#define HIRA_BF16 1

/* device status word bits written by hira_append and hira_build */
#define HIRA_STATUS_PARENTS_FULL 1 /* no free parent slot left for an orphan key */
#define HIRA_STATUS_GP_FULL 2      /* no free grandparent slot left              */
#define HIRA_STATUS_ASSIGN_FAILED 4 /* hira_build: the tensor-core assignment gave up on a bounded
                                       wait for some points (their hira_assign index is -1); the
                                       build placed them under centre 0, so the index is valid but
                                       of poor quality: rebuild with use_tensor_cores = 0 */

/* search flags */
#define HIRA_GATE_GT 0x0          /* keep node iff q.c + r >  tau (reference Triton kernels, kernels/triton_search_kernels.py:49,114,131) */
#define HIRA_GATE_GE 0x1          /* keep node iff q.c + r >= tau (reference CPU kernels, kernels/cpp/torch_ext_v3.cpp:182,212)         */
#define HIRA_LEAF_CANDIDATES 0x0  /* emit every child of a kept parent (reference Triton kernels: no leaf test)                         */
#define HIRA_LEAF_GE 0x2          /* emit child iff q.k >= tau (reference CPU kernels, torch_ext_v3.cpp:237-240)                        */
#define HIRA_LEAF_GT 0x4          /* emit child iff q.k >  tau                                                                          */

/* threshold methods */
#define HIRA_TAU_SAMPLE_MAX 0       /* max of the sample scores                      (cache/threshold_finder.py:1-3)   */
#define HIRA_TAU_SAMPLE_MEAN_TOPK 1 /* mean of the k largest sample scores           (cache/threshold_finder.py:6-8)   */
#define HIRA_TAU_SAMPLE_KTH 2       /* k-th largest sample score                                                        */

typedef struct hira_index {
    int32_t dtype;        /* HIRA_F32 | HIRA_BF16: children, parents, grand_parents   */
    int32_t vdtype;       /* element type of values                                    */
    int32_t depth;        /* 2 or 3 (CUDAIndexer.DEPTH, indexer/cuda.py:18-21)         */
    int32_t bf;           /* branching factor, 1..1024                                 */
    int32_t dim;          /* D, multiple of 8, <= 256                                  */
    int32_t vdim;         /* V, multiple of 8, <= 256; 0 when values == NULL           */
    int32_t n_heads;      /* (batch, kv_head) pairs                                    */
    int32_t cap_parents;  /* parent slots allocated per head (depth 3: cap_gp * bf)    */
    int32_t cap_gp;       /* grandparent slots allocated per head (depth 3), else 0    */
    int32_t active_parents; /* host's upper bound on the parent slots in use (0 = unknown: all of
                               cap_parents).  Search, sparse attention and hira_kth_score skip the
                               tiles beyond it: their out_count entries are neither written nor read.
                               The reference has no such field (it sizes every launch by the
                               tensors' extents, searcher/cuda.py:96-143).                    */
    void* children;        /* [n_heads][cap_parents*bf][dim]                           */
    void* values;          /* [n_heads][cap_parents*bf][vdim] or NULL                  */
    int32_t* slot2token;   /* [n_heads][cap_parents*bf] token position in slot, -1 empty */
    void* parents;         /* [n_heads][cap_parents][dim]                              */
    float* parent_radii;   /* [n_heads][cap_parents]                                   */
    float* parent_sqnorm;  /* [n_heads][cap_parents] cached ||c||^2                    */
    int32_t* child_counts; /* [n_heads][cap_parents] filled child slots (contiguous from 0) */
    void* grand_parents;   /* [n_heads][cap_gp][dim]   (depth 3)                       */
    float* gp_radii;       /* [n_heads][cap_gp]                                        */
    float* gp_sqnorm;      /* [n_heads][cap_gp]                                        */
    int32_t* gp_counts;    /* [n_heads][cap_gp] filled parent slots per grandparent    */
    int32_t* used;         /* [n_heads][4]: {parent slots in use (high-water mark),
                              grandparents in use, keys stored, reserved}             */
    /* Optional int8 side copy of the children (dim == 128 only; all three NULL = none).  With it
       hira_search reads 128-byte int8 rows, scores them on the tensor cores and re-reads only the
       rows that can reach the threshold in the index dtype; results are bit-identical.  Written by
       hira_build, kept up to date by the appends, recomputed by hira_q8_refresh.  The reference
       has no counterpart.                                                                       */
    void* children_q8;        /* [n_heads][cap_parents*bf][128] int8, 16-byte chunks of slot r
                                 permuted by r & 7                                             */
    uint32_t* children_q8_meta; /* [n_heads][cap_parents*bf]: (quantisation step, error bound) as two fp16 */
    float* q8_chan_scale;     /* [n_heads][HIRA_Q8_CHAN]: 128 per-channel scales, their minimum,
                                 and three words the searches keep (how many stages the last
                                 search's gates kept: decides how the next one streams)          */
    void* q8_query_scratch;   /* [n_heads][HIRA_Q8_QUERY_CHUNKS][HIRA_Q8_QUERY_BYTES] bytes that
                                 every hira_search through the side copy rewrites (the query
                                 heads as int8 terms): searches of ONE index that overlap on the
                                 GPU must not both use the side copy                            */
} hira_index_t;
#define HIRA_Q8_CHAN 136
#define HIRA_Q8_QUERY_CHUNKS 4
#define HIRA_Q8_QUERY_BYTES 2112

const char* hira_last_error(void);
const char* hira_version(void);

/* ------------------------------------------------------------------------- */
/* Search.  Replaces CUDASearcher.search -> triton_two_level_filter /
 * triton_three_level_filter (searcher/cuda.py:56-143,
 * kernels/triton_search_wrappers.py:113-211,287-358,
 * kernels/triton_search_kernels.py:6-148) and, with HIRA_GATE_GE|HIRA_LEAF_GE,
 * the CPU fused_tree_search_v3 semantics (kernels/cpp/torch_ext_v3.cpp:36-247)
 * on the blocked layout.
 *
 *   q        [n_qheads][dim] fp32     tau [n_qheads] fp32
 *   scaling  [n_qheads] fp32 or NULL (1.0): multiplies emitted scores only
 *   qnorm    [n_qheads] fp32 or NULL: gate uses q.c + qnorm*r; NULL = unit query
 *            (the reference assumes a unit query, searcher/cpu.py:61-63)
 *   q2kv     [n_qheads] int32 or NULL: NULL = query head i belongs to kv head
 *            i / (n_qheads / n_heads)
 *   max_group: with an explicit q2kv, the largest number of query heads that
 *            map to one kv head (0 = unknown: n_qheads is assumed); ignored
 *            when q2kv is NULL
 *   out_dense  [n_qheads][cap_parents*bf] fp32 or NULL: score*scaling where
 *            emitted, 0 elsewhere; every element is written (no memset needed)
 *   out_idx / out_score [n_qheads][cap_parents*bf], out_count
 *            [n_qheads][n_tiles] or all NULL: compacted output.  Tile t of a
 *            head covers parent slots [t*tile_parents, (t+1)*tile_parents);
 *            its emitted child slots are written in ascending slot order to
 *            out_idx/out_score starting at element t*tile_parents*bf, and their
 *            number to out_count[qh][t].
 *   stats    [n_qheads][HIRA_SEARCH_STATS] uint32 or NULL; added to, not cleared:
 *            {gp tested, gp kept, parents tested, parents kept, child rows read
 *             on behalf of this head, children emitted, U, P} where U and P
 *            (booked on the first query head of each group) count the child
 *            rows and parent rows actually loaded, i.e. for the union of the
 *            group's heads -- the kernel's real memory traffic; with the int8 side copy also
 *            {C, S} (again on the first head of a group): child rows re-read in the index dtype
 *            after the int8 pre-filter, and int8 rows scored
 *   tile_parents: use hira_search_tile_parents(); n_tiles =
 *            ceil(cap_parents / tile_parents).
 */
#define HIRA_SEARCH_STATS 10
int hira_search_tile_parents(const hira_index_t* index);
int hira_search(const hira_index_t* index, const float* q, const float* tau,
                const float* scaling, const float* qnorm, const int32_t* q2kv,
                int32_t n_qheads, int32_t max_group, int32_t flags,
                int32_t tile_parents,
                float* out_dense, int32_t* out_idx, float* out_score,
                int32_t* out_count, uint32_t* stats, void* stream);

/* ------------------------------------------------------------------------- */
/* Sparse attention over the compacted search output (the reference names
 * hira_attention but ships only a stub, attention/hira_attention.py:1-3).
 * Softmax over {emitted children} U {queued keys}; logits of emitted children
 * are out_score (so pass scaling = ||q|| * softmax_scale to hira_search);
 * logits of queued keys are scaling * (q . k_queued) computed here.
 *
 *   queued_k/queued_v [n_heads][n_queued][dim|vdim] in index dtype/vdtype with
 *            row strides queued_head_stride (elements between heads, the same for
 *            both arrays: n_queued > 0 therefore requires dim == vdim, else
 *            HIRA_ERR_SHAPE); may be NULL when n_queued == 0
 *   workspace: n_qheads * n_splits * (vdim + 2) floats of scratch
 *   out      [n_qheads][vdim] fp32, normalised attention output
 *   out_ml   [n_qheads][2] fp32 or NULL: (running max m, denominator l) so that
 *            shards can be merged with hira_merge_partials
 *   n_splits: CTAs per query head (>= 1); use hira_attn_default_splits()
 *   out_head_stride / ml_head_stride: floats between the rows of consecutive query heads in
 *            out / out_ml (0 = dense: vdim and 2), so that both can be written straight into a
 *            packed [n_qheads][2 + vdim] message of (m, l, out) rows
 */
int hira_attn_default_splits(int32_t n_qheads, int32_t n_tiles);
int hira_sparse_attn(const hira_index_t* index, const float* q,
                     const float* scaling, const int32_t* q2kv,
                     int32_t n_qheads, int32_t tile_parents,
                     const int32_t* idx, const float* score,
                     const int32_t* count, const void* queued_k,
                     const void* queued_v, int32_t n_queued,
                     int64_t queued_head_stride, int32_t n_splits,
                     float* workspace, float* out, float* out_ml,
                     int64_t out_head_stride, int64_t ml_head_stride, void* stream);

/* hira_sparse_attn without a caller workspace.  No counterpart in the reference: it
 * exists for callers that cannot allocate device memory at this point -- a decode
 * loop that must not call cudaMalloc after warm-up, a plugin that is handed only its
 * inputs and outputs, a C host with no device allocator.  The split-KV partials go to
 * an array built into the library (HIRA_NOALLOC_SCRATCH_FLOATS floats = 4 MiB, held on
 * every GPU that loads the library until the process exits); the call fails with
 * HIRA_ERR_CAPACITY when n_qheads * n_splits * (vdim + 2) is larger than that.
 * Same arguments and results as hira_sparse_attn minus `workspace`.  It calls no
 * cudaMalloc / cudaFree and no allocating library routine.  The first call on a device
 * looks up the array's device address (with that device current): make that call
 * before any stream capture begins.  All calls share the one array, which keeps the
 * previous call's partials; nothing in it needs clearing, but two calls that overlap
 * on the GPU (different streams, or different threads) race on it. */
#define HIRA_NOALLOC_SCRATCH_FLOATS (1 << 20)
int hira_sparse_attn_noalloc(const hira_index_t* index, const float* q,
                             const float* scaling, const int32_t* q2kv,
                             int32_t n_qheads, int32_t tile_parents,
                             const int32_t* idx, const float* score,
                             const int32_t* count, const void* queued_k,
                             const void* queued_v, int32_t n_queued,
                             int64_t queued_head_stride, int32_t n_splits,
                             float* out, float* out_ml, int64_t out_head_stride,
                             int64_t ml_head_stride, void* stream);

/* Log-sum-exp merge of partial softmax results (used across sequence shards
 * after an all-gather).  part_o [n_parts][n_qheads][vdim] holds NORMALISED
 * outputs, part_ml [n_parts][n_qheads][2] their (m, l); the four strides (in
 * floats; 0 = dense) let both point into one gathered buffer of packed
 * [n_parts][n_qheads][2 + vdim] rows.  Writes the normalised merged output
 * [n_qheads][vdim] and optionally its (m, l) [n_qheads][2]. */
int hira_merge_partials(const float* part_o, const float* part_ml,
                        int32_t n_parts, int32_t n_qheads, int32_t vdim,
                        int64_t o_part_stride, int64_t o_head_stride,
                        int64_t ml_part_stride, int64_t ml_head_stride,
                        float* out, float* out_ml, void* stream);

/* ------------------------------------------------------------------------- */
/* Sequence shards over several GPUs of one node: exchange of the partials over
 * NVLink peer memory, fused with their merge (no counterpart in the reference,
 * which is single-device).  One process per GPU.  Every rank allocates one
 * exchange buffer of hira_exchange_bytes() with hira_peer_alloc, passes the
 * 64-byte handle to its peers by any host channel, opens theirs with
 * hira_peer_open, and then calls hira_exchange_merge once per decode step
 * after hira_sparse_attn:
 *
 *   local_rows [n_qheads][2 + vdim] fp32: this rank's (m, l, normalised out)
 *              rows -- point hira_sparse_attn's out_ml at row + 0 and out at
 *              row + 2 with head strides of 2 + vdim
 *   peer_bufs  HOST array of `world` device pointers: entry r is rank r's
 *              exchange buffer as mapped in THIS process (entry `rank` is the
 *              pointer hira_peer_alloc returned)
 *   seq        step number, the same on every rank, never 0, +1 per step (a
 *              launch argument: a captured step carries its number, so a graph
 *              holding this call is good for one replay per recording)
 *   phases     3 = push this rank's rows to every peer, wait for every
 *              source's rows, merge (the decode step); 1 = push only,
 *              2 = wait + merge only (for drivers that run several ranks'
 *              kernels on one GPU, where kernels must not wait on each other)
 *   wait_seconds bound of the wait (0 = 2 s); when it runs out *status (device
 *              int32, zeroed by the caller) becomes 1 and `out` is not written
 *   out [n_qheads][vdim], out_ml [n_qheads][2] or NULL: as hira_merge_partials,
 *              whose arithmetic this reproduces bit for bit
 *
 * Buffers are written with plain peer stores; nothing is multicast.  Close the
 * peers' mappings (hira_peer_close) before their owners free them
 * (hira_peer_free), with a host barrier in between. */
#define HIRA_MAX_PEERS 16
#define HIRA_PEER_HANDLE_BYTES 64
int64_t hira_exchange_bytes(int32_t world, int32_t n_qheads, int32_t vdim);
int hira_peer_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle);
int hira_peer_open(const unsigned char* handle, void** dev_ptr);
int hira_peer_close(void* dev_ptr);
int hira_peer_free(void* dev_ptr);
int hira_exchange_merge(const float* local_rows, void* const* peer_bufs,
                        int32_t world, int32_t rank, int32_t n_qheads,
                        int32_t vdim, uint32_t seq, int32_t phases,
                        float wait_seconds, float* out, float* out_ml,
                        int32_t* status, void* stream);

/* ------------------------------------------------------------------------- */
/* Append.  Replaces CUDAIndexer.update (indexer/cuda.py:544-701) and its
 * Triton kernels (kernels/triton_update_kernels.py:6-418) for decode-time
 * insertion: nearest valid parent by ||c||^2 - 2 x.c (ties -> lowest index),
 * slot claim, K/V row write, parent radius widen, grandparent radius widen
 * (indexer/cuda.py:1200-1231); a key whose nearest parent is full becomes a
 * new parent of radius 0 holding itself (the reference's behaviour for one
 * key per head, indexer/cuda.py:730-733,818-820,877-887), placed under its
 * nearest grandparent if that has a free parent slot (:917-962), else under a
 * new grandparent (:1070-1072).  The n_new keys of a head are inserted one
 * after another in order, so the result is deterministic.
 *
 *   new_k [n_heads][n_new][dim], new_v [n_heads][n_new][vdim]: index dtypes,
 *          head strides in elements
 *   token_base: token position of new key 0 is token_base + used[h][2]
 *          when token_base < 0, else token_base + i
 *   status: device int32, OR-ed with HIRA_STATUS_* on capacity exhaustion
 *   workspace: optional scratch of hira_append_workspace_bytes(index, n_new)
 *          bytes (0 = not applicable, for n_new > 32).  With it the parent scan is
 *          spread over the whole GPU (one kernel scans slices, a second one picks
 *          the arg-min and inserts); without it (NULL) one CTA per head does
 *          everything.  The result is identical either way.
 */
size_t hira_append_workspace_bytes(const hira_index_t* index, int32_t n_new);
int hira_append(const hira_index_t* index, const void* new_k, const void* new_v,
                int32_t n_new, int64_t k_head_stride, int64_t v_head_stride,
                int32_t token_base, int32_t* status, void* workspace,
                size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Threshold finder (the reference names sample_max / sample_mean_topk but
 * both raise NotImplementedError, cache/threshold_finder.py:1-14).
 *   samples [n_heads][n_samples][dim] in `dtype`, head stride in elements
 *   tau_out [n_qheads]: method applied to the scores q . sample
 *   n_samples <= 4096;  k in [1, n_samples] for the top-k methods. */
int hira_threshold(const void* samples, int32_t dtype, int32_t n_heads,
                   int32_t n_samples, int32_t dim, int64_t head_stride,
                   const float* q, const int32_t* q2kv, int32_t n_qheads,
                   int32_t method, int32_t k, float* tau_out, void* stream);

/* Search with the next append's parent scan folded in.  A decode step that appends one key
 * per head right after its search reads every parent row twice: once for the search gates, once
 * for the append's nearest-parent scan.  hira_search_scan does both on the single read: while the
 * gates of a tile are computed, the same parent rows are scored against `scan_key` (the key that
 * will be appended) exactly as hira_append scores them, and the best (score, slot) of each head is
 * kept in scan_out by a 64-bit atomicMin.  hira_append_scanned then inserts that key without a scan
 * of its own and resets the slot.  The index must not change between the two calls.  The reference
 * has no counterpart: its update runs its own nearest-parent kernel (kernels/
 * triton_update_kernels.py:6-60).  Default head grouping only (no q2kv).
 *   scan_key [n_heads] rows of `dim` elements in the index dtype, stride in elements
 *   scan_out [n_heads] uint64, all bits set before the first call (hira_append_scanned leaves
 *            it so); holds order-preserving-key(score) << 32 | parent slot                     */
int hira_search_scan(const hira_index_t* index, const float* q, const float* tau,
                     const float* scaling, const float* qnorm, int32_t n_qheads, int32_t flags,
                     int32_t tile_parents, float* out_dense, int32_t* out_idx,
                     float* out_score, int32_t* out_count, uint32_t* stats,
                     const void* scan_key, int64_t scan_key_stride, uint64_t* scan_out, void* stream);
int hira_append_scanned(const hira_index_t* index, const void* new_k, const void* new_v,
                        int64_t k_head_stride, int64_t v_head_stride, int32_t token_base,
                        int32_t* status, uint64_t* scan, void* stream);

/* Query preparation for a decode step: q_hat[qh] = q[qh] / ||q[qh]|| in fp32 and
 * logit_scale[qh] = ||q[qh]|| * sm_scale, i.e. the unit query the tree bound assumes and the
 * `scaling` that turns emitted scores into attention logits (searcher/cpu.py:58-63).
 *   q [n_qheads][dim] in `dtype` (dense). */
int hira_prepare_query(const void* q, int32_t dtype, int32_t n_qheads, int32_t dim,
                       float sm_scale, float* q_hat, float* logit_scale, void* stream);

/* One decode step's attention in one call: hira_prepare_query, hira_search (compact output, gate
 * and leaf rule in `flags`, scores scaled to logits) and hira_sparse_attn, enqueued back to back on
 * `stream`.  It is what a host does per generated token for one layer once the threshold is known
 * (the reference's decode path: cache/hira_cache.py:95-140 -> searcher.search -> attention);
 * folding the three calls into one saves the caller two trips through its FFI.
 *   q [n_qheads][dim] raw queries in `q_dtype`;  tau [n_qheads] on the scale of q_hat . k;
 *   q_hat [n_qheads][dim], logit_scale [n_qheads]: scratch, left holding the prepared query;
 *   idx/score/count, workspace, out, out_ml, queued_*: as in hira_search / hira_sparse_attn;
 *   scan_key, scan_key_stride, scan_out: as in hira_search_scan, or NULL, 0, NULL;
 *   searched: optional cudaEvent_t recorded on `stream` right after the search kernel, so that an
 *            append on another stream can start while the attention still runs (it must not start
 *            earlier: the search reads what the append writes). */
int hira_decode_attention(const hira_index_t* index, const void* q, int32_t q_dtype, float sm_scale,
                          const float* tau, const int32_t* q2kv, int32_t n_qheads, int32_t max_group,
                          int32_t flags, int32_t tile_parents, float* q_hat, float* logit_scale,
                          int32_t* idx, float* score, int32_t* count,
                          const void* queued_k, const void* queued_v, int32_t n_queued,
                          int64_t queued_head_stride, int32_t n_splits, float* workspace,
                          float* out, float* out_ml, int64_t out_head_stride, int64_t ml_head_stride,
                          const void* scan_key, int64_t scan_key_stride, uint64_t* scan_out,
                          void* searched, void* stream);

/* One whole decode step of one layer from HOST buffers, in one call: the copy of the query to the
 * device, query preparation, the threshold (given, or found on the device from the step's
 * samples), search, sparse attention, the copy of the output back to the host and -- when k_host
 * is given -- the 1-key-per-head append, whose host-to-device copies and kernels run on
 * `side_stream` beside the query copy, the search's tail and the attention (it starts when the
 * search has finished; the step ends, on `stream`, when both the output copy and the append are
 * done).  It is the reference's per-token path cache/hira_cache.py:96-153 -> indexer.update,
 * searcher.search (searcher/cuda.py:56-143) -> attention, without a host round trip between the
 * launches.  Nothing is allocated; the caller owns the scratch in hira_step_t and creates its
 * events once with hira_step_events_create.  q_host [n_qheads][dim] in q_dtype, k_host
 * [n_heads][dim] / v_host [n_heads][vdim] in the index dtypes, out_host [n_qheads][vdim] fp32;
 * use pinned host memory, or the copies serialise with the host.  Default head grouping only.
 * The index's active_parents must cover the slots the append may open (see hira_index_t). */
typedef struct hira_step {
    void* q_dev;          /* [n_qheads][dim] in q_dtype                                        */
    void* k_dev;          /* [n_heads][dim] index dtype: the appended key (NULL: never appends) */
    void* v_dev;          /* [n_heads][vdim] values dtype                                      */
    float* q_hat;         /* [n_qheads][dim]                                                   */
    float* logit_scale;   /* [n_qheads]                                                        */
    float* tau;           /* [n_qheads] scratch for a threshold found on the device, or NULL   */
    int32_t* idx;         /* compacted search output, as in hira_search                        */
    float* score;
    int32_t* count;
    float* workspace;     /* n_qheads * n_splits * (vdim + 2) floats                           */
    float* out_dev;       /* [n_qheads][vdim]                                                  */
    uint64_t* scan;       /* [n_heads] all bits set, or NULL.  Non-NULL folds the append's parent
                             scan into the search (hira_search_scan): the search then waits for
                             the key's copy                                                     */
    int32_t* status;      /* device status word of the appends                                 */
    void* append_ws;      /* optional hira_append workspace (scan == NULL)                     */
    size_t append_ws_bytes;
    const void* tau_samples;      /* [n_heads][n_samples][dim] index dtype, for tau_dev == NULL */
    int64_t samples_head_stride;  /* elements between the heads' samples                        */
    int32_t n_samples, tau_method, tau_k;   /* as in hira_threshold                             */
    int32_t n_splits, tile_parents, flags;  /* as in hira_sparse_attn / hira_search             */
    void* ev_copied;      /* cudaEvent_t, set by hira_step_events_create                       */
    void* ev_searched;
    void* ev_appended;
} hira_step_t;
int hira_step_events_create(hira_step_t* step);
int hira_step_events_destroy(hira_step_t* step);
int hira_decode_step(const hira_index_t* index, const hira_step_t* step, const void* q_host,
                     int32_t q_dtype, float sm_scale, int32_t n_qheads, const float* tau_dev,
                     const void* k_host, const void* v_host, float* out_host, void* stream,
                     void* side_stream);

/* Exact k-th largest of the scores in a compacted search output (run
 * hira_search with HIRA_LEAF_CANDIDATES, tau = -inf and scaling = NULL first).
 * k [n_qheads] int32 per-head ranks (1 = largest).  tau_out[qh] = that score,
 * or -inf when fewer than k scores exist. */
int hira_kth_score(const hira_index_t* index, int32_t n_qheads,
                   int32_t tile_parents, const float* score,
                   const int32_t* count, const int32_t* k, float* tau_out,
                   void* stream);

/* ------------------------------------------------------------------------- */
/* Build.  Replaces CUDAIndexer.build (indexer/cuda.py:56-108) with its
 * helpers (:114-538): per level, nearest-centroid assignment, capacity-bf
 * grouping closest-first with overflow into free slots, blocked layout,
 * radii from the layout.  n_iters = 1 assigns once to the sampled points (the
 * reference CUDA behaviour, :229-245); n_iters > 1 runs n_iters-1 Lloyd mean
 * updates first.
 *
 *   keys [n_heads][n_keys][dim], values [n_heads][n_keys][vdim] (index dtypes),
 *          head strides in elements; n_keys <= cap_parents*bf
 *   cent_idx1 [n_heads][ceil(n_keys/bf)] int32: key positions used as initial
 *          parent centres; cent_idx2 [n_heads][ceil(n1/bf)] (depth 3): parent
 *          ids used as initial grandparent centres.  NULL = evenly strided.
 *   The index arrays are (re)initialised: unused slots are zero rows, radius 0, count 0,
 *   slot2token -1.  With index->active_parents == 0 the whole capacity is cleared; with a bound
 *   there (the host vouches that no parent slot beyond it was ever used, and that the arrays
 *   were zero / -1 when allocated) only the slots below max(bound, what this build fills).
 *   balance_rounds: 0 = the reference's rule (every centre keeps its bf closest points, the
 *          overflow is dealt to whatever slots are free).  R > 0 = capacity-aware assignment: the
 *          overflow chooses again, R times, among the centres that still have room (nearest
 *          first, closest points accepted first); only what is left after that is dealt out.
 *          Tighter balls at the price of R more assignment passes; radii as always from the layout.
 *   use_tensor_cores: 1 = tcgen05 assignment GEMM when dtype is bf16 and the
 *          shapes allow it, 0 = CUDA-core fp32 assignment.
 *   status: device int32 or NULL, OR-ed with HIRA_STATUS_ASSIGN_FAILED (see there).
 */
size_t hira_build_workspace_bytes(const hira_index_t* index, int32_t n_keys);
int hira_build(const hira_index_t* index, const void* keys, const void* values,
               int32_t n_keys, int64_t k_head_stride, int64_t v_head_stride,
               int32_t token_base, const int32_t* cent_idx1,
               const int32_t* cent_idx2, int32_t n_iters, int32_t balance_rounds,
               int32_t use_tensor_cores, int32_t* status, void* workspace,
               size_t workspace_bytes, void* stream);

/* Radii recomputed from the layout (indexer/cuda.py:114-198): parent radius =
 * max over filled children of ||child - parent||; grandparent radius = max
 * over filled parents of (||parent - gp|| + parent radius); empty -> 0.  Also
 * refreshes the ||c||^2 caches. */
int hira_recompute_radii(const hira_index_t* index, void* stream);

/* (Re)computes the int8 side copy (per-channel scales, rows, error bounds) from the children as
 * they are stored now: after the index arrays were loaded from elsewhere.  Visits the parent
 * slots below index->active_parents (0 = all). */
int hira_q8_refresh(const hira_index_t* index, void* stream);

/* Diagnostic: the number of CTAs of the int8 pre-filter search on the current
 * device that took their exact fallback (every row of a kept parent re-scored
 * in the index dtype) because one of their bounded waits ran out, since the
 * library was loaded.  Results are unaffected by such an event, the search is
 * only slower; a non-zero count explains an outlier in the step times.
 * Synchronises the device. */
int hira_q8_fallback_count(uint32_t* host_out);

/* Gather the stored keys/values back into token order (slot2token) for a
 * rebuild: out_k [n_heads][n_out][dim]; rows of tokens not present are left
 * untouched.  token_base is subtracted from slot2token.  Visits the parent
 * slots below index->active_parents (0 = all). */
int hira_export(const hira_index_t* index, int32_t token_base, int32_t n_out,
                void* out_k, void* out_v, void* stream);

/* Nearest-centroid assignment on its own (the dense contraction of the build,
 * torch.cdist + argmin at indexer/cuda.py:244-245): for each point the index
 * of the centroid minimising ||c||^2 - 2 x.c (ties -> lowest index) and that
 * minimum plus ||x||^2 clamped at 0 (squared distance).
 *   With use_tensor_cores, a CTA whose bounded wait on its copy / MMA barriers runs out writes
 *   out_idx = -1 (and distance 0) for its 128 points instead of hanging: check for it.
 *   points [n_heads][n][dim], cents [n_heads][k][dim] in `dtype` (dense);
 *   csq_scratch: n_heads*k floats of scratch (receives ||c||^2). */
int hira_assign(const void* points, const void* cents, int32_t dtype,
                int32_t n_heads, int32_t n, int32_t k, int32_t dim,
                int32_t use_tensor_cores, float* csq_scratch, int32_t* out_idx,
                float* out_dist2, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HIRA_B200_H */
