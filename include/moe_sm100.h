/*
 * moe_sm100.h -- C ABI of libmoe_sm100.so: the top-k mixture-of-experts expert-compute
 * path of arthurfeeney/moe-explore, written for NVIDIA B200 (sm_100a).
 *
 * The reference project has no FFI: its boundary is the Python functional API
 * (src/moe_explore/functional/topk_moe.py:10-64).  Each entry point below names the
 * reference function (file:line inside the reference project) whose work it performs;
 * the Python package `moe_explore` in this repository calls these through ctypes and
 * keeps the reference's names and signatures.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - the caller owns every allocation; nothing here calls cudaMalloc, except where an
 *     entry point says otherwise;
 *   - every launch is asynchronous on `stream` (a cudaStream_t passed as void*);
 *   - functions return MOE_OK (0) or a negative status; moe_last_error() returns a
 *     thread-local description of the most recent failure;
 *   - `dtype` is MOE_DTYPE_BF16 or MOE_DTYPE_F16 (16-bit inputs, fp32 accumulation);
 *   - `status` (may be NULL) is a device int32 that a kernel sets to a non-zero code when
 *     one of its bounded waits runs out or its metadata is inconsistent (first code wins; the word is
 *     never cleared by a kernel); the host reads it with moe_check_status / moe_read_status.
 *     Callers should check it once per step: after a time-out the outputs of that launch are incomplete.
 *
 * Data layout ("padded expert-sorted rows")
 *   Routed rows (token t, slot s) have flat position j = t*topk + s.  Rows are stably
 *   sorted by expert; expert e's rows occupy padded rows [pad_offsets[e], pad_offsets[e+1]),
 *   a range rounded up to a multiple of MOE_TILE_M so that no 128-row GEMM tile spans two
 *   experts.  Padding rows hold zeros and have row_src == -1.  Every [RP, *] activation
 *   buffer uses this layout, RP = moe_padded_rows_bound(R, E).
 */
#ifndef MOE_SM100_H_
#define MOE_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_OK 0
#define MOE_ERR_INVALID (-1)     /* bad argument (null pointer, negative size, misaligned) */
#define MOE_ERR_UNSUPPORTED (-2) /* shape or device this library does not handle */
#define MOE_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed; see moe_last_error() */
#define MOE_ERR_TIMEOUT (-4)     /* a device-side bounded wait ran out (from moe_check_status) */

#define MOE_DTYPE_BF16 0
#define MOE_DTYPE_F16 1
#define MOE_DTYPE_F32 2 /* accepted by moe_router_topk only */

#define MOE_ACT_NONE 0
#define MOE_ACT_SILU 1
#define MOE_ACT_GELU 2   /* exact erf form */
#define MOE_ACT_SWIGLU 3 /* silu(even column) * odd column */
#define MOE_ACT_GEGLU 4  /* gelu(even column) * odd column */
#define MOE_ACT_GELU_TANH 5 /* tanh form of gelu ("approx_gelu", triton_kernels/activation.py:9-14) */

#define MOE_TILE_M 128

/* Thread-local text of the last error reported by this library (never NULL). */
const char* moe_last_error(void);

/* Device query: SM count and compute capability of `device`.  Replaces
 * gpu_utils.get_gpu_sm_count (src/moe_explore/gpu_utils.py:4-8).  Returns
 * MOE_ERR_UNSUPPORTED when the device is not compute capability 10.x. */
int moe_query_device(int device, int* sm_count, int* cc_major, int* cc_minor);

/* Reads a device status word (synchronises `stream`).  MOE_OK; MOE_ERR_INVALID for an expert id out of range
 * (code 100) or metadata that does not fit the call (code 5); MOE_ERR_TIMEOUT for a wait that ran out (codes 1-3:
 * outputs incomplete; code 4: only the wave barrier of a grouped GEMM gave up, its results are valid). */
int moe_check_status(const int32_t* status, void* stream);

/* Copies the status word into *code (host) and, when reset != 0, clears the word afterwards; synchronises `stream`. */
int moe_read_status(const int32_t* status, int32_t* code, int reset, void* stream);

/* Limit, in SM clock cycles, of every device-side wait in the launches that follow (process-wide; cycles <= 0
 * restores the default of 2^32, about two seconds).  A wait that runs out makes its kernel set the status word,
 * let the copies in flight land, free its tensor memory and return by itself.  No counterpart in the reference. */
int moe_set_wait_limit_cycles(int64_t cycles);

/* Upper bounds used to size buffers without reading routing results on the host:
 * padded row count RP (a multiple of MOE_TILE_M) and number of 128-row tiles. */
int64_t moe_padded_rows_bound(int64_t num_rows, int num_experts);
int64_t moe_mtiles_bound(int64_t num_rows, int num_experts);

/* ---------------------------------------------------------------------------------
 * Router tail in one launch: logits [T, E] -> (fp32 softmax over E when softmax_before_topk) -> top-k ->
 * (softmax over the k selected logits otherwise) -> (division by the sum of the k when normalize) -> scores [T, k]
 * in the logits' dtype, indices int64 [T, k], and the per-expert histogram expert_counts int32 [E] (may be NULL).
 * Replaces the softmax / torch.topk / softmax / cast launches of topk_router (src/moe_explore/router.py:17-35); the
 * logits GEMM stays with the caller.  Declared tie rule (torch.topk's is unspecified): equal values are taken in
 * ascending expert index, the k results come in descending value order, NaN is never selected.  One warp per
 * token; E <= 1024, k <= 32.  dtype: MOE_DTYPE_BF16 / F16 / F32.
 * --------------------------------------------------------------------------------- */
int moe_router_topk(const void* logits, void* scores, int64_t* indices, int32_t* expert_counts,
                    int64_t num_tokens, int num_experts, int topk, int softmax_before_topk,
                    int normalize, int dtype, void* stream);

/* ---------------------------------------------------------------------------------
 * (a) Routing metadata.  Replaces get_token_indices (src/moe_explore/expert_permute.py:19-41):
 * argsort of the flattened expert ids, per-expert histogram, prefix sum.  The sort here is
 * the STABLE counting sort (equal experts keep flat-position order).
 *   expert_idx    int64 [R]      expert id of flat position j (R = T*topk)
 *   group_indices int32 [E+1]    exclusive prefix sum of per-expert counts
 *   perm          int64 [R]      perm[r] = flat position of the r-th row in expert order
 *   pad_offsets   int32 [E+1]    padded row offset of each expert (multiples of MOE_TILE_M)
 *   row_src       int32 [RP]     flat position held by padded row p, or -1 for padding
 *   dst_row       int32 [R]      padded row that holds flat position j (inverse of row_src)
 *   mtile_expert  int32 [moe_mtiles_bound]  expert of each 128-row tile
 *   tile_pairs    int32 [moe_mtiles_bound + E + 1]  row tiles grouped in pairs of the same expert
 *                                (two row tiles share one weight tile on a pair of SMs): entry p = first
 *                                tile (bits 0-19) | expert (bits 20-30) | bit 31 when tile+1 is in
 *                                the pair too; from index moe_mtiles_bound on, the exclusive prefix of
 *                                the per-expert pair counts ([E+1] entries)
 *   num_mtiles    int32 [4]      {128-row tiles in use, tile pairs in use, moe_mtiles_bound(R, E), 0}
 * Any of perm / row_src / dst_row / (mtile_expert, tile_pairs, num_mtiles) may be NULL to skip it.
 * ids outside [0, E) are rejected on the device: such rows are in no expert's segment, their
 * dst_row entry and the unused tail of perm are -1 (every consumer here skips negative rows) and
 * `status` is set to 100.  Workspace: moe_routing_workspace_bytes(R, E) bytes.
 * --------------------------------------------------------------------------------- */
size_t moe_routing_workspace_bytes(int64_t num_rows, int num_experts);
int moe_routing_metadata(const int64_t* expert_idx, int64_t num_rows, int num_experts,
                         int32_t* group_indices, int64_t* perm, int32_t* pad_offsets,
                         int32_t* row_src, int32_t* dst_row, int32_t* mtile_expert,
                         int32_t* tile_pairs, int32_t* num_mtiles, int32_t* status,
                         void* workspace, size_t workspace_bytes, void* stream);

/* The same computation for callers that cannot allocate device memory (fixed arenas, plugin
 * hosts that hand an operator only its inputs and outputs, loops that must stay off the
 * allocator): the scratch is a 1 MiB array built into the library image, present on every GPU
 * that loads it.  Inputs and outputs are still the caller's.  It has no counterpart in the
 * reference.  Limits: moe_routing_workspace_bytes(num_rows, num_experts) must not exceed
 * moe_routing_static_scratch_bytes() (e.g. 524288 rows x 256 experts fits exactly), otherwise
 * MOE_ERR_UNSUPPORTED.  All calls on one device share the array, so calls that overlap on the
 * GPU race; the array needs no clearing between calls.  The first call on each device resolves
 * the array's device address and should be made outside stream capture. */
size_t moe_routing_static_scratch_bytes(void);
int moe_routing_metadata_static(const int64_t* expert_idx, int64_t num_rows, int num_experts,
                                int32_t* group_indices, int64_t* perm, int32_t* pad_offsets,
                                int32_t* row_src, int32_t* dst_row, int32_t* mtile_expert,
                                int32_t* tile_pairs, int32_t* num_mtiles, int32_t* status,
                                void* stream);

/* Same outputs from an existing exclusive prefix `group_indices` [E+1] (rows already in
 * expert order, identity permutation): used by the plain ragged grouped GEMM
 * (m_grouped_gemm with gather=scatter=False, triton_kernels/m_grouped_gemm.py:332-393).
 * row_src[p] is the unpadded row index.  A prefix that is not monotone from 0 to num_rows sets `status`
 * (may be NULL) to 5; the offending segments get no rows. */
int moe_layout_from_groups(const int32_t* group_indices, int64_t num_rows, int num_experts,
                           int32_t* pad_offsets, int32_t* row_src, int32_t* dst_row,
                           int32_t* mtile_expert, int32_t* tile_pairs, int32_t* num_mtiles,
                           int32_t* status, void* stream);

/* Copies `bytes` (a multiple of 8) from device memory to PAGE-LOCKED host memory with a kernel that stores through
 * the unified address space, asynchronously on `stream`; the host reads the buffer after synchronising the stream.
 * For the small host reads of a step (expert-parallel split sizes): a cudaMemcpy of a few hundred bytes is queued on
 * a copy engine behind any large host transfer another stream has in flight there, and measured a whole
 * read-back (18-48 ms) of delay per step; a kernel store is not.  No counterpart in the reference. */
int moe_store_to_host(const void* src, void* dst_pinned_host, size_t bytes, void* stream);

/* ---------------------------------------------------------------------------------
 * Row movement (HBM-bound).  Replace row_gather / row_scatter
 * (triton_kernels/row_gather_scatter.py:36-116) and scale_and_reduce
 * (functional/scale_and_reduce.py:3-5).
 * --------------------------------------------------------------------------------- */

/* dst[p, :] = src[row_src[p] / div, :] for padded rows p < 128*num_mtiles, zeros where
 * row_src[p] < 0.  div = topk gathers token rows; div = 1 gathers flat-position rows. */
int moe_gather_rows(const void* src, int64_t src_rows, const int32_t* row_src,
                    const int32_t* num_mtiles, void* dst, int64_t padded_rows, int cols,
                    int div, int dtype, void* stream);

/* The layer's dispatch, token-major: dst[dst_row[t*topk + s], :] = src[t, :] for every token t and slot s
 * (each token row is read once and written topk times), padding rows (row_src[p] < 0, p < 128*num_mtiles)
 * are zeroed.  Same result as moe_gather_rows with div = topk.  Slots with dst_row < 0 are skipped. */
int moe_dispatch_rows(const void* src, const int32_t* dst_row, const int32_t* row_src,
                      const int32_t* num_mtiles, void* dst, int64_t num_tokens, int topk,
                      int64_t padded_rows, int cols, int dtype, void* stream);

/* Expert-parallel dispatch as a pull: dst[p, :] = scale[p] * peer_bases[src_rank[p]][src_row[p], :]
 * for padded rows p < 128*num_mtiles, zeros where src_rank[p] < 0.  peer_bases is a DEVICE array with
 * one base pointer per rank of the node (peer-mapped buffers of [*, cols] rows, e.g. symmetric memory);
 * rows are read with ordinary loads over NVLink.  scale (fp32, may be NULL) is applied in fp32.
 * chunk_count > 1 restricts the call to the rows of the experts [E*chunk_index/chunk_count,
 * E*(chunk_index+1)/chunk_count) (see moe_mgrouped_gemm); chunk_count < 0 selects the explicit expert range
 * [chunk_index, -chunk_count) instead; pair_end > pair_begin selects the rows of the row-tile pairs
 * [pair_begin, pair_end) of the pair list (the slice moe_gemm_options.pair_begin / pair_end names); tile_pairs and
 * num_experts are needed for all three.
 * bulk_ctas > 0 selects the copy-engine kernel on that many CTAs (one per SM that is free for it): every warp
 * moves whole rows with cp.async.bulk through a shared-memory slot, which keeps ~170 KB of remote reads in
 * flight per SM; bulk_ctas == 0 selects the load/store kernel: spread over all SMs in 128-thread CTAs that also fit
 * beside a GEMM CTA (dedicated_ctas == 0), or as dedicated_ctas CTAs of 1024 threads, each of which has an SM to
 * itself (the caller keeps that many SMs free of GEMM CTAs with moe_gemm_options.max_ctas).
 * No counterpart in the reference (it is single-GPU). */
int moe_gather_rows_peer(const void* const* peer_bases, const int32_t* src_rank,
                         const int32_t* src_row, const float* scale, const int32_t* num_mtiles,
                         const int32_t* tile_pairs, int num_experts, int chunk_index,
                         int chunk_count, int pair_begin, int pair_end, void* dst, int64_t padded_rows,
                         int cols, int dtype, int bulk_ctas, int dedicated_ctas, int32_t* status,
                         void* stream);

/* Expert-parallel dispatch on the copy engines: `count` independent device-to-device copies (host arrays of
 * destination addresses, source addresses -- typically blocks of peers' buffers -- and sizes), each issued as one
 * plain asynchronous memcpy on `stream`.  When every source has sorted its rows by destination expert, the rows an
 * expert receives from one source are one contiguous block on both sides, so the whole dispatch is E_local x ranks
 * such copies and no SM touches a row.  moe_zero_padding_rows zeroes the rows of the padded layout that no copy
 * fills (row_src < 0).  No counterpart in the reference. */
int moe_copy_blocks(void* const* dst, const void* const* src, const size_t* bytes, int count, void* stream);
int moe_zero_padding_rows(const int32_t* row_src, const int32_t* num_mtiles, void* dst,
                          int64_t padded_rows, int cols, int dtype, void* stream);

/* out[j, :] = src[dst_row[j], :] for j < R: padded layout back to flat-position order (zeros where
 * dst_row[j] < 0). */
int moe_unpad_rows(const void* src, const int32_t* dst_row, void* out, int64_t num_rows,
                   int cols, int dtype, void* stream);

/* out[t, :] = sum_s scale(t,s) * ys[dst_row[t*topk+s], :], fp32 accumulation, one rounding.
 * scores: [T, topk] in `dtype`, or NULL for scale 1 (used for dX). */
int moe_combine_topk(const void* ys, const void* scores, const int32_t* dst_row, void* out,
                     int64_t num_tokens, int topk, int cols, int dtype, void* stream);

/* Backward of the combine: for padded row p holding flat position j = (t, s):
 *   gs[p, :]   = scores[j] * dout[t, :]
 *   dscores[j] = dot(dout[t, :], ys[p, :])      (fp32 accumulation, stored in `dtype`)
 * padding rows of gs are zeroed.  gs may be NULL when only dscores is wanted. */
int moe_combine_bwd(const void* dout, const void* scores, const void* ys,
                    const int32_t* row_src, const int32_t* num_mtiles, void* gs, void* dscores,
                    int64_t num_tokens, int topk, int64_t padded_rows, int cols, int dtype,
                    void* stream);

/* ---------------------------------------------------------------------------------
 * (b),(c),(d) Grouped GEMMs on tcgen05 tensor cores (TMA operand tiles, TMEM accumulators,
 * persistent tile loop).  Replace m_grouped_gemm and its fused epilogues
 * (triton_kernels/m_grouped_gemm.py:33-267, epilogue_split.py:4-44,
 * triton_kernels/activation.py:5-36).  All row counts are in the padded layout.
 * Requirements: every column count a multiple of 8; pointers 16-byte aligned.
 * --------------------------------------------------------------------------------- */

/* Per-launch options of the grouped GEMMs (host struct; NULL or zeros = the library's choices).
 *   max_ctas      cap on the CTAs of the launch (the kernels are persistent: a cap of sm_count - n leaves n SMs
 *                 free for a kernel on another stream); 0 = one CTA per SM
 *   wave_sync     0 = library's choice (on for K >= 8192), 1 = on, -1 = off: the persistent workers start each
 *                 work item together, which keeps shared operand tiles in L2.  The barrier presumes all workers
 *                 resident; a worker whose wait (~1 ms) runs out carries on unsynchronised and sets status 4
 *   wave_workers  arrivals per wave the barrier waits for; 0 = the launch's worker count (anything larger can
 *                 never be reached: the documented way to exercise the time-out path)
 *   group_m       row units per scheduling group; 0 = default (12)
 *   align_experts 0 = library's choice, 1 / -1 = scheduling groups never / may span two experts
 *   single_cta    0 = library's choice (CTA pairs, unless the experts average at most one 128-row tile: one-SM
 *                 kernels then stream the weights faster), 1 = one-SM kernels, -1 = CTA pairs
 *   separate_copies 1 = fetch every 64-column block of an N-contiguous operand tile with a copy of its own instead
 *                 of one copy over a blocked view of the matrix (which needs the column count to be a multiple
 *                 of 64 and is otherwise the default): for comparison measurements
 *   lane_stores   1 = output tiles in the padded layout are written with 16-byte stores by the lanes instead of bulk
 *                 tensor stores from the staging tile (the default when the column count is a multiple of 64): for
 *                 comparison measurements
 *   expert_begin, expert_end  M-grouped kernels: when end > begin, process exactly the experts [begin, end) (needs
 *                 tile_pairs); overrides chunk_index / chunk_count.  Lets a caller cut the expert list into slices
 *                 of unequal size, e.g. by row counts
 *   pair_begin, pair_end  M-grouped kernels: when end > begin, process exactly the row-tile pairs [begin, end) of the
 *                 pair list (needs tile_pairs); overrides the expert range.  Slices of this kind may cut through an
 *                 expert: what the expert-parallel pipeline needs when one expert holds most of a rank's rows.  Pair p
 *                 of the list covers the 128-row tiles tile_pairs[p] & 0xFFFFF and, if bit 31 is set, the next one
 *   wave_counter  device word for the barrier's arrivals, zeroed by the call on `stream`; NULL = a slot of the
 *                 library's own ring (shared by all streams: a clash only costs a launch its barrier) */
typedef struct moe_gemm_options {
  int32_t max_ctas;
  int32_t wave_sync;
  int32_t wave_workers;
  int32_t group_m;
  int32_t align_experts;
  int32_t single_cta;
  int32_t separate_copies;
  int32_t lane_stores;
  int32_t expert_begin;
  int32_t expert_end;
  int32_t pair_begin;
  int32_t pair_end;
  uint32_t* wave_counter;
} moe_gemm_options;

/* sizeof(moe_gemm_options) as this library was built: lets a binding written in another language check its own
 * declaration of the struct. */
size_t moe_gemm_options_size(void);

/* M-grouped: out = epilogue(a[rows of tile] @ w[expert of tile]).
 *   mtile_expert / tile_pairs / num_mtiles come from moe_routing_metadata; tile_pairs may be
 *   NULL, which selects the one-SM-per-tile kernels instead of the paired-SM ones.
 *   padded_rows must be the moe_padded_rows_bound value the metadata was built with (the pair prefix is
 *   found at tile_pairs[padded_rows / 128]; a mismatch with num_mtiles[2] sets status 5 and computes nothing).
 *   chunk_count > 1 processes only the experts [E*chunk_index/chunk_count, E*(chunk_index+1)/chunk_count)
 *   (needs tile_pairs): a caller can run the row movement of chunk c+1 on another stream while the GEMMs
 *   of chunk c run.  chunk_count <= 1 processes everything.
 *   a    [RP, K]
 *   w    [E, K, N] when w_transposed == 0, [E, N, K] when w_transposed == 1
 *   act  MOE_ACT_NONE/SILU/GELU/GELU_TANH: out [RP, N];  MOE_ACT_SWIGLU/GEGLU: out [RP, N/2].
 *        When pre_act != NULL (and act != MOE_ACT_NONE), pre_act [RP, N] receives the un-activated
 *        product, which moe_mgrouped_gemm_dglu needs in the backward pass. */
int moe_mgrouped_gemm(const void* a, const void* w, void* out, void* pre_act,
                      const int32_t* mtile_expert, const int32_t* tile_pairs,
                      const int32_t* num_mtiles,
                      int64_t padded_rows, int K, int N, int num_experts, int w_transposed,
                      int act, int dtype, int chunk_index, int chunk_count,
                      const moe_gemm_options* options, int32_t* status, void* stream);

/* The same contraction with the row gather fused into the operand loads (the GATHER_ROWS branch of the
 * reference kernel, triton_kernels/m_grouped_gemm.py:104-109): padded row p reads row row_src[p] / div of
 * src [src_rows, K] (zeros where row_src[p] < 0), fetched four rows at a time by tile::gather4 tensor copies;
 * no [RP, K] copy of the rows exists.  w is [E, K, N].  src must be this GPU's own memory. */
int moe_mgrouped_gemm_gather(const void* src, int64_t src_rows, const int32_t* row_src, int div,
                             const void* w, void* out, void* pre_act, const int32_t* mtile_expert,
                             const int32_t* tile_pairs, const int32_t* num_mtiles,
                             int64_t padded_rows, int K, int N, int num_experts, int act, int dtype,
                             const moe_gemm_options* options, int32_t* status, void* stream);

/* The contraction with the top-k fold fused into the epilogue (the SCATTER_ROWS branch of the reference kernel,
 * triton_kernels/m_grouped_gemm.py:168-172, plus functional/scale_and_reduce.py:3-5): accumulator row p
 * (flat position j = row_src[p], skipped when negative) is multiplied by scores[j] (scale 1 when scores is NULL)
 * and ADDED to row j / topk of out [T, N] with 16-byte vector reductions.  out must be zero when the call
 * starts.  The k summands of a token are rounded to `dtype` one by one and arrive in no fixed order, so results
 * are not bit-reproducible; moe_mgrouped_gemm + moe_combine_topk is the deterministic form. */
int moe_mgrouped_gemm_combine(const void* a, const void* w, void* out, const int32_t* row_src,
                              const void* scores, int topk, const int32_t* mtile_expert,
                              const int32_t* tile_pairs, const int32_t* num_mtiles,
                              int64_t padded_rows, int K, int N, int num_experts, int w_transposed,
                              int dtype, const moe_gemm_options* options, int32_t* status,
                              void* stream);

/* The contraction with the row scatter fused into the epilogue (the SCATTER_ROWS branch of the reference kernel,
 * triton_kernels/m_grouped_gemm.py:168-172): accumulator row p, after an optional element-wise activation
 * (MOE_ACT_NONE/SILU/GELU/GELU_TANH), is stored at row out_rows[p] of out [*, N] (skipped when out_rows[p] < 0),
 * whole 128-byte row segments per store.  The input rows may be gathered by the loads at the same time:
 * a_row_src != NULL reads row a_row_src[p] / a_div of a [a_rows, K] (zeros where negative) as in
 * moe_mgrouped_gemm_gather; a_row_src == NULL takes a as [RP, K] in the padded layout (a_rows, a_div ignored). */
int moe_mgrouped_gemm_scatter(const void* a, int64_t a_rows, const int32_t* a_row_src, int a_div,
                              const void* w, void* out, const int32_t* out_rows,
                              const int32_t* mtile_expert, const int32_t* tile_pairs,
                              const int32_t* num_mtiles, int64_t padded_rows, int K, int N,
                              int num_experts, int w_transposed, int act, int dtype,
                              const moe_gemm_options* options, int32_t* status, void* stream);

/* Expert-parallel combine fused into the GEMM: the same contraction as moe_mgrouped_gemm without an
 * activation, but the epilogue stores accumulator row p at row dest_row[p] of the [*, N] matrix based at
 * peer_bases[dest_rank[p]] -- the buffer of the GPU that owns the token -- with ordinary stores over
 * NVLink, tile by tile while the next tile's math runs; rows with dest_rank[p] < 0 are skipped.
 * peer_bases is a DEVICE array of one base pointer per rank.  The caller synchronises the ranks before
 * the destination buffers are read.  No counterpart in the reference. */
int moe_mgrouped_gemm_push(const void* a, const void* w, void* const* peer_bases,
                           const int32_t* dest_rank, const int32_t* dest_row,
                           const int32_t* mtile_expert, const int32_t* tile_pairs,
                           const int32_t* num_mtiles, int64_t padded_rows, int K, int N,
                           int num_experts, int w_transposed, int dtype, int chunk_index,
                           int chunk_count, const moe_gemm_options* options, int32_t* status,
                           void* stream);

/* Backward through the activation: d_pre = act'(pre_act) * (g[RP, K] @ w[E, N, K]^T),
 * i.e. for the layer: g = score-scaled dOut rows, w = weight2 [E, I, d] (N = I, K = d),
 * pre_act = the product saved by the forward GEMM.
 *   MOE_ACT_SWIGLU / MOE_ACT_GEGLU: pre_act and d_pre are [RP, 2N] (gate, up interleaved);
 *   MOE_ACT_SILU / MOE_ACT_GELU / MOE_ACT_GELU_TANH: pre_act and d_pre are [RP, N].
 * No counterpart in the reference (it has no backward). */
int moe_mgrouped_gemm_dglu(const void* g, const void* w, const void* pre_act, void* d_pre,
                           const int32_t* mtile_expert, const int32_t* tile_pairs,
                           const int32_t* num_mtiles,
                           int64_t padded_rows, int K, int N, int num_experts, int act,
                           int dtype, int chunk_index, int chunk_count,
                           const moe_gemm_options* options, int32_t* status, void* stream);

/* K-grouped (expert weight gradients): dw[e] = a[rows of e]^T @ b[rows of e],
 *   a [RP, M], b [RP, N], dw [E, M, N]; experts without rows get zeros.
 * No counterpart in the reference (it has no backward). */
int moe_kgrouped_gemm(const void* a, const void* b, void* dw, const int32_t* pad_offsets,
                      int64_t padded_rows, int M, int N, int num_experts, int dtype,
                      const moe_gemm_options* options, int32_t* status, void* stream);

/* The same with the rows of `a` gathered by the operand loads: padded row p contributes row row_src[p] / div
 * of src [src_rows, M] (nothing where row_src[p] < 0).  Used for the gradient of weight1, whose `a` is the
 * layer input in token order. */
int moe_kgrouped_gemm_gather(const void* src, int64_t src_rows, const int32_t* row_src, int div,
                             const void* b, void* dw, const int32_t* pad_offsets,
                             int64_t padded_rows, int M, int N, int num_experts, int dtype,
                             const moe_gemm_options* options, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_SM100_H_ */
