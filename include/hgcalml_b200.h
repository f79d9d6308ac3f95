/*
 * hgcalml_b200 -- C ABI of the sm_100a CUDA library behind the HGCalML custom ops of the
 * GravNet / object-condensation inference path.
 *
 * Conventions
 *  - Every pointer whose name starts with d_ is DEVICE memory; all tensors are dense,
 *    row-major, float32 or int32, exactly as the TensorFlow ops receive them.
 *  - The library allocates nothing that the caller sees: scratch memory is passed in
 *    (`workspace`, sized by the matching *_workspace_bytes query; 256-byte aligned).
 *  - All work is enqueued on `stream` (a cudaStream_t passed as void*); no call
 *    synchronises the device and no call touches the legacy default stream unless the
 *    caller passes it.  The device that owns `stream` and the d_ pointers must be the calling
 *    thread's current device (cudaSetDevice) when an entry is called.  The entries that wait
 *    for their own stream say so: hgc_workspace_status, hgc_binned_select_knn_static_status and
 *    hgc_build_and_assign_condensates when it is asked for the condensate count on the host.
 *  - Return value: HGC_OK or a negative HGC_ERR_* code.  Nothing throws, nothing prints.
 *    Problems that only the device can see (an index outside its table, a bin outside the
 *    grid, an iteration cap reached) set a status word in the workspace, which
 *    hgc_workspace_status() reads back.
 *  - Re-entrant: the only global state is a statistics counter of kernel launches; concurrent
 *    calls need distinct workspaces.  The one exception is hgc_binned_select_knn_static, whose
 *    scratch is a per-device array inside the library (see there).
 *
 * The paths named in the comments are relative to the cms-pepr/HGCalML repository.
 */
#ifndef HGCALML_B200_H
#define HGCALML_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HGC_OK                     0
#define HGC_ERR_INVALID_ARGUMENT  -1   /* shapes / attributes the reference op rejects too        */
#define HGC_ERR_WORKSPACE         -2   /* workspace missing, misaligned or too small              */
#define HGC_ERR_UNSUPPORTED       -3   /* valid for the reference, outside this library's limits  */
#define HGC_ERR_CUDA              -4   /* a CUDA runtime call failed (see hgc_last_cuda_error)     */
#define HGC_ERR_DEVICE_STATUS     -5   /* hgc_workspace_status found a non-zero device status word */
#define HGC_ERR_STATIC_SCRATCH_TOO_SMALL -6 /* problem larger than the built-in scratch of a *_static entry */

/* Bits of the device status word. */
#define HGC_STATUS_BIN_OUT_OF_RANGE    1u  /* a per-dimension bin index fell outside [0, n_bins)   */
#define HGC_STATUS_FLAT_BIN_OVERFLOW   2u  /* a flat bin index was >= the number of bins           */
#define HGC_STATUS_INDEX_OUT_OF_RANGE  4u  /* a gathered index was >= its table size               */
#define HGC_STATUS_ITERATION_CAP       8u  /* an iterative kernel stopped at its iteration cap     */

typedef void *hgc_stream_t; /* cudaStream_t */

const char *hgc_strerror(int code);
/* Text of the last CUDA error seen by the calling thread inside this library. */
const char *hgc_last_cuda_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int hgc_version(void);
/* Number of kernels this library has launched in the calling process so far. */
unsigned long long hgc_launch_count(void);

/* Copies the status word of a workspace used by a previous call on `stream` to *status_out
 * (host) and waits for that stream.  Returns HGC_ERR_DEVICE_STATUS when it is non-zero. */
int hgc_workspace_status(const void *workspace, hgc_stream_t stream, unsigned *status_out);

/* ---------------------------------------------------------------------------------------
 * BinByCoordinates -- replaces BinByCoordinatesOpFunctor
 * (modules/compiled/bin_by_coordinates_kernel.h:9-32, GPU body bin_by_coordinates_kernel.cu.cc:47-165).
 * d_coords [n_vert, n_coords] (already shifted to >= 0), d_row_splits [n_rs], d_bin_width [1],
 * d_n_bins [n_coords]; outputs d_assigned_bin [n_vert, n_coords+1] = [event, c_0 .. c_{n-1}],
 * d_flat_assigned_bin [n_vert], d_n_per_bin [n_total_bins] (zeroed always, filled when
 * calc_n_per_bin).  n_total_bins = prod(n_bins) * (n_rs-1), computed by the caller as the
 * reference's NbinsHelper does (bin_by_coordinates_kernel.cc:17-35).
 * ------------------------------------------------------------------------------------- */
size_t hgc_bin_by_coordinates_workspace_bytes(int n_vert, int n_coords, int n_rs, int n_total_bins);
int hgc_bin_by_coordinates(
        const float *d_coords, const int *d_row_splits, const float *d_bin_width, const int *d_n_bins,
        int *d_assigned_bin, int *d_flat_assigned_bin, int *d_n_per_bin,
        int n_vert, int n_coords, int n_rs, int n_total_bins, int calc_n_per_bin,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * BinnedSelectKnn -- replaces BinnedSelectKnnOpFunctor
 * (modules/compiled/binned_select_knn_kernel.h:8-38, GPU body binned_select_knn_kernel.cu.cc:80-288).
 * All inputs in bin-sorted order: d_coord [n_vert, n_coords], d_bin_idx [n_vert],
 * d_direction [n_vert] (read only when use_direction), d_dim_bin_idx [n_vert, n_bin_dim+1],
 * d_bin_boundaries [n_bboundaries], d_n_bins [n_bin_dim], d_bin_width [1].
 * Outputs d_indices / d_dist [n_vert, n_neigh]: slot 0 is the query itself, slots 1.. hold the
 * n_neigh-1 nearest other hits of the same event in ascending (distance, index) order -- the
 * reference leaves them in scan order; as a set the rows are identical -- padded with -1
 * (or the query's own index when tf_compat) and distance 0.
 * Limits: 2 <= n_bin_dim <= 5, 2 <= n_coords <= 16, 1 <= n_neigh <= 513.
 * Precondition beyond the reference's: d_dim_bin_idx and d_bin_width must be the bins of the
 * leading n_bin_dim columns of d_coord (up to a common shift of the coordinates), which is what
 * BinByCoordinates produces.  From the second shell of bins on, the search leaves out bins whose
 * index distance from the query's bin already puts them beyond the current K-th best; the
 * reference scans every bin of a shell and so tolerates bins that do not match the coordinates.
 * A build with -DHGC_KNN_BINPRUNE=0 scans the reference's full candidate set.
 * ------------------------------------------------------------------------------------- */
size_t hgc_binned_select_knn_workspace_bytes(int n_vert, int n_neigh, int n_coords, int n_bin_dim);
int hgc_binned_select_knn(
        const float *d_coord, const int *d_bin_idx, const int *d_direction, const int *d_dim_bin_idx,
        const int *d_bin_boundaries, const int *d_n_bins, const float *d_bin_width,
        int *d_indices, float *d_dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * BinnedSelectKnn for callers that cannot hand over device memory.  (No counterpart in the
 * reference: there TensorFlow's allocator is always at hand.)
 *
 * Some users of this ABI have no way to obtain a workspace: a plain C or Fortran reconstruction
 * job that links the library directly and owns no device allocator, or a serving process whose
 * framework has claimed the GPU's memory up front, so that a cudaMalloc from inside the op either
 * fails or is forbidden by the deployment's rules.  For them this entry takes the same arguments
 * as hgc_binned_select_knn minus the workspace and computes the same result, keeping its scratch
 * (a status word and the packed coordinates) in a fixed array that is part of the library's device
 * image: 4.25 MiB + 256 bytes on every GPU that loads the library, held until the process exits.
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Limits: n_vert <= HGC_STATIC_KNN_MAX_VERT and n_coords <= HGC_STATIC_KNN_MAX_COORDS, otherwise
 * HGC_ERR_STATIC_SCRATCH_TOO_SMALL is returned and nothing is launched.
 * First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and remembers it; make that first call outside any stream capture.
 * The remembered address belongs to the device's current primary context: after a
 * cudaDeviceReset it is stale, so a process that resets a device must not call this entry on that
 * device again.  The scratch is chosen by the calling thread's current device, which must be the
 * device of `stream` and of the d_ pointers.
 * Sharing: all calls on one device use the same array, which still holds the previous call's
 * data; the entry rewrites what it reads and clears the status word itself, but two calls that
 * overlap on the GPU (different streams, or different host threads) race on it -- serialise them.
 * The same precondition on d_dim_bin_idx / d_bin_width as for hgc_binned_select_knn applies.
 *
 * hgc_binned_select_knn_static_status is this entry's hgc_workspace_status: it copies the status
 * word that the last hgc_binned_select_knn_static call on the current device left in the built-in
 * scratch to *status_out (host memory), waits for `stream`, and returns HGC_ERR_DEVICE_STATUS when
 * the word is non-zero.  It allocates nothing either.
 * ------------------------------------------------------------------------------------- */
#define HGC_STATIC_KNN_MAX_VERT   262144
#define HGC_STATIC_KNN_MAX_COORDS 4
int hgc_binned_select_knn_static(
        const float *d_coord, const int *d_bin_idx, const int *d_direction, const int *d_dim_bin_idx,
        const int *d_bin_boundaries, const int *d_n_bins, const float *d_bin_width,
        int *d_indices, float *d_dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction, hgc_stream_t stream);
int hgc_binned_select_knn_static_status(hgc_stream_t stream, unsigned *status_out);

/* ---------------------------------------------------------------------------------------
 * IndexReplacer -- replaces IndexReplacerOpFunctor (modules/compiled/index_replacer_kernel.h:8-20):
 * replaced[i] = replacements[to_be_replaced[i]], negative entries pass through, entries beyond
 * the table are left unwritten (and flagged in d_status when given; may be NULL).
 * ------------------------------------------------------------------------------------- */
int hgc_index_replacer(
        const int *d_to_be_replaced, const int *d_replacements, int *d_replaced,
        int n_to_be_replaced, int n_replacements, unsigned *d_status, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * AccumulateKnn -- replaces AccumulateKnnOpFunctor
 * (modules/compiled/accumulate_knn_kernel.h:9-29, GPU body accumulate_knn_kernel.cu.cc:23-139).
 * d_weights [n_vert, n_neigh] is the op's `distances` input, used verbatim as a weight;
 * d_feat [n_vert, n_feat]; d_idxs [n_vert, n_neigh] (-1 = skip).  d_out_feat [n_vert, n_out_feat]
 * with n_out_feat = 2*n_feat ([mean | max]) when mean_and_max, else n_feat; d_out_maxidxs
 * [n_vert, n_feat] (written only when mean_and_max; may be NULL to skip it).
 * No workspace.  Sums run over the slots in order, so the mean is bit-identical to the CPU op;
 * the max and its index follow the op's rule (the last slot whose product is >= the running
 * maximum wins, accumulate_knn_kernel.cc:65).  Two corners differ from the CPU loop: a NaN product
 * is ignored by the maximum (the CPU op keeps one that sits in slot 0), and when the maximum is a
 * zero reached by products of both signs its sign bit may differ (+0 here, the later product's
 * there); neither occurs with finite, non-negative weights and features without NaN and -0.
 * Without d_out_maxidxs the arg-max bookkeeping is not run at all (about a third faster).
 * ------------------------------------------------------------------------------------- */
int hgc_accumulate_knn(
        const float *d_weights, const float *d_feat, const int *d_idxs,
        float *d_out_feat, int *d_out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int n_moments, int mean_and_max,
        hgc_stream_t stream);

/* Same op with the weighting of the Python wrapper fused in (modules/accknn_op.py:52):
 * weight = exp(-(distance_scale * d_distances[v,k])), the product rounded to float32 first, so
 * distance_scale = 10 on squared distances is GravNet's AccumulateKnn(10.*distsq, ..)
 * (modules/GravNetLayersRagged.py:3269) and distance_scale = 1 is the wrapper as is.
 * d_order (may be NULL) is a permutation of the hits giving the order in which rows are
 * processed -- results do not depend on it, cache locality does. */
int hgc_accumulate_knn_exp(
        const float *d_distances, const float *d_feat, const int *d_idxs,
        float *d_out_feat, int *d_out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int mean_and_max,
        float distance_scale, const int *d_order, hgc_stream_t stream);

/* The neighbour-collection step of the GravNet layers in one call
 * (modules/GravNetLayersRagged.py:3195-3204 RaggedGravNet.create_output_features and :3587-3600
 * DistanceWeightedMessagePassing.create_output_features): the layers slice the self slot off the
 * kNN output (idx[:,1:], dist[:,1:], :3260), call AccumulateKnn(10.*distsq, features, idx) and take
 * the hit's own features off both halves (features -= tile(prev_feat,[1,2])) before concatenating.
 * Here the slice is an offset and a row stride, the weighting and the subtraction happen in the
 * accumulation kernel, and the result lands in its columns of the caller's concatenation buffer:
 *   d_distances, d_idxs [n_vert, ld_neigh]: slots first_slot .. first_slot+n_neigh-1 are used
 *   d_feat [n_vert, n_feat]
 *   d_out: first of 2*n_feat output columns (mean | max) of a row-major buffer with row stride
 *          ld_out floats
 *   d_out_maxidxs [n_vert, n_feat] or NULL
 *   subtract_self != 0: out[v, f] -= feat[v, f] and out[v, n_feat+f] -= feat[v, f] (one rounding each,
 *          applied to the rounded mean and max, as the separate TF subtraction does). */
int hgc_gravnet_collect(
        const float *d_distances, const int *d_idxs, int ld_neigh, int first_slot, int n_neigh,
        const float *d_feat, float *d_out, int ld_out, int *d_out_maxidxs,
        int n_vert, int n_feat, float distance_scale, int subtract_self, const int *d_order,
        hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * BinnedSelectKnn, wrapper level -- replaces the whole Python function BinnedSelectKnn
 * (modules/binned_select_knn_op.py:32-95: BinByCoordinates + argsort + gathers + the op +
 * IndexReplacer + scatter back) in one call with no host synchronisation.
 * d_coords [n_vert, n_coords] and d_row_splits [n_rs] in the caller's order; outputs
 * d_indices / d_dist [n_vert, n_neigh] in the caller's order and numbering.
 * n_bins <= 0 selects the wrapper's default (binned_select_knn_op.py:59-63).
 * d_sorting_out (may be NULL) receives the bin-sorting permutation [n_vert].
 * ------------------------------------------------------------------------------------- */
size_t hgc_binned_select_knn_ragged_workspace_bytes(int n_vert, int n_neigh, int n_coords, int n_rs,
                                                    int n_bins, int max_bin_dims);
int hgc_binned_select_knn_ragged(
        const float *d_coords, const int *d_row_splits, const int *d_direction,
        int *d_indices, float *d_dist, int *d_sorting_out,
        int n_vert, int n_neigh, int n_coords, int n_rs,
        int n_bins, int max_bin_dims, int tf_compat, int use_direction,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * BinnedAssignToCondensates -- replaces BinnedCondensatesFinderOpFunctor
 * (modules/compiled/binned_assign_to_condensates_kernel.h:8-38; the reference has a CPU body
 * only, binned_assign_to_condensates_kernel.cc:128-241).  Argument order and meaning as the
 * functor's; all arrays in bin-sorted order, *_h are the high-beta subset.  Outputs:
 * d_high_assigned_status_h [n_h] (1 for condensates), d_assignment [n_vert], d_association
 * [n_vert], d_alpha_indices [n_h] (-1 padded per event), d_n_condensates [num_rows+1].
 * ------------------------------------------------------------------------------------- */
size_t hgc_binned_assign_to_condensates_workspace_bytes(int n_vert, int n_vert_h, int num_rows,
                                                        int dimensions);
int hgc_binned_assign_to_condensates(
        int dimensions, int dimensions_binning,
        const float *d_ccoords_h, const float *d_dist_h, const float *d_beta_h,
        const int *d_no_condensation_mask_h,
        int *d_high_assigned_status_h,
        const int *d_original_indices_h, const int *d_row_splits_h,
        const float *d_ccoords, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_indices_to_filtered,
        int *d_assignment, int *d_association, int *d_n_condensates, int *d_alpha_indices,
        const int *d_bin_splits, const int *d_n_bins, const float *d_bin_widths,
        const int *d_row_splits, int num_rows, int n_vert, int n_vert_h, int assign_by_max_beta,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* BuildAndAssignCondensatesBinned, wrapper level -- the Python function of
 * modules/assign_condensate_op.py:210-310 up to (not including) keep_noise: dist / distance_threshold,
 * ccoords -= min over the batch, BinByCoordinates on the first nbin_dims coordinates with
 * n_bins_sc = max(4, min(ceil((n_vert/5)^(1/3)), 25)), stable sort by bin, gathers, the high-beta
 * filter (betas > beta_threshold or mask > 0) with indices_to_filtered / original_indices /
 * row_splits_h, the op, the mapping back to the caller's order, alpha_indices[alpha_indices != -1]
 * and the condensate flags.
 *   inputs, caller's order: d_ccoords [n_vert, dimensions], d_betas, d_dist [n_vert],
 *          d_no_condensation_mask [n_vert] or NULL, d_row_splits [n_rs] (spanning 0 .. n_vert)
 *   outputs: d_assignment, d_association [n_vert]; d_alpha_idx [n_vert]: the condensates' hit ids,
 *          event by event, -1 after the last; d_is_cond [n_vert] bytes (0 / 1);
 *          d_n_condensates [n_rs] cumulative count
 *   h_n_alpha (host, may be NULL): receives the number of condensates; the call then returns after
 *          the stream has finished.
 * The number of high-beta hits never leaves the device (the op's kernels and sorts are launched for
 * up to n_vert of them and read the count themselves), so with h_n_alpha == NULL the call is a plain
 * enqueue like every other entry. */
size_t hgc_build_and_assign_condensates_workspace_bytes(int n_vert, int dimensions, int n_rs, int nbin_dims);
int hgc_build_and_assign_condensates(
        const float *d_ccoords, const float *d_betas, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_row_splits,
        int *d_assignment, int *d_association, int *d_alpha_idx, unsigned char *d_is_cond,
        int *d_n_condensates, int *h_n_alpha,
        int n_vert, int dimensions, int n_rs, float beta_threshold, float distance_threshold,
        int assign_by_max_beta, int nbin_dims,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Backward ops (registered as the gradients of AccumulateKnn and BinnedSelectKnn:
 * modules/accknn_op.py:71-90, modules/binned_select_knn_op.py:107-118).
 *
 * AccumulateKnnGrad -- replaces AccumulateKnnGradOpFunctor
 * (modules/compiled/accumulate_knn_grad_kernel.h:11-34; argument order as there).
 * d_grad_from_out_features [n_vert, n_grad_from_out_feat] with n_grad_from_out_feat = 2*n_feat
 * ([d mean | d max]) when mean_and_max, else n_feat; d_distances = the forward op's weights
 * [n_vert, n_neigh]; d_feat [n_vert, n_feat]; d_max_feat_indices [n_vert, n_feat] (forward output);
 * d_neigh_indices [n_vert, n_neigh].  Outputs d_out_grad_distances [n_vert, n_neigh] (gradient
 * w.r.t. the weights) and d_out_grad_features [n_vert, n_feat].  No atomics: contributions to a
 * hit are summed in (source hit, slot) order, which is the order of the reference's CPU loop.
 *
 * SelectKnnGrad -- replaces SelectKnnGradOpFunctor
 * (modules/compiled/select_knn_grad_kernel.h:15-31): gradient of the squared distances w.r.t. the
 * coordinates, d_grad_coord [n_vert, n_coords]; d_dist is accepted and not read, as in the
 * reference.  Deterministic for the same reason.
 *
 * Both take a workspace of hgc_knn_grad_workspace_bytes (about 24 bytes per (hit, slot) pair) and
 * need n_vert * n_neigh < 2^31.
 * ------------------------------------------------------------------------------------- */
size_t hgc_knn_grad_workspace_bytes(int n_vert, int n_neigh);
int hgc_accumulate_knn_grad(
        const float *d_grad_from_out_features, const float *d_distances, const float *d_feat,
        const int *d_max_feat_indices, const int *d_neigh_indices,
        float *d_out_grad_distances, float *d_out_grad_features,
        int n_vert, int n_neigh, int n_feat, int n_grad_from_out_feat, int n_moments, int mean_and_max,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* The same gradient with a processing order: d_order (may be NULL) is a permutation of the hits,
 * e.g. the bin-sorting permutation that hgc_binned_select_knn_ragged returns.  Results do not depend
 * on it (every target sums its incoming edges in (hit, slot) order); with spatially close hits next
 * to each other the gathered rows of consecutive hits overlap and are found in cache. */
int hgc_accumulate_knn_grad_ordered(
        const float *d_grad_from_out_features, const float *d_distances, const float *d_feat,
        const int *d_max_feat_indices, const int *d_neigh_indices,
        float *d_out_grad_distances, float *d_out_grad_features,
        int n_vert, int n_neigh, int n_feat, int n_grad_from_out_feat, int n_moments, int mean_and_max,
        const int *d_order, void *workspace, size_t workspace_bytes, hgc_stream_t stream);
int hgc_select_knn_grad(
        const float *d_grad_dist, const int *d_indices, const float *d_dist, const float *d_coord,
        float *d_grad_coord, int n_vert, int n_neigh, int n_coords,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Sibling ops on the same neighbour tables (used by the graph-condensation layers).
 *
 * LocalDistance -- replaces LocalDistanceOpFunctor (modules/compiled/local_distance_kernel.h):
 * d_distances[i,k] = squared distance between hit i and hit d_neigh_idxs[i,k]; 0 for -1 and for the
 * hit itself.  d_coords [n_in_vert, n_coords], d_neigh_idxs / d_distances [n_out_vert, n_neigh].
 *
 * PushKnn -- replaces PushKnnOpFunctor (modules/compiled/push_knn_kernel.h):
 * d_out_feat[m,f] = sum over all (i,k) with d_idxs[i,k] == m of d_feat[i,f] * d_weights[i,k], summed
 * in (i,k) order without atomics (bit-identical to the reference's CPU loop).  Workspace:
 * hgc_knn_grad_workspace_bytes(n_vert, n_neigh).
 * ------------------------------------------------------------------------------------- */
int hgc_local_distance(
        const int *d_neigh_idxs, const float *d_coords, float *d_distances,
        int n_coords, int n_in_vert, int n_out_vert, int n_neigh, hgc_stream_t stream);
int hgc_push_knn(
        const float *d_weights, const float *d_feat, const int *d_idxs, float *d_out_feat,
        int n_vert, int n_neigh, int n_feat, void *workspace, size_t workspace_bytes, hgc_stream_t stream);
/* PushKnnGrad -- replaces PushKnnGradOpFunctor (modules/compiled/push_knn_grad_kernel.h; argument order as
 * there): d_feat_grad[i,f] = sum_k d_grad[m_k,f] * d_weights[i,k], d_w_grad[i,k] = sum_f d_grad[m_k,f] *
 * d_feat[i,f], both summed in order.  No workspace. */
int hgc_push_knn_grad(
        const float *d_grad, const float *d_weights, const float *d_feat, const int *d_idxs,
        float *d_feat_grad, float *d_w_grad, int n_vert, int n_neigh, int n_feat, hgc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HGCALML_B200_H */
