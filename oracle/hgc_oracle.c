/*
 * TEST INFRASTRUCTURE ONLY -- a plain-C, single-threaded restatement of the
 * CPU algorithms of the HGCalML custom ops on the GravNet / object-condensation
 * inference path.  It exists so the CUDA library can be checked on machines
 * that have no HGCalML checkout; it is validated against the reference's own
 * compiled CPU kernels and against committed golden vectors by the CPU test
 * suite.  Only tests, the smoke check and the CPU-baseline leg of the bench may
 * load it; the product never does.
 *
 * Every function names the reference file:line it restates (paths relative to
 * the cms-pepr/HGCalML repository).  Build with -ffp-contract=off: the float
 * expressions below must round exactly as written.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define HGC_MAX_BIN_DIMS 8

/* ------------------------------------------------------------------------
 * BinByCoordinates
 * restates modules/compiled/bin_by_coordinates_kernel.cc:36-114 (set_defaults + calc).
 * coords are already shifted to be >= 0 by the Python wrapper.  The LAST
 * coordinate is the fastest-varying digit of the flat index, the event
 * (row-split) index the slowest.  Out-of-range per-dimension indices are
 * forced to 0; a flat index beyond the bin count leaves the hit's outputs
 * untouched.  n_per_bin is always zeroed, filled only on request.
 * ---------------------------------------------------------------------- */
void oracle_bin_by_coordinates(
        const float *coords, const int *row_splits, const float *bin_width, const int *n_bins,
        int *assigned_bin, int *flat_assigned_bin, int *n_per_bin,
        int n_vert, int n_coords, int n_rs, int n_total_bins, int calc_n_per_bin)
{
    for (int b = 0; b < n_total_bins; b++) n_per_bin[b] = 0;

    const float bw = bin_width[0];
    int event = 0; /* row splits ascend, so the event of hit v is found incrementally */
    for (int v = 0; v < n_vert; v++) {
        int stride = 1, flat = 0;
        for (int c = n_coords - 1; c >= 0; c--) {
            int ci = (int)(coords[(size_t)v * n_coords + c] / bw);
            if (ci < 0 || ci >= n_bins[c]) ci = 0;
            assigned_bin[(size_t)v * (n_coords + 1) + c + 1] = ci;
            flat += ci * stride;
            stride *= n_bins[c];
        }
        /* number of row_splits[1..n_rs-1] that are <= v, stopping at the first larger one */
        while (event + 1 < n_rs && row_splits[event + 1] <= v) event++;
        flat += event * stride;
        if (flat >= n_total_bins) continue;
        assigned_bin[(size_t)v * (n_coords + 1)] = event;
        flat_assigned_bin[v] = flat;
        if (calc_n_per_bin) n_per_bin[flat] += 1;
    }
}

/* ------------------------------------------------------------------------
 * BinnedSelectKnn
 * restates modules/compiled/binned_select_knn_kernel.cc:19-196 together with
 * the shell walker modules/compiled/binstepper.h:11-97.
 *
 * All inputs are in bin-sorted order.  Row layout of the outputs: slot 0 is
 * the query itself; slots 1.. are filled in scan order, afterwards the slot
 * holding the current largest distance is overwritten whenever a strictly
 * closer candidate shows up, and the largest is searched again over slots
 * 1..K-1 (first slot among equals).  Shells of bins at Chebyshev distance
 * d = 0,1,2,.. around the query's bin are visited in cube order (dimension 0
 * slowest); the search stops after a shell with no bin inside the grid, or
 * once the row is full and ((bw*d)*bw)*d exceeds the largest kept distance.
 * ---------------------------------------------------------------------- */
static float oracle_distsq(const float *a, const float *b, int n_coords)
{
    float s = 0.f;
    for (int c = 0; c < n_coords; c++) {
        float t = a[c] - b[c];
        s += t * t;
    }
    return s;
}

int oracle_binned_select_knn(
        const float *coord, const int *bin_idx, const int *direction, const int *dim_bin_idx,
        const int *bin_boundaries, const int *n_bins, const float *bin_width,
        int *indices, float *dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction)
{
    if (n_bin_dim < 1 || n_bin_dim > HGC_MAX_BIN_DIMS) return -1;
    const int K = n_neigh;
    const float bw = bin_width[0];

    int bins_per_event = 1;
    for (int d = 0; d < n_bin_dim; d++) bins_per_event *= n_bins[d];

    for (int i = 0; i < n_vert; i++) {
        int *row_i = indices + (size_t)i * K;
        float *row_d = dist + (size_t)i * K;
        for (int s = 0; s < K; s++) {
            row_i[s] = (s == 0 || tf_compat) ? i : -1;
            row_d[s] = 0.f;
        }
    }

    for (int i = 0; i < n_vert; i++) {
        if (use_direction && (direction[i] == 0 || direction[i] == 2)) continue;

        int *row_i = indices + (size_t)i * K;
        float *row_d = dist + (size_t)i * K;
        const int *qbin = dim_bin_idx + (size_t)i * (n_bin_dim + 1) + 1;
        const int event_offset = bins_per_event * (bin_idx[i] / bins_per_event);

        int filled = 1, worst_slot = 0;
        float worst = 0.f;

        for (int shell = 0;; shell++) {
            int any_bin_in_grid = 0;
            int off[HGC_MAX_BIN_DIMS];
            for (int d = 0; d < n_bin_dim; d++) off[d] = -shell;

            for (;;) {
                /* (a) only the surface of the cube, (b) only bins inside the grid */
                int on_surface = 0, inside = 1, flat = 0, stride = 1;
                for (int d = n_bin_dim - 1; d >= 0; d--) {
                    int a = off[d] < 0 ? -off[d] : off[d];
                    if (a == shell) on_surface = 1;
                    int g = qbin[d] + off[d];
                    if (g < 0 || g >= n_bins[d]) inside = 0;
                    flat += g * stride;
                    stride *= n_bins[d];
                }
                if (on_surface && inside && flat >= 0 && flat < bins_per_event) {
                    int b = flat + event_offset;
                    if (b < n_bboundaries - 1) {
                        any_bin_in_grid = 1;
                        for (int j = bin_boundaries[b]; j < bin_boundaries[b + 1]; j++) {
                            if (j == i) continue;
                            if (use_direction && (direction[j] == 1 || direction[j] == 2)) continue;
                            float dsq = oracle_distsq(coord + (size_t)i * n_coords,
                                                      coord + (size_t)j * n_coords, n_coords);
                            if (filled < K) {
                                row_i[filled] = j;
                                row_d[filled] = dsq;
                                if (dsq > worst) { worst = dsq; worst_slot = filled; }
                                filled++;
                            } else if (dsq < worst) {
                                row_i[worst_slot] = j;
                                row_d[worst_slot] = dsq;
                                worst = 0.f;
                                worst_slot = 0;
                                for (int s = 1; s < K; s++)
                                    if (row_d[s] > worst) { worst = row_d[s]; worst_slot = s; }
                            }
                        }
                    }
                }
                /* next offset vector, last dimension fastest */
                int d = n_bin_dim - 1;
                while (d >= 0 && off[d] == shell) { off[d] = -shell; d--; }
                if (d < 0) break;
                off[d]++;
            }

            if (!any_bin_in_grid) break;
            if (filled == K && bw * shell * bw * shell > worst) break;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * IndexReplacer
 * restates modules/compiled/index_replacer_kernel.cc:28-41: negative entries
 * pass through, entries beyond the table are left unwritten.
 * ---------------------------------------------------------------------- */
void oracle_index_replacer(const int *to_be_replaced, const int *replacements, int *replaced,
                           int n_to_be_replaced, int n_replacements)
{
    for (int i = 0; i < n_to_be_replaced; i++) {
        int r = to_be_replaced[i];
        if (r < 0) replaced[i] = r;
        else if (r < n_replacements) replaced[i] = replacements[r];
    }
}

/* ------------------------------------------------------------------------
 * AccumulateKnn
 * restates modules/compiled/accumulate_knn_kernel.cc:27-83.  "weights" is the
 * op's `distances` input, used verbatim as a multiplicative weight.  The sum
 * runs over the slots in order and is divided by K (not by the number of
 * valid slots).  The maximum starts from 0, is reset by slot 0 when slot 0 is
 * valid, and a later slot wins ties (>=).
 * ---------------------------------------------------------------------- */
void oracle_accumulate_knn(
        const float *weights, const float *feat, const int *idxs,
        float *out_feat, int *out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int mean_and_max)
{
    for (int v = 0; v < n_vert; v++) {
        const int *nb = idxs + (size_t)v * n_neigh;
        const float *w = weights + (size_t)v * n_neigh;
        for (int f = 0; f < n_feat; f++) {
            float sum = 0.f, best = 0.f;
            int best_id = 0;
            for (int s = 0; s < n_neigh; s++) {
                int j = nb[s];
                if (j < 0) continue;
                float t = feat[(size_t)j * n_feat + f] * w[s];
                sum += t;
                if (mean_and_max && (t >= best || s == 0)) { best = t; best_id = j; }
            }
            out_feat[(size_t)v * n_out_feat + f] = sum / (float)n_neigh;
            if (mean_and_max) {
                out_feat[(size_t)v * n_out_feat + n_feat + f] = best;
                out_maxidxs[(size_t)v * n_feat + f] = best_id;
            }
        }
    }
}

/* ------------------------------------------------------------------------
 * BinnedAssignToCondensates
 * restates modules/compiled/binned_assign_to_condensates_kernel.cc:23-241 and
 * the box walker modules/compiled/binstepper.h:100-165.
 *
 * Per event: repeatedly pick, among the high-beta ("_h") hits not yet claimed,
 * the one with the largest beta (first among equals); it becomes the next
 * condensate and claims hits inside its radius, found by scanning the bins
 * that overlap its bounding box in the binned dimensions.  The box walker
 * forms flat bin indices from per-dimension indices that may lie outside the
 * grid and only rejects flat indices outside [0, bins_per_event).
 *
 * The pick loop tests no_condensation_mask_h at position (row_offset_h+iv_h > 0),
 * i.e. at 0 or 1, exactly as the reference does.
 * Returns -1 where the reference would throw (no progress), else 0.
 * ---------------------------------------------------------------------- */
int oracle_binned_assign_to_condensates(
        int dims, int dims_binning,
        int *claimed_h,
        const float *ccoords_h, const float *dist_h, const float *beta_h,
        const int *mask_h,
        int *is_condensate_h,
        const int *original_indices_h, const int *row_splits_h,
        const float *ccoords, const float *dist, const int *mask,
        const int *indices_to_filtered,
        float *min_distance,
        int *assignment, int *association, int *n_condensates, int *alpha_indices,
        const int *bin_splits, const int *n_bins, const float *bin_widths,
        const int *row_splits, int num_rows, int assign_by_max_beta)
{
    (void)dist;
    if (dims_binning < 1 || dims_binning > HGC_MAX_BIN_DIMS) return -2;
    const float bw = bin_widths[0];
    int bins_per_event = 1;
    for (int d = 0; d < dims_binning; d++) bins_per_event *= n_bins[d];

    n_condensates[0] = 0;
    int running_total = 0;
    float *centre = (float *)malloc(sizeof(float) * (size_t)(dims > 0 ? dims : 1));

    for (int r = 0; r < num_rows; r++) {
        const int off = row_splits[r], n = row_splits[r + 1] - row_splits[r];
        const int off_h = row_splits_h[r], n_h = row_splits_h[r + 1] - row_splits_h[r];
        const int *event_bin_splits = bin_splits + (size_t)bins_per_event * r;

        for (int i = 0; i < n_h; i++) {
            is_condensate_h[off_h + i] = 0;
            claimed_h[off_h + i] = 0;
            alpha_indices[off_h + i] = -1;
        }
        for (int i = 0; i < n; i++) {
            assignment[off + i] = -1;
            association[off + i] = -1;
            if (!assign_by_max_beta) min_distance[off + i] = 10e20;
        }

        int shower = 0, previous = -1;
        for (;;) {
            float top_beta = -1.f;
            int alpha = -1;
            for (int i = 0; i < n_h; i++) {
                if (claimed_h[off_h + i] != 0) continue;
                if (mask_h[(off_h + i) > 0]) { alpha = i; top_beta = 0.f; break; }
                if (beta_h[off_h + i] > top_beta) { top_beta = beta_h[off_h + i]; alpha = i; }
            }
            if (top_beta == -1.f) break;
            if (alpha == previous) { free(centre); return -1; }
            previous = alpha;

            const int a = off_h + alpha;
            float radius = dist_h[a];
            const float radius_sq = radius * radius;
            for (int d = 0; d < dims; d++) centre[d] = ccoords_h[(size_t)a * dims + d];
            int lonely = 0;
            if (mask_h[a] > 0) { radius = 0.f; lonely = 1; }

            int lo[HGC_MAX_BIN_DIMS], span[HGC_MAX_BIN_DIMS], n_box = 1;
            for (int d = 0; d < dims_binning; d++) {
                lo[d] = (int)floorf((centre[d] - radius) / bw);
                int hi = (int)ceilf((centre[d] + radius) / bw);
                span[d] = hi - lo[d] + 1;
                n_box *= span[d];
            }
            is_condensate_h[a] = 1;
            claimed_h[a] = 1;

            for (int step = 0; step < n_box; step++) {
                int flat = 0, stride = 1, rem = step;
                for (int d = dims_binning - 1; d >= 0; d--) {
                    flat += (lo[d] + rem % span[d]) * stride;
                    rem /= span[d];
                    stride *= n_bins[d];
                }
                if (flat < 0 || flat >= bins_per_event) continue;

                for (int v = event_bin_splits[flat]; v < event_bin_splits[flat + 1]; v++) {
                    if (assign_by_max_beta && assignment[v] != -1) continue;
                    float dsq = 0.f;
                    for (int d = 0; d < dims; d++) {
                        float t = centre[d] - ccoords[(size_t)v * dims + d];
                        dsq += t * t;
                    }
                    int inside = (dsq <= radius_sq && !lonely && mask[v] == 0) ||
                                 (lonely && indices_to_filtered[v] == a);
                    if (!inside) continue;
                    if (!assign_by_max_beta) {
                        if (!(min_distance[v] * radius_sq >= dsq)) continue;
                        min_distance[v] = dsq;
                    }
                    assignment[v] = shower;
                    association[v] = original_indices_h[a];
                    if (indices_to_filtered[v] != -1) claimed_h[indices_to_filtered[v]] = 1;
                }
            }

            alpha_indices[off_h + shower] = original_indices_h[a];
            shower++;
        }
        running_total += shower;
        n_condensates[r + 1] = running_total;
    }
    free(centre);
    return 0;
}

/* ------------------------------------------------------------------------
 * AccumulateKnnGrad
 * restates modules/compiled/accumulate_knn_grad_kernel.cc:25-163.
 * Feature gradient: every (hit i, slot k) with neighbour m adds
 *   (g[i,f] / K) * w[i,k]  +  [m == arg-max neighbour of (i,f)] * gmax[i,f] * w[i,k]
 * to grad_feat[m,f]; when the arg-max neighbour is the hit itself only its first
 * occurrence in the row counts.  Contributions arrive in (i, k) order.
 * Weight gradient: grad_w[i,k] = (sum_f g[i,f] * feat[m,f]) * (1/K in double)
 *   + sum_f [m == arg-max neighbour of (i,f)] * gmax[i,f] * feat[m,f].
 * ---------------------------------------------------------------------- */
void oracle_accumulate_knn_grad(
        const float *grad_out, const float *weights, const float *feat,
        const int *max_idx, const int *nidx,
        float *grad_weights, float *grad_feat,
        int n_vert, int n_neigh, int n_feat, int n_grad_out, int mean_and_max)
{
    for (size_t t = 0; t < (size_t)n_vert * n_feat; t++) grad_feat[t] = 0.f;

    for (int i = 0; i < n_vert; i++) {
        for (int f = 0; f < n_feat; f++) {
            const float g = grad_out[(size_t)i * n_grad_out + f];
            float gmax = 0.f;
            int amax = -1;
            if (mean_and_max) {
                gmax = grad_out[(size_t)i * n_grad_out + n_feat + f];
                amax = max_idx[(size_t)i * n_feat + f];
            }
            int self_seen = 0;
            for (int k = 0; k < n_neigh; k++) {
                const int m = nidx[(size_t)i * n_neigh + k];
                if (m < 0) continue;
                const float w = weights[(size_t)i * n_neigh + k];
                const float mean_part = g / (float)n_neigh * w;
                float max_part = 0.f;
                if (m == amax) {
                    if (m != i) max_part = gmax * w;
                    else if (!self_seen) { max_part = gmax * w; self_seen = 1; }
                }
                grad_feat[(size_t)m * n_feat + f] += mean_part + max_part;
            }
        }
    }

    for (int i = 0; i < n_vert; i++) {
        for (int k = 0; k < n_neigh; k++) {
            const int m = nidx[(size_t)i * n_neigh + k];
            if (m < 0) { grad_weights[(size_t)i * n_neigh + k] = 0.f; continue; }
            float mean_part = 0.f, max_part = 0.f;
            for (int f = 0; f < n_feat; f++) {
                const float g = grad_out[(size_t)i * n_grad_out + f];
                const float x = feat[(size_t)m * n_feat + f];
                mean_part += g * x * 1.f;
                if (mean_and_max && m == max_idx[(size_t)i * n_feat + f])
                    max_part += grad_out[(size_t)i * n_grad_out + n_feat + f] * x * 1.f;
            }
            mean_part *= 1. / (float)n_neigh;
            grad_weights[(size_t)i * n_neigh + k] = mean_part + max_part;
        }
    }
}

/* ------------------------------------------------------------------------
 * SelectKnnGrad
 * The reference's CPU functor for this op is empty
 * (modules/compiled/select_knn_grad_kernel.cc:24-42); this restates its GPU kernels
 * (modules/compiled/select_knn_grad_kernel.cu.cc:81-165):
 *   grad_x[i,c]  = - sum_k 2 * g[i,k] * (x[m,c] - x[i,c])          (accumulated in the reference's mixed
 *                                                                  float/double arithmetic, k ascending)
 *   grad_x[m,c] +=   (float)(2 * g[i,k] * (x[m,c] - x[i,c]))       for every (i,k) with neighbour m.
 * The reference adds the second part with atomics in no fixed order; here it is added in (i, k) order.
 * PARITY UNPINNED: no reference CPU code exists to run; checked against the analytic gradient instead.
 * ---------------------------------------------------------------------- */
void oracle_select_knn_grad(
        const float *grad_dist, const int *nidx, const float *coord, float *grad_coord,
        int n_vert, int n_neigh, int n_coords)
{
    for (int i = 0; i < n_vert; i++)
        for (int c = 0; c < n_coords; c++) {
            const float xi = coord[(size_t)i * n_coords + c];
            float self = 0.f;
            for (int k = 0; k < n_neigh; k++) {
                const int m = nidx[(size_t)i * n_neigh + k];
                if (m < 0 || m >= n_vert) continue;
                const float g = grad_dist[(size_t)i * n_neigh + k];
                const float xm = coord[(size_t)m * n_coords + c];
                self -= 2. * g * (xm - xi);
            }
            grad_coord[(size_t)i * n_coords + c] = self;
        }
    for (int i = 0; i < n_vert; i++)
        for (int k = 0; k < n_neigh; k++) {
            const int m = nidx[(size_t)i * n_neigh + k];
            if (m < 0 || m >= n_vert) continue;
            const float g = grad_dist[(size_t)i * n_neigh + k];
            for (int c = 0; c < n_coords; c++) {
                const float add = 2. * g * (coord[(size_t)m * n_coords + c] - coord[(size_t)i * n_coords + c]);
                grad_coord[(size_t)m * n_coords + c] += add;
            }
        }
}

/* ------------------------------------------------------------------------
 * LocalDistance
 * restates modules/compiled/local_distance_kernel.cc:22-70: squared distance from
 * every hit to each of its listed neighbours (0 for padding and for the hit itself).
 * ---------------------------------------------------------------------- */
void oracle_local_distance(const int *nidx, const float *coords, float *dist,
                           int n_coords, int n_in_vert, int n_out_vert, int n_neigh)
{
    (void)n_in_vert;
    for (int i = 0; i < n_out_vert; i++)
        for (int k = 0; k < n_neigh; k++) {
            const int j = nidx[(size_t)i * n_neigh + k];
            float d = 0.f;
            if (j >= 0 && j != i)
                d = oracle_distsq(coords + (size_t)i * n_coords, coords + (size_t)j * n_coords, n_coords);
            dist[(size_t)i * n_neigh + k] = d;
        }
}

/* ------------------------------------------------------------------------
 * PushKnn
 * restates modules/compiled/push_knn_kernel.cc:35-71: every hit adds its weighted
 * features to each of its neighbours, out[m,f] += feat[i,f] * w[i,k], in (i, k) order.
 * ---------------------------------------------------------------------- */
void oracle_push_knn(const float *weights, const float *feat, const int *nidx, float *out,
                     int n_vert, int n_neigh, int n_feat)
{
    for (size_t t = 0; t < (size_t)n_vert * n_feat; t++) out[t] = 0.f;
    for (int i = 0; i < n_vert; i++)
        for (int f = 0; f < n_feat; f++) {
            const float x = feat[(size_t)i * n_feat + f];
            for (int k = 0; k < n_neigh; k++) {
                const int m = nidx[(size_t)i * n_neigh + k];
                if (m < 0) continue;
                out[(size_t)m * n_feat + f] += x * weights[(size_t)i * n_neigh + k];
            }
        }
}

/* ------------------------------------------------------------------------
 * PushKnnGrad
 * restates modules/compiled/push_knn_grad_kernel.cc:22-95:
 *   feat_grad[i,f] = sum_k grad[m_k,f] * w[i,k]      (k ascending)
 *   w_grad[i,k]    = sum_f grad[m_k,f] * feat[i,f]   (f ascending; 0 for padding)
 * ---------------------------------------------------------------------- */
void oracle_push_knn_grad(const float *grad, const float *weights, const float *feat, const int *nidx,
                          float *feat_grad, float *w_grad, int n_vert, int n_neigh, int n_feat)
{
    for (int i = 0; i < n_vert; i++)
        for (int f = 0; f < n_feat; f++) {
            float acc = 0.f;
            for (int k = 0; k < n_neigh; k++) {
                const int m = nidx[(size_t)i * n_neigh + k];
                if (m < 0) continue;
                acc += grad[(size_t)m * n_feat + f] * weights[(size_t)i * n_neigh + k];
            }
            feat_grad[(size_t)i * n_feat + f] = acc;
        }
    for (int i = 0; i < n_vert; i++)
        for (int k = 0; k < n_neigh; k++) {
            const int m = nidx[(size_t)i * n_neigh + k];
            float acc = 0.f;
            if (m >= 0)
                for (int f = 0; f < n_feat; f++)
                    acc += grad[(size_t)m * n_feat + f] * feat[(size_t)i * n_feat + f];
            w_grad[(size_t)i * n_neigh + k] = acc;
        }
}
