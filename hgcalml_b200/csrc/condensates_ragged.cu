// Wrapper-level BuildAndAssignCondensatesBinned: the tensor glue of modules/assign_condensate_op.py:245-310
// around the op (threshold scaling, shift by the batch minimum, BinByCoordinates, sort by bin, gathers,
// the high-beta filter with its index maps, the op, the mapping back and the condensate flags) as one
// call on the device.  The one value the host needs in between is the number of high-beta hits (it
// sizes the op's filtered inputs, as the boolean masks do in the reference); it is read back once.
#include "common.cuh"
#include "binning.cuh"
#include "../../include/hgcalml_b200.h"

namespace hgc {
namespace {

constexpr int kMaxCondDims = 8;

// Sorted position i takes hit perm[i]: coordinates shifted by the batch minimum of every dimension
// (ccoords -= reduce_min(ccoords, axis=0)), distance over the threshold, mask, and the high-beta flag
// (betas > beta_threshold or mask > 0).
__global__ void gather_sorted_kernel(const float *__restrict__ ccoords, const float *__restrict__ betas,
                                     const float *__restrict__ dist, const int *__restrict__ mask,
                                     const int *__restrict__ perm, const GridParams *__restrict__ grid,
                                     int dims, float distance_threshold, float beta_threshold,
                                     float *__restrict__ s_ccoords, float *__restrict__ s_betas,
                                     float *__restrict__ s_dist, int *__restrict__ s_mask,
                                     int *__restrict__ high, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int src = perm[i];
    for (int c = 0; c < dims; c++)
        s_ccoords[(size_t)i * dims + c] = __fsub_rn(ccoords[(size_t)src * dims + c], grid->all_min[c]);
    const float b = betas[src];
    const int m = mask ? mask[src] : 0;
    s_betas[i] = b;
    s_dist[i] = __fdiv_rn(dist[src], distance_threshold);
    s_mask[i] = m;
    high[i] = (b > beta_threshold || m > 0) ? 1 : 0;
}

// high_excl = exclusive prefix sum of the flags.  Writes indices_to_filtered, the filtered copies,
// and the filtered row splits; total[0] = number of high-beta hits.
__global__ void compact_high_kernel(const int *__restrict__ high_excl, const float *__restrict__ s_ccoords,
                                    const float *__restrict__ s_betas, const float *__restrict__ s_dist,
                                    const int *__restrict__ s_mask, const int *__restrict__ perm, int dims,
                                    float beta_threshold, int *__restrict__ itf, float *__restrict__ h_ccoords,
                                    float *__restrict__ h_betas, float *__restrict__ h_dist,
                                    int *__restrict__ h_mask, int *__restrict__ h_orig, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const bool is_high = s_betas[i] > beta_threshold || s_mask[i] > 0;
    const int pos = high_excl[i];
    itf[i] = is_high ? pos : -1;
    if (!is_high) return;
    for (int c = 0; c < dims; c++) h_ccoords[(size_t)pos * dims + c] = s_ccoords[(size_t)i * dims + c];
    h_betas[pos] = s_betas[i];
    h_dist[pos] = s_dist[i];
    h_mask[pos] = s_mask[i];
    h_orig[pos] = perm[i];
}

__global__ void filtered_row_splits_kernel(const int *__restrict__ high_excl, const float *__restrict__ s_betas,
                                           const int *__restrict__ s_mask, float beta_threshold,
                                           const int *__restrict__ row_splits, int n_rs, int n,
                                           int *__restrict__ row_splits_h, int *__restrict__ total)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e > n_rs) return;
    int all = 0;
    if (n > 0) all = high_excl[n - 1] + ((s_betas[n - 1] > beta_threshold || s_mask[n - 1] > 0) ? 1 : 0);
    if (e == n_rs) { total[0] = all; return; }
    const int r = row_splits[e];
    row_splits_h[e] = r >= n ? all : (r <= 0 ? 0 : high_excl[r]);
}

// Back to the caller's order: out[perm[i]] = sorted[i].
__global__ void scatter_back_kernel(const int *__restrict__ s_assignment, const int *__restrict__ s_asso,
                                    const int *__restrict__ perm, int *__restrict__ assignment,
                                    int *__restrict__ asso, unsigned char *__restrict__ is_cond, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int dst = perm[i];
    assignment[dst] = s_assignment[i];
    asso[dst] = s_asso[i];
    is_cond[i] = 0;
}

// alpha_indices[alpha_indices != -1], and the flags of those hits.  Within an event's filtered range
// the op lists the condensates first and pads with -1, so entry a of event e moves to
// n_condensates[e] + (a - row_splits_h[e]).
__global__ void compact_alpha_kernel(const int *__restrict__ alpha_h, const int *__restrict__ row_splits_h,
                                     const int *__restrict__ n_condensates, int num_rows, int n_h_max,
                                     const int *__restrict__ n_h_dev,
                                     int *__restrict__ alpha_out, unsigned char *__restrict__ is_cond)
{
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= min(n_h_max, *n_h_dev)) return;
    const int id = alpha_h[a];
    if (id < 0) return;
    int lo = 1, hi = num_rows + 1;  // event = number of row_splits_h[1..num_rows] that are <= a
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_splits_h[mid] <= a) lo = mid + 1; else hi = mid;
    }
    const int e = lo - 1;
    alpha_out[n_condensates[e] + (a - row_splits_h[e])] = id;
    is_cond[id] = 1;
}

__global__ void fill_minus_one_kernel(int *__restrict__ p, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = -1;
}

struct Plan {
    int cb;
    long long max_bins;
    int n_bins_sc;
};

// n_bins_sc of the wrapper (assign_condensate_op.py:265-266) and an upper bound on the grid's size.
bool make_plan(int n_vert, int dims, int nbin_dims, int n_rs, Plan *p)
{
    p->cb = dims < nbin_dims ? dims : nbin_dims;
    if (p->cb < 1 || p->cb > kMaxBinDims) return false;
    int nb = (int)ceil(pow((double)n_vert / 5., 1. / 3.));
    nb = nb > 25 ? 25 : nb;
    nb = nb < 4 ? 4 : nb;
    p->n_bins_sc = nb;
    long long b = n_rs > 1 ? n_rs - 1 : 1;
    for (int d = 0; d < p->cb; d++) {
        b *= nb + 1;
        if (b > (1LL << 30)) return false;
    }
    p->max_bins = b;
    return true;
}

struct Buffers {
    GridParams *grid;
    float *partial;
    int *keys, *skeys, *perm, *tk, *tv, *hist, *high, *scan_tmp, *itf, *s_mask, *h_mask, *h_orig;
    int *row_splits_h, *total, *s_assignment, *s_asso, *alpha_h, *status_h;
    float *s_ccoords, *s_betas, *s_dist, *h_ccoords, *h_betas, *h_dist;
    void *op_ws;
    size_t op_ws_bytes;
};

template <typename W>
void layout(W &ws, int n_vert, int dims, int num_rows, Buffers *out)
{
    const size_t n = n_vert > 0 ? n_vert : 0;
    const size_t d = dims > 0 ? dims : 1;
    Buffers b;
    b.grid = ws.template take<GridParams>(1);
    b.partial = ws.template take<float>((size_t)range_partial_blocks(n_vert) * 2 * kMaxBinDims);
    b.keys = ws.template take<int>(n);
    b.skeys = ws.template take<int>(n);
    b.perm = ws.template take<int>(n);
    b.tk = ws.template take<int>(n);
    b.tv = ws.template take<int>(n);
    b.hist = ws.template take<int>(sort_hist_ints(n_vert));
    b.high = ws.template take<int>(n);
    b.scan_tmp = ws.template take<int>(scan_scratch_ints(n_vert));
    b.itf = ws.template take<int>(n);
    b.s_mask = ws.template take<int>(n);
    b.h_mask = ws.template take<int>(n);
    b.h_orig = ws.template take<int>(n);
    b.row_splits_h = ws.template take<int>((size_t)num_rows + 1);
    b.total = ws.template take<int>(1);
    b.s_assignment = ws.template take<int>(n);
    b.s_asso = ws.template take<int>(n);
    b.alpha_h = ws.template take<int>(n);
    b.status_h = ws.template take<int>(n);
    b.s_ccoords = ws.template take<float>(n * d);
    b.s_betas = ws.template take<float>(n);
    b.s_dist = ws.template take<float>(n);
    b.h_ccoords = ws.template take<float>(n * d);
    b.h_betas = ws.template take<float>(n);
    b.h_dist = ws.template take<float>(n);
    b.op_ws_bytes = hgc_binned_assign_to_condensates_workspace_bytes(n_vert, n_vert, num_rows, dims);
    b.op_ws = ws.template take<unsigned char>(b.op_ws_bytes);
    if (out) *out = b;
}

struct SizerW {
    Sizer s;
    template <typename T> T *take(size_t n) { s.take<T>(n); return nullptr; }
};

}  // namespace
}  // namespace hgc

namespace hgc {
int assign_to_condensates(
        int dimensions, int dimensions_binning,
        const float *d_ccoords_h, const float *d_dist_h, const float *d_beta_h,
        const int *d_no_condensation_mask_h, int *d_high_assigned_status_h,
        const int *d_original_indices_h, const int *d_row_splits_h,
        const float *d_ccoords, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_indices_to_filtered,
        int *d_assignment, int *d_association, int *d_n_condensates, int *d_alpha_indices,
        const int *d_bin_splits, const int *d_n_bins, const float *d_bin_widths,
        const int *d_row_splits, int num_rows, int n_vert, int n_vert_h, const int *d_n_vert_h,
        int assign_by_max_beta, void *workspace, size_t workspace_bytes, hgc_stream_t stream);
}
using namespace hgc;

extern "C" size_t hgc_build_and_assign_condensates_workspace_bytes(int n_vert, int dimensions, int n_rs,
                                                                   int nbin_dims)
{
    Plan p;
    if (dimensions < 1 || dimensions > kMaxCondDims || n_rs < 1 || !make_plan(n_vert, dimensions, nbin_dims, n_rs, &p))
        return 0;
    SizerW w;
    layout(w, n_vert, dimensions, n_rs - 1, nullptr);
    return w.s.used;
}

extern "C" int hgc_build_and_assign_condensates(
        const float *d_ccoords, const float *d_betas, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_row_splits,
        int *d_assignment, int *d_association, int *d_alpha_idx, unsigned char *d_is_cond,
        int *d_n_condensates, int *h_n_alpha,
        int n_vert, int dimensions, int n_rs, float beta_threshold, float distance_threshold,
        int assign_by_max_beta, int nbin_dims,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // argument rules of the wrapper (assign_condensate_op.py:245-247)
    if (n_vert < 0 || n_rs < 1 || dimensions < 1 || nbin_dims < 1 || nbin_dims > 6) return HGC_ERR_INVALID_ARGUMENT;
    if (!(beta_threshold >= 0.f && beta_threshold <= 1.f) || !(distance_threshold > 0.f)) return HGC_ERR_INVALID_ARGUMENT;
    if (dimensions > kMaxCondDims) return HGC_ERR_UNSUPPORTED;
    Plan p;
    if (!make_plan(n_vert, dimensions, nbin_dims, n_rs, &p)) return HGC_ERR_UNSUPPORTED;
    const int num_rows = n_rs - 1;
    if (!d_n_condensates || !d_row_splits) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert > 0 && (!d_ccoords || !d_betas || !d_dist || !d_assignment || !d_association || !d_alpha_idx || !d_is_cond))
        return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_build_and_assign_condensates_workspace_bytes(n_vert, dimensions, n_rs, nbin_dims);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    Buffers b;
    layout(ws, n_vert, dimensions, num_rows, &b);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    if (h_n_alpha) *h_n_alpha = 0;
    if (n_vert == 0) {
        HGC_CUDA_TRY(cudaMemsetAsync(d_n_condensates, 0, sizeof(int) * (size_t)n_rs, stream));
        return HGC_OK;
    }

    // grid of BinByCoordinates(ccoords[:, :nbin_dims] - min, n_bins=n_bins_sc, pre_normalized=True), keys, order
    if (int rc = compute_grid(d_ccoords, dimensions, p.cb, dimensions, n_vert, d_row_splits, n_rs, p.n_bins_sc,
                              32, /*pre_normalized=*/0, b.partial, b.grid, stream))
        return rc;
    if (int rc = launch_bin_keys(d_ccoords, dimensions, p.cb, b.grid->shift, d_row_splits, n_rs,
                                 &b.grid->bin_width, b.grid->n_bins, nullptr, nullptr, b.keys, n_vert, 0,
                                 &b.grid->n_total_bins, ws.status(), stream))
        return rc;
    if (int rc = sort_pairs(b.keys, nullptr, b.skeys, b.perm, b.tk, b.tv, b.hist, n_vert, bits_for(p.max_bins), stream))
        return rc;
    const int blocks = div_up(n_vert, 256);
    gather_sorted_kernel<<<blocks, 256, 0, stream>>>(d_ccoords, d_betas, d_dist, d_no_condensation_mask, b.perm,
                                                     b.grid, dimensions, distance_threshold, beta_threshold,
                                                     b.s_ccoords, b.s_betas, b.s_dist, b.s_mask, b.high, n_vert);
    HGC_LAUNCH_CHECK();
    if (int rc = exclusive_scan_ints(b.high, n_vert, b.scan_tmp, stream)) return rc;
    compact_high_kernel<<<blocks, 256, 0, stream>>>(b.high, b.s_ccoords, b.s_betas, b.s_dist, b.s_mask, b.perm,
                                                    dimensions, beta_threshold, b.itf, b.h_ccoords, b.h_betas,
                                                    b.h_dist, b.h_mask, b.h_orig, n_vert);
    HGC_LAUNCH_CHECK();
    filtered_row_splits_kernel<<<div_up(n_rs + 1, 256), 256, 0, stream>>>(b.high, b.s_betas, b.s_mask, beta_threshold,
                                                                          d_row_splits, n_rs, n_vert,
                                                                          b.row_splits_h, b.total);
    HGC_LAUNCH_CHECK();
    // The number of high-beta hits stays on the device: the op is launched for up to n_vert of them
    // and reads the count itself, so nothing waits for the host here.
    if (int rc = assign_to_condensates(
                dimensions, p.cb, b.h_ccoords, b.h_dist, b.h_betas, b.h_mask, b.status_h, b.h_orig, b.row_splits_h,
                b.s_ccoords, b.s_dist, b.s_mask, b.itf, b.s_assignment, b.s_asso, d_n_condensates, b.alpha_h,
                nullptr, b.grid->n_bins, &b.grid->bin_width, d_row_splits, num_rows, n_vert, n_vert, b.total,
                assign_by_max_beta, b.op_ws, b.op_ws_bytes, stream_))
        return rc;

    scatter_back_kernel<<<blocks, 256, 0, stream>>>(b.s_assignment, b.s_asso, b.perm, d_assignment, d_association,
                                                    d_is_cond, n_vert);
    HGC_LAUNCH_CHECK();
    fill_minus_one_kernel<<<blocks, 256, 0, stream>>>(d_alpha_idx, n_vert);
    HGC_LAUNCH_CHECK();
    compact_alpha_kernel<<<blocks, 256, 0, stream>>>(b.alpha_h, b.row_splits_h, d_n_condensates, num_rows, n_vert,
                                                     b.total, d_alpha_idx, d_is_cond);
    HGC_LAUNCH_CHECK();
    if (h_n_alpha) {
        HGC_CUDA_TRY(cudaMemcpyAsync(h_n_alpha, d_n_condensates + num_rows, sizeof(int), cudaMemcpyDeviceToHost, stream));
        HGC_CUDA_TRY(cudaStreamSynchronize(stream));
    }
    return HGC_OK;
}
