// Wrapper-level BinnedSelectKnn: the whole Python function of modules/binned_select_knn_op.py:32-95
// (grid from the batch's coordinate range, BinByCoordinates, stable sort by bin, gathers, the
// neighbour search, index remap and scatter back to the caller's order) as one enqueue with no
// host round trip.  The search writes each row straight to the caller's row and numbering, which
// replaces IndexReplacer and the two scatter_nd calls.
#include "common.cuh"
#include "binning.cuh"
#include "select_knn.cuh"

namespace hgc {
namespace {

__global__ void gather_rows_kernel(const int *__restrict__ src, int width, const int *__restrict__ perm,
                                   int *__restrict__ dst, int n)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)n * width) return;
    const int i = (int)(t / width), c = (int)(t % width);
    dst[t] = src[(size_t)perm[i] * width + c];
}

struct RaggedPlan {
    int cb;              // binned dimensions
    long long max_bins;  // upper bound on the number of bins of the device-derived grid
};

bool make_plan(int n_coords, int n_rs, int n_bins, int max_bin_dims, RaggedPlan *p)
{
    p->cb = max_bin_dims < n_coords ? max_bin_dims : n_coords;
    if (p->cb < 1 || p->cb > kMaxBinDims) return false;
    // bins per dimension = int(extent/width + 1) <= n_bins + 1; the default n_bins is at most 30
    const long long per_dim = (n_bins > 0 ? n_bins : 30) + 1;
    long long b = n_rs > 1 ? n_rs - 1 : 1;
    for (int d = 0; d < p->cb; d++) {
        b *= per_dim;
        if (b > (1LL << 30)) return false;
    }
    p->max_bins = b;
    return true;
}

}  // namespace
}  // namespace hgc

using namespace hgc;

namespace {

struct RaggedBuffers {
    GridParams *grid;
    float *partial;
    int *keys, *subkeys, *skeys, *perm, *k1, *v1, *tkeys, *tvals, *hist, *assigned, *sassigned, *bounds, *sdir;
    KnnScratch knn;
};

// One definition of the layout serves both the size query (Sizer) and the real carve (Carver).
template <typename W>
void layout(W &ws, int n_vert, int n_coords, const RaggedPlan &p, bool use_dir, RaggedBuffers *b)
{
    const size_t n = n_vert > 0 ? n_vert : 0;
    RaggedBuffers t;
    t.grid = ws.template take<GridParams>(1);
    t.partial = ws.template take<float>((size_t)range_partial_blocks(n_vert) * 2 * kMaxBinDims);
    t.keys = ws.template take<int>(n);
    t.subkeys = ws.template take<int>(n);
    t.k1 = ws.template take<int>(n);
    t.v1 = ws.template take<int>(n);
    t.skeys = ws.template take<int>(n);
    t.perm = ws.template take<int>(n);
    t.tkeys = ws.template take<int>(n);
    t.tvals = ws.template take<int>(n);
    t.hist = ws.template take<int>(sort_hist_ints(n_vert));
    t.assigned = ws.template take<int>(n * (p.cb + 1));
    t.sassigned = ws.template take<int>(n * (p.cb + 1));
    t.bounds = ws.template take<int>((size_t)p.max_bins + 1);
    t.knn = knn_scratch_layout(ws, n_vert, n_coords);
    t.sdir = ws.template take<int>(use_dir ? n : 0);
    if (b) *b = t;
}

struct SizerW {
    Sizer s;
    template <typename T> T *take(size_t n) { s.take<T>(n); return nullptr; }
};

}  // namespace

extern "C" size_t hgc_binned_select_knn_ragged_workspace_bytes(int n_vert, int n_neigh, int n_coords,
                                                               int n_rs, int n_bins, int max_bin_dims)
{
    (void)n_neigh;
    RaggedPlan p;
    if (n_coords < 1 || !make_plan(n_coords, n_rs, n_bins, max_bin_dims, &p)) return 0;
    SizerW w;
    layout(w, n_vert, n_coords, p, true, nullptr);
    return w.s.used;
}

extern "C" int hgc_binned_select_knn_ragged(
        const float *d_coords, const int *d_row_splits, const int *d_direction,
        int *d_indices, float *d_dist, int *d_sorting_out,
        int n_vert, int n_neigh, int n_coords, int n_rs,
        int n_bins, int max_bin_dims, int tf_compat, int use_direction,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_vert < 0 || n_neigh < 1 || n_rs < 2 || n_coords < 2) return HGC_ERR_INVALID_ARGUMENT;
    RaggedPlan p;
    if (!make_plan(n_coords, n_rs, n_bins, max_bin_dims, &p)) return HGC_ERR_UNSUPPORTED;
    if (p.cb < 2) return HGC_ERR_INVALID_ARGUMENT;  // the op wants at least 2 binned dimensions
    if (p.cb > 5 || n_coords > 16 || n_neigh > 513) return HGC_ERR_UNSUPPORTED;
    if (n_vert == 0) return HGC_OK;
    if (!d_coords || !d_row_splits || !d_indices || !d_dist || (use_direction && !d_direction))
        return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_binned_select_knn_ragged_workspace_bytes(n_vert, n_neigh, n_coords, n_rs,
                                                                     n_bins, max_bin_dims);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;

    Carver ws(workspace);
    RaggedBuffers b;
    layout(ws, n_vert, n_coords, p, use_direction != 0, &b);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));

    if (int rc = compute_grid(d_coords, n_coords, p.cb, n_coords, n_vert, d_row_splits, n_rs, n_bins, n_neigh,
                              /*pre_normalized=*/0, b.partial, b.grid, stream))
        return rc;
    if (int rc = launch_bin_keys(d_coords, n_coords, p.cb, b.grid->shift, d_row_splits, n_rs,
                                 &b.grid->bin_width, b.grid->n_bins, b.assigned, nullptr, b.keys, n_vert,
                                 0, &b.grid->n_total_bins, ws.status(), stream, b.grid, n_coords, b.subkeys))
        return rc;
    // Order: by bin (what the reference's argsort gives), and inside a bin by the locality code
    // instead of by original index -- a free choice, since results do not depend on it.  Two stable
    // counting sorts, least significant key first.
    if (int rc = sort_pairs(b.subkeys, nullptr, b.k1, b.v1, b.tkeys, b.tvals, b.hist, n_vert, kSubBits, stream))
        return rc;
    {
        gather_rows_kernel<<<div_up(n_vert, 256), 256, 0, stream>>>(b.keys, 1, b.v1, b.k1, n_vert);
        HGC_LAUNCH_CHECK();
    }
    if (int rc = sort_pairs(b.k1, b.v1, b.skeys, b.perm, b.tkeys, b.tvals, b.hist, n_vert,
                            bits_for(p.max_bins), stream))
        return rc;
    if (int rc = boundaries_from_sorted_keys(b.skeys, n_vert, b.bounds, (int)p.max_bins, stream)) return rc;
    if (int rc = pack_points(d_coords, n_coords, b.perm, b.knn, n_vert, stream)) return rc;
    {
        const long long total = (long long)n_vert * (p.cb + 1);
        gather_rows_kernel<<<div_up(total, 256), 256, 0, stream>>>(b.assigned, p.cb + 1, b.perm, b.sassigned, n_vert);
        HGC_LAUNCH_CHECK();
        if (use_direction) {
            gather_rows_kernel<<<div_up(n_vert, 256), 256, 0, stream>>>(d_direction, 1, b.perm, b.sdir, n_vert);
            HGC_LAUNCH_CHECK();
        }
    }
    if (int rc = launch_select_knn(b.knn, n_coords, b.skeys, b.sassigned, b.bounds, b.grid->n_bins,
                                   &b.grid->bin_width, use_direction ? b.sdir : nullptr, d_indices, d_dist,
                                   b.perm, b.perm, n_vert, n_neigh, p.cb, (int)p.max_bins + 1, tf_compat,
                                   use_direction != 0, ws.status(), stream))
        return rc;
    if (d_sorting_out)
        HGC_CUDA_TRY(cudaMemcpyAsync(d_sorting_out, b.perm, sizeof(int) * (size_t)n_vert,
                                     cudaMemcpyDeviceToDevice, stream));
    return HGC_OK;
}
