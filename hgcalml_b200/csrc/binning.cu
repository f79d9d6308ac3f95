// Grid binning of hits: per-hit bin keys, the batch-global coordinate range, and the histogram
// (hits per bin) obtained from the sorted keys instead of from atomics.
#include "common.cuh"
#include "binning.cuh"

namespace hgc {

// ---- per-hit keys ---------------------------------------------------------------------------
// Follows modules/compiled/bin_by_coordinates_kernel.cc:64-113: truncating float division per
// dimension (last dimension fastest), out-of-range indices forced to 0, event index above all.
// `shift` (may be null) is subtracted from the coordinates first, as the Python wrapper does
// before calling the op (modules/bin_by_coordinates_op.py:49-52).
__global__ void bin_keys_kernel(const float *__restrict__ coords, int coord_stride, int n_dims,
                                const float *__restrict__ shift,
                                const int *__restrict__ row_splits, int n_rs,
                                const float *__restrict__ bin_width, const int *__restrict__ n_bins,
                                int *__restrict__ assigned, int *__restrict__ flat_out,
                                int *__restrict__ sort_keys, int n_vert, int n_total_bins,
                                const int *__restrict__ n_total_bins_dev, unsigned *status,
                                const GridParams *__restrict__ grid, int n_all, int *__restrict__ sub_keys)
{
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n_vert) return;
    unsigned frac[kMaxBinDims];  // position inside the cell as a 16-bit fraction (ordering code only)
#pragma unroll
    for (int c = 0; c < kMaxBinDims; c++) frac[c] = 0u;
    const float bw = bin_width[0];
    const int total = n_total_bins_dev ? n_total_bins_dev[0] : n_total_bins;
    int stride = 1, flat = 0;
    for (int c = n_dims - 1; c >= 0; c--) {
        float x = coords[(size_t)v * coord_stride + c];
        if (shift) x = __fsub_rn(x, shift[c]);
        int ci = __float2int_rz(__fdiv_rn(x, bw));
        const int nb = n_bins[c];
        if (sub_keys) {
            const float u = __fdiv_rn(x, bw) - (float)ci;
#pragma unroll
            for (int k = 0; k < kMaxBinDims; k++)
                if (k == c) frac[k] = (unsigned)fminf(fmaxf(u * 65536.f, 0.f), 65535.f);
        }
        if (ci < 0 || ci >= nb) {
            ci = 0;
            flag_status(status, HGC_STATUS_BIN_OUT_OF_RANGE);
        }
        if (assigned) assigned[(size_t)v * (n_dims + 1) + c + 1] = ci;
        flat += ci * stride;
        stride *= nb;
    }
    // event = number of row_splits[1..n_rs-1] that are <= v (row splits ascend)
    int lo = 1, hi = n_rs;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_splits[mid] <= v) lo = mid + 1; else hi = mid;
    }
    const int event = lo - 1;
    flat += event * stride;
    if (flat >= total || flat < 0) {
        flag_status(status, HGC_STATUS_FLAT_BIN_OVERFLOW);
        if (sort_keys) sort_keys[v] = total;  // sentinel: sorts last, belongs to no bin
        return;
    }
    if (assigned) assigned[(size_t)v * (n_dims + 1)] = event;
    if (flat_out) flat_out[v] = flat;
    if (sort_keys) sort_keys[v] = flat;
    if (sub_keys) {
#pragma unroll
        for (int c = 0; c < kMaxBinDims; c++)
            if (c >= n_dims && c < n_all) {
                const float ext = grid->all_ext[c];
                const float u = ext > 0.f ? (coords[(size_t)v * coord_stride + c] - grid->all_min[c]) / ext : 0.f;
                frac[c] = (unsigned)fminf(fmaxf(u * 65536.f, 0.f), 65535.f);
            }
        unsigned code = 0u;
#pragma unroll
        for (int k = 0; k < kSubBits; k++) {
            const int c = grid->sub_seq[k];
            unsigned f = 0u;
#pragma unroll
            for (int q = 0; q < kMaxBinDims; q++)
                if (q == c) { f = frac[q]; frac[q] = (frac[q] << 1) & 0xffffu; }
            code = (code << 1) | (f >> 15);
        }
        sub_keys[v] = (int)code;
    }
}

__global__ void adjacent_difference_kernel(const int *__restrict__ bounds, int *__restrict__ out, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bounds[i + 1] - bounds[i];
}

// ---- batch-global min / max of the first n_dims coordinates -----------------------------------

__global__ void __launch_bounds__(256)
range_partial_kernel(const float *__restrict__ coords, int coord_stride, int n_dims, int n_vert,
                     float *__restrict__ partial /* [gridDim.x][2][kMaxBinDims] */)
{
    float mn[kMaxBinDims], mx[kMaxBinDims];
#pragma unroll
    for (int c = 0; c < kMaxBinDims; c++) { mn[c] = INFINITY; mx[c] = -INFINITY; }
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vert; v += gridDim.x * blockDim.x) {
#pragma unroll
        for (int c = 0; c < kMaxBinDims; c++)
            if (c < n_dims) {
                const float x = coords[(size_t)v * coord_stride + c];
                mn[c] = fminf(mn[c], x);
                mx[c] = fmaxf(mx[c], x);
            }
    }
    __shared__ float s_mn[8][kMaxBinDims], s_mx[8][kMaxBinDims];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int c = 0; c < kMaxBinDims; c++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn[c] = fminf(mn[c], __shfl_xor_sync(0xffffffffu, mn[c], o));
            mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], o));
        }
        if (lane == 0) { s_mn[warp][c] = mn[c]; s_mx[warp][c] = mx[c]; }
    }
    __syncthreads();
    if (threadIdx.x < kMaxBinDims) {
        const int c = threadIdx.x;
        float a = s_mn[0][c], b = s_mx[0][c];
        for (int w = 1; w < 8; w++) { a = fminf(a, s_mn[w][c]); b = fmaxf(b, s_mx[w][c]); }
        partial[((size_t)blockIdx.x * 2 + 0) * kMaxBinDims + c] = a;
        partial[((size_t)blockIdx.x * 2 + 1) * kMaxBinDims + c] = b;
    }
}

constexpr int kGridSetupThreads = 256;

// One block: finishes the min/max reduction and derives the grid exactly as the Python wrappers do
// (modules/bin_by_coordinates_op.py:49-71, modules/binned_select_knn_op.py:57-63), in float32.
__global__ void __launch_bounds__(kGridSetupThreads)
grid_setup_kernel(const float *__restrict__ partial, int n_partials, int n_dims, int n_all,
                  const int *__restrict__ row_splits, int n_rs, int n_bins_arg, int n_neigh,
                  int pre_normalized, GridParams *__restrict__ g)
{
    // min / max over the per-block partial results: thread t looks at coordinate t % 8 of every
    // (kGridSetupThreads / 8)-th partial, a shared-memory pass combines the threads of a coordinate
    static_assert(kMaxBinDims == 8 && kGridSetupThreads % 8 == 0, "layout of the reduction");
    __shared__ float s_mn[kGridSetupThreads], s_mx[kGridSetupThreads];
    {
        const int cc = threadIdx.x & 7;
        float a = INFINITY, b = -INFINITY;
        for (int p = threadIdx.x >> 3; p < n_partials; p += kGridSetupThreads / 8) {
            a = fminf(a, partial[((size_t)p * 2 + 0) * kMaxBinDims + cc]);
            b = fmaxf(b, partial[((size_t)p * 2 + 1) * kMaxBinDims + cc]);
        }
        s_mn[threadIdx.x] = a;
        s_mx[threadIdx.x] = b;
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;  // the rest is one warp's work
    const int c = threadIdx.x;
    float mn = 0.f, mx = 0.f;
    if (c < n_all) {
        mn = INFINITY; mx = -INFINITY;
        for (int t = c; t < kGridSetupThreads; t += 8) {
            mn = fminf(mn, s_mn[t]);
            mx = fmaxf(mx, s_mx[t]);
        }
    }
    // The wrapper shifts by the minimum first; x -> x - mn is monotone, so the shifted extremes
    // are the extremes shifted.
    const float shift = pre_normalized ? 0.f : mn;
    const float smin = __fsub_rn(mn, shift);
    float dmax = __fsub_rn(mx, shift);
    if (smin == dmax) dmax = __fadd_rn(dmax, 1.f);
    dmax = __fadd_rn(dmax, 1e-3f);
    if (!isfinite(dmax)) dmax = 1.f;

    int n_bins = n_bins_arg;
    if (n_bins <= 0) {
        const float first_event = n_rs > 1 ? (float)row_splits[1] : 1.f;
        const float t = powf(__fdiv_rn(first_event, (float)n_neigh / 32.f), 1.f / (float)n_dims);
        n_bins = (int)t;
        n_bins = n_bins < 5 ? 5 : (n_bins > 30 ? 30 : n_bins);
    }
    float bw = c < n_dims ? __fdiv_rn(dmax, (float)n_bins) : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bw = fmaxf(bw, __shfl_xor_sync(0xffffffffu, bw, o));
    int nb = 1;
    if (c < n_dims) nb = (int)__fadd_rn(__fdiv_rn(dmax, bw), 1.f);
    int prod = nb;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) prod *= __shfl_xor_sync(0xffffffffu, prod, o);
    if (c < n_dims) { g->shift[c] = shift; g->n_bins[c] = nb; }
    if (c == 0) {
        g->bin_width = bw;
        g->bins_per_event = prod;
        g->n_total_bins = prod * (n_rs - 1);
    }
    // within-bin ordering code: start from the bin width (binned) or the batch range (others)
    float ext = 0.f;
    if (c < n_dims) ext = bw;
    else if (c < n_all) { ext = mx - mn; if (!isfinite(ext)) ext = 0.f; }
    if (c < kMaxBinDims) { g->all_min[c] = mn; g->all_ext[c] = ext; }
    float cell[kMaxBinDims];
#pragma unroll
    for (int k = 0; k < kMaxBinDims; k++) cell[k] = __shfl_sync(0xffffffffu, ext, k);
    if (c == 0) {
        for (int k = 0; k < kSubBits; k++) {
            int best = 0;
#pragma unroll
            for (int q = 1; q < kMaxBinDims; q++)
                if (cell[q] > cell[best]) best = q;
            g->sub_seq[k] = best;
#pragma unroll
            for (int q = 0; q < kMaxBinDims; q++)
                if (q == best) cell[q] *= 0.5f;
        }
    }
}

int compute_grid(const float *coords, int coord_stride, int n_dims, int n_all, int n_vert,
                 const int *row_splits, int n_rs, int n_bins_arg, int n_neigh, int pre_normalized,
                 float *partial, GridParams *grid, cudaStream_t stream)
{
    if (n_all < n_dims) n_all = n_dims;
    if (n_all > kMaxBinDims) n_all = kMaxBinDims;
    const int blocks = range_partial_blocks(n_vert);
    range_partial_kernel<<<blocks, 256, 0, stream>>>(coords, coord_stride, n_all, n_vert, partial);
    HGC_LAUNCH_CHECK();
    grid_setup_kernel<<<1, kGridSetupThreads, 0, stream>>>(partial, blocks, n_dims, n_all, row_splits, n_rs, n_bins_arg,
                                           n_neigh, pre_normalized, grid);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

int range_partial_blocks(int n_vert)
{
    // a fixed cap (the workspace size depends on it, so it must not depend on the device)
    constexpr int kMaxPartialBlocks = 296;
    int b = div_up(n_vert > 0 ? n_vert : 1, 256 * 8);
    return b > kMaxPartialBlocks ? kMaxPartialBlocks : b;
}

int launch_bin_keys(const float *coords, int coord_stride, int n_dims, const float *shift,
                    const int *row_splits, int n_rs, const float *bin_width, const int *n_bins,
                    int *assigned, int *flat_out, int *sort_keys, int n_vert, int n_total_bins,
                    const int *n_total_bins_dev, unsigned *status, cudaStream_t stream,
                    const GridParams *grid, int n_all, int *sub_keys)
{
    if (n_vert <= 0) return HGC_OK;
    if (n_all > kMaxBinDims) n_all = kMaxBinDims;
    bin_keys_kernel<<<div_up(n_vert, 256), 256, 0, stream>>>(
            coords, coord_stride, n_dims, shift, row_splits, n_rs, bin_width, n_bins, assigned, flat_out,
            sort_keys, n_vert, n_total_bins, n_total_bins_dev, status, grid, n_all, grid ? sub_keys : nullptr);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

}  // namespace hgc

using namespace hgc;

extern "C" size_t hgc_bin_by_coordinates_workspace_bytes(int n_vert, int n_coords, int n_rs, int n_total_bins)
{
    (void)n_coords; (void)n_rs;
    Sizer s;
    const size_t n = n_vert > 0 ? n_vert : 0;
    s.take<int>(n);                                   // sort keys
    s.take<int>(n); s.take<int>(n);                   // sorted keys / values
    s.take<int>(n); s.take<int>(n);                   // ping-pong
    s.take<int>(sort_hist_ints(n_vert));
    s.take<int>((size_t)(n_total_bins > 0 ? n_total_bins : 0) + 1);
    return s.used;
}

extern "C" int hgc_bin_by_coordinates(
        const float *d_coords, const int *d_row_splits, const float *d_bin_width, const int *d_n_bins,
        int *d_assigned_bin, int *d_flat_assigned_bin, int *d_n_per_bin,
        int n_vert, int n_coords, int n_rs, int n_total_bins, int calc_n_per_bin,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_vert < 0 || n_coords < 1 || n_rs < 1 || n_total_bins < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (n_coords > kMaxBinDims) return HGC_ERR_UNSUPPORTED;
    if (!d_bin_width || !d_n_bins || !d_row_splits || (n_vert > 0 && (!d_coords || !d_assigned_bin || !d_flat_assigned_bin)))
        return HGC_ERR_INVALID_ARGUMENT;
    if (n_total_bins > 0 && !d_n_per_bin) return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_bin_by_coordinates_workspace_bytes(n_vert, n_coords, n_rs, n_total_bins);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;

    Carver ws(workspace);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, sizeof(unsigned), stream));
    const size_t n = n_vert;
    int *keys = ws.take<int>(n);
    int *skeys = ws.take<int>(n), *svals = ws.take<int>(n);
    int *tkeys = ws.take<int>(n), *tvals = ws.take<int>(n);
    int *hist = ws.take<int>(sort_hist_ints(n_vert));
    int *bounds = ws.take<int>((size_t)n_total_bins + 1);

    const bool histogram = calc_n_per_bin != 0 && n_total_bins > 0;
    if (int rc = launch_bin_keys(d_coords, n_coords, n_coords, nullptr, d_row_splits, n_rs, d_bin_width,
                                 d_n_bins, d_assigned_bin, d_flat_assigned_bin, histogram ? keys : nullptr,
                                 n_vert, n_total_bins, nullptr, ws.status(), stream))
        return rc;
    if (n_total_bins == 0) return HGC_OK;
    if (!histogram) {
        HGC_CUDA_TRY(cudaMemsetAsync(d_n_per_bin, 0, sizeof(int) * (size_t)n_total_bins, stream));
        return HGC_OK;
    }
    if (int rc = sort_pairs(keys, nullptr, skeys, svals, tkeys, tvals, hist, n_vert,
                            bits_for(n_total_bins), stream))
        return rc;
    if (int rc = boundaries_from_sorted_keys(skeys, n_vert, bounds, n_total_bins, stream)) return rc;
    adjacent_difference_kernel<<<div_up(n_total_bins, 256), 256, 0, stream>>>(bounds, d_n_per_bin, n_total_bins);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}
