// Internal interface of binning.cu, shared with the fused wrapper-level entries.
#pragma once
#include "common.cuh"

namespace hgc {

constexpr int kMaxBinDims = 8;

// The binning grid of one call, derived on the device so that no host round trip is needed.
struct GridParams {
    float shift[kMaxBinDims];   // subtracted from the coordinates before binning
    int n_bins[kMaxBinDims];    // bins per binned dimension
    float bin_width;            // one width for all dimensions
    int bins_per_event;         // prod(n_bins)
    int n_total_bins;           // bins_per_event * number of events
};

int range_partial_blocks(int n_vert);

// min/max over all hits -> shift, bin width, bins per dimension (float32 arithmetic of the wrappers).
// `partial` needs range_partial_blocks(n_vert) * 2 * kMaxBinDims floats.
int compute_grid(const float *coords, int coord_stride, int n_dims, int n_vert,
                 const int *row_splits, int n_rs, int n_bins_arg, int n_neigh, int pre_normalized,
                 float *partial, GridParams *grid, cudaStream_t stream);

// Per-hit bin keys.  Any of assigned / flat_out / sort_keys may be null.  The bin count is read
// from n_total_bins_dev when that is non-null (device-derived grid), else taken from n_total_bins.
int launch_bin_keys(const float *coords, int coord_stride, int n_dims, const float *shift,
                    const int *row_splits, int n_rs, const float *bin_width, const int *n_bins,
                    int *assigned, int *flat_out, int *sort_keys, int n_vert, int n_total_bins,
                    const int *n_total_bins_dev, unsigned *status, cudaStream_t stream);

}  // namespace hgc
