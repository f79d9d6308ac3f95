// Internal interface of binning.cu, shared with the fused wrapper-level entries.
#pragma once
#include "common.cuh"

namespace hgc {

constexpr int kMaxBinDims = 8;

// The binning grid of one call, derived on the device so that no host round trip is needed.
constexpr int kSubBits = 16;    // bits of the within-bin ordering code

struct GridParams {
    float shift[kMaxBinDims];   // subtracted from the coordinates before binning
    int n_bins[kMaxBinDims];    // bins per binned dimension
    float bin_width;            // one width for all dimensions
    int bins_per_event;         // prod(n_bins)
    int n_total_bins;           // bins_per_event * number of events
    // Within-bin ordering (a locality heuristic only, results never depend on it): hits of a bin
    // are ordered by a code that interleaves the leading bits of their position inside the bin
    // (binned coordinates) and inside the batch's range (other coordinates), always taking the
    // next bit from the coordinate whose cells are currently the largest.
    float all_min[kMaxBinDims]; // batch minimum of every coordinate
    float all_ext[kMaxBinDims]; // cell extent the code starts from: bin width or batch range
    int sub_seq[kSubBits];      // coordinate that supplies bit k of the code (most significant first)
};

int range_partial_blocks(int n_vert);

// min/max over all hits -> shift, bin width, bins per dimension (float32 arithmetic of the wrappers).
// `partial` needs range_partial_blocks(n_vert) * 2 * kMaxBinDims floats.
// n_all >= n_dims coordinates (at most kMaxBinDims) take part in the within-bin ordering code.
int compute_grid(const float *coords, int coord_stride, int n_dims, int n_all, int n_vert,
                 const int *row_splits, int n_rs, int n_bins_arg, int n_neigh, int pre_normalized,
                 float *partial, GridParams *grid, cudaStream_t stream);

// Per-hit bin keys.  Any of assigned / flat_out / sort_keys may be null.  The bin count is read
// from n_total_bins_dev when that is non-null (device-derived grid), else taken from n_total_bins.
// With `grid` and `sub_keys` given, the within-bin ordering code of every hit is written as well.
int launch_bin_keys(const float *coords, int coord_stride, int n_dims, const float *shift,
                    const int *row_splits, int n_rs, const float *bin_width, const int *n_bins,
                    int *assigned, int *flat_out, int *sort_keys, int n_vert, int n_total_bins,
                    const int *n_total_bins_dev, unsigned *status, cudaStream_t stream,
                    const GridParams *grid = nullptr, int n_all = 0, int *sub_keys = nullptr);

}  // namespace hgc
