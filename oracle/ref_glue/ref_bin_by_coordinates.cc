// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for BinByCoordinates.  The functor source is compiled from where it
// lies in the HGCalML checkout (include path given by the Makefile); nothing
// of it is copied here.
#include <cmath>
#include "bin_by_coordinates_kernel.cc"

extern "C" void ref_bin_by_coordinates(
        const float *coords, const int *row_splits, const float *bin_width, const int *n_bins,
        int *assigned_bin, int *flat_assigned_bin, int *n_per_bin,
        int n_vert, int n_coords, int n_rs, int n_total_bins, int calc_n_per_bin) {
    tensorflow::functor::BinByCoordinatesOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), coords, row_splits, bin_width, n_bins,
            assigned_bin, flat_assigned_bin, n_per_bin,
            n_vert, n_coords, n_rs, n_total_bins, calc_n_per_bin != 0);
}
