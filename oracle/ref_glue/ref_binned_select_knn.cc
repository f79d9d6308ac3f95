// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// kernel for BinnedSelectKnn, compiled from the HGCalML checkout.
//
// The reference's CPU functor dispatches on the number of binning dimensions
// with a typo (binned_select_knn_kernel.cc:275-279: the <5> instantiation is
// guarded by n_bin_dim==4), so for 4 binning dimensions it would run <4> and
// then <5> out of bounds, and for 5 it would do nothing.  The static
// set_defaults / select_knn_kernel<D> templates are therefore called directly
// here, which is exactly what the functor does for 2 and 3 dimensions.
#include <cmath>
#include "binned_select_knn_kernel.cc"

extern "C" int ref_binned_select_knn(
        const float *coord, const int *bin_idx, const int *direction, const int *dim_bin_idx,
        const int *bin_boundaries, const int *n_bins, const float *bin_width,
        int *indices, float *dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction) {
    using namespace tensorflow::functor;
    set_defaults(indices, dist, tf_compat != 0, n_vert, n_neigh);
#define HGC_CALL(D) select_knn_kernel<D>(coord, bin_idx, direction, dim_bin_idx, bin_boundaries, \
        n_bins, bin_width, indices, dist, n_vert, n_neigh, n_coords, n_bin_dim, n_bboundaries, use_direction != 0)
    switch (n_bin_dim) {
        case 2: HGC_CALL(2); break;
        case 3: HGC_CALL(3); break;
        case 4: HGC_CALL(4); break;
        case 5: HGC_CALL(5); break;
        default: return -1;
    }
#undef HGC_CALL
    return 0;
}

// The functor exactly as the op calls it (valid for 2 and 3 binning dimensions).
extern "C" void ref_binned_select_knn_functor(
        const float *coord, const int *bin_idx, const int *direction, const int *dim_bin_idx,
        const int *bin_boundaries, const int *n_bins, const float *bin_width,
        int *indices, float *dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction) {
    tensorflow::functor::BinnedSelectKnnOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), coord, bin_idx, direction, dim_bin_idx, bin_boundaries, n_bins,
            bin_width, indices, dist, n_vert, n_neigh, n_coords, n_bin_dim, n_bboundaries,
            tf_compat != 0, use_direction != 0);
}
