// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for LocalDistance, compiled from the HGCalML checkout.
#include <cmath>
#include "local_distance_kernel.cc"

extern "C" void ref_local_distance(const int *neigh_idxs, const float *coords, float *distances,
                                   int n_coords, int n_in_vert, int n_out_vert, int n_neigh) {
    tensorflow::functor::LocalDistanceOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), neigh_idxs, coords, distances, n_coords, n_in_vert, n_out_vert, n_neigh);
}
