// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for AccumulateKnnGrad, compiled from the HGCalML checkout.
#include <cmath>
#include "accumulate_knn_grad_kernel.cc"

extern "C" void ref_accumulate_knn_grad(
        const float *grad_from_out_features, const float *distances, const float *feat,
        const int *max_feat_indices, const int *neigh_indices,
        float *out_grad_distances, float *out_grad_features,
        int n_vert, int n_neigh, int n_feat, int n_grad_from_out_feat, int mean_and_max) {
    tensorflow::functor::AccumulateKnnGradOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), grad_from_out_features, distances, feat, max_feat_indices,
            neigh_indices, out_grad_distances, out_grad_features,
            n_vert, n_neigh, n_feat, n_grad_from_out_feat, 0, mean_and_max != 0);
}
