// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for AccumulateKnn, compiled from the HGCalML checkout.
#include <cmath>
#include "accumulate_knn_kernel.cc"

extern "C" void ref_accumulate_knn(
        const float *distances, const float *feat, const int *idxs,
        float *out_feat, int *out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int n_moments, int mean_and_max) {
    tensorflow::functor::AccumulateKnnOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), distances, feat, idxs, out_feat, out_maxidxs,
            n_vert, n_neigh, n_feat, n_out_feat, n_moments, mean_and_max != 0);
}
