// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for PushKnn, compiled from the HGCalML checkout.  (The functor prints one line per call.)
#include <cmath>
#include "push_knn_kernel.cc"

extern "C" void ref_push_knn(const float *weights, const float *feat, const int *idxs, float *out_feat,
                             int n_vert, int n_neigh, int n_feat) {
    tensorflow::functor::PushKnnOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), weights, feat, idxs, out_feat, n_vert, n_neigh, n_feat);
}
