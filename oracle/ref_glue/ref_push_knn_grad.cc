// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own CPU
// functor for PushKnnGrad, compiled from the HGCalML checkout.  (The functor prints one line per call.)
#include <cmath>
#include "push_knn_grad_kernel.cc"

extern "C" void ref_push_knn_grad(const float *grad, const float *weights, const float *feat, const int *idxs,
                                  float *feat_grad, float *w_grad, int n_vert, int n_neigh, int n_feat) {
    tensorflow::functor::PushKnnGradOpFunctor<tensorflow::CPUDevice, int>()(
            tensorflow::CPUDevice(), grad, weights, feat, idxs, feat_grad, w_grad, n_vert, n_neigh, n_feat);
}
