// TEST INFRASTRUCTURE ONLY: C entry point around the reference's own GPU functor for SelectKnnGrad
// (modules/compiled/select_knn_grad_kernel.cu.cc:81-216; the op has no CPU implementation), compiled
// with nvcc from the HGCalML checkout against the stand-in header in tf_stub/.  The functor launches
// on the legacy default stream and synchronises the device itself.
#define GOOGLE_CUDA 1
#include <cstdio>
#include "select_knn_grad_kernel.cu.cc"

extern "C" int ref_cuda_select_knn_grad(const float *d_grad_dist, const int *d_indices, const float *d_dist,
                                        const float *d_coord, float *d_grad_coord, int n_vert, int n_neigh,
                                        int n_coords)
{
    Eigen::GpuDevice device;
    tensorflow::functor::SelectKnnGradOpFunctor<Eigen::GpuDevice, int>()(
            device, d_grad_dist, d_indices, d_dist, d_coord, d_grad_coord, n_vert, n_neigh, n_coords);
    return (int)cudaGetLastError();
}
