// TEST INFRASTRUCTURE ONLY.
//
// Stand-in for TensorFlow's "tensorflow/core/util/gpu_kernel_helper.h", just large enough that the
// CUDA translation units of the HGCalML custom ops (modules/compiled/*_kernel.cu.cc) compile with
// nvcc WITHOUT TensorFlow: they only need Eigen::GpuDevice::stream().  The stand-in device always
// answers with the legacy default stream.
#ifndef HGC_ORACLE_TF_STUB_GPU_KERNEL_HELPER_H
#define HGC_ORACLE_TF_STUB_GPU_KERNEL_HELPER_H

#include <cuda_runtime.h>

namespace Eigen {
struct ThreadPoolDevice {};
struct GpuDevice {
    cudaStream_t stream() const { return nullptr; }
};
}  // namespace Eigen

#endif
