// Instantiates the search kernel for hits of 3 packed float4 record(s) (up to 12 coordinates).
#include "select_knn_kernel.cuh"
namespace hgc {
template int launch_knn_nv<3>(const KnnArgs &, int, bool, cudaStream_t);
}
