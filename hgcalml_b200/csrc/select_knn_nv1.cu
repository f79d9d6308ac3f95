// Instantiates the search kernel for hits of 1 packed float4 record(s) (up to 4 coordinates).
#include "select_knn_kernel.cuh"
namespace hgc {
template int launch_knn_nv<1>(const KnnArgs &, int, bool, cudaStream_t);
}
