// Instantiates the search kernel for hits of 2 packed float4 record(s) (up to 8 coordinates).
#include "select_knn_kernel.cuh"
namespace hgc {
template int launch_knn_nv<2>(const KnnArgs &, int, bool, cudaStream_t);
}
