// Instantiates the search kernel for hits of 4 packed float4 record(s) (up to 16 coordinates).
#include "select_knn_kernel.cuh"
namespace hgc {
template int launch_knn_nv<4>(const KnnArgs &, int, bool, cudaStream_t);
}
