// Internal interface of select_knn.cu, shared with the fused wrapper-level entry.
#pragma once
#include "common.cuh"

namespace hgc {

// float4 records per hit for n_coords coordinates (zero padded)
int knn_nv4(int n_coords);

// coords [n_vert, n_coords] (row perm[i] when perm is given) -> packed float4 records
int pack_points(const float *coords, int n_coords, const int *perm, float4 *out, int n_vert,
                cudaStream_t stream);

// The neighbour search on bin-sorted, packed points.  Row i of the result is written to output
// row row_map[i] and neighbour ids are translated through id_map (both may be null = identity).
int launch_select_knn(const float4 *pts, int n_coords, const int *bin_idx, const int *dim_bin_idx,
                      const int *bin_boundaries, const int *n_bins, const float *bin_width,
                      const int *direction, int *out_idx, float *out_dist, const int *row_map,
                      const int *id_map, int n_vert, int K, int n_bin_dim, int n_bboundaries,
                      int tf_compat, bool use_dir, unsigned *status, cudaStream_t stream);

}  // namespace hgc
