// Internal interface of the neighbour search, shared with the fused wrapper-level entry.
#pragma once
#include "common.cuh"

namespace hgc {

struct KnnArgs {
    const float4 *pts;          // [n_vert][NV4] packed, bin-sorted
    const float4 *chunk_lo;     // [ceil(n_vert/32)][NV4] bounding boxes of 32 consecutive hits
    const float4 *chunk_hi;
    const int *bin_idx;         // [n_vert]
    const int *dim_bin_idx;     // [n_vert][CB+1]
    const int *bin_boundaries;  // [n_bboundaries]
    const int *n_bins;          // [CB]
    const float *bin_width;     // [1]
    const int *direction;       // [n_vert] or null
    int *out_idx;               // [n_vert][K]
    float *out_dist;            // [n_vert][K]
    const int *row_map;         // output row of bin-sorted query i (null: i)
    const int *id_map;          // output id of bin-sorted hit j (null: j)
    int n_vert, K, n_bboundaries;
    int tf_compat;
    int fetch, blocks_per_sm;   // queries a warp takes at a time; grid size per SM
    int long_range;             // ranges longer than this are scanned chunk-wise with box tests
    unsigned *status;
    unsigned *work_counter;     // zeroed before the launch; hands out runs of queries to warps
    unsigned long long *stats;  // optional work counters (tuning aid), null in normal use
};

template <int NV4>
int launch_knn_nv(const KnnArgs &a, int n_bin_dim, bool use_dir, cudaStream_t stream);

// float4 records per hit for n_coords coordinates (zero padded)
inline int knn_nv4(int n_coords) { return (n_coords + 3) / 4; }
inline size_t knn_chunks(int n_vert) { return ((size_t)(n_vert > 0 ? n_vert : 0) + 31) / 32; }

// Scratch of the search: packed points and the chunk boxes.
struct KnnScratch {
    float4 *pts, *chunk_lo, *chunk_hi;
};
template <typename W>
inline KnnScratch knn_scratch_layout(W &ws, int n_vert, int n_coords)
{
    KnnScratch s;
    const size_t nv4 = knn_nv4(n_coords);
    s.pts = ws.template take<float4>((size_t)(n_vert > 0 ? n_vert : 0) * nv4);
    s.chunk_lo = ws.template take<float4>(knn_chunks(n_vert) * nv4);
    s.chunk_hi = ws.template take<float4>(knn_chunks(n_vert) * nv4);
    return s;
}

// coords [n_vert, n_coords] (row perm[i] when perm is given) -> packed float4 records, plus the
// bounding boxes of every 32 consecutive records
int pack_points(const float *coords, int n_coords, const int *perm, const KnnScratch &s, int n_vert,
                cudaStream_t stream);

// The neighbour search on bin-sorted, packed points.  Row i of the result is written to output
// row row_map[i] and neighbour ids are translated through id_map (both may be null = identity).
int launch_select_knn(const KnnScratch &s, int n_coords, const int *bin_idx, const int *dim_bin_idx,
                      const int *bin_boundaries, const int *n_bins, const float *bin_width,
                      const int *direction, int *out_idx, float *out_dist, const int *row_map,
                      const int *id_map, int n_vert, int K, int n_bin_dim, int n_bboundaries,
                      int tf_compat, bool use_dir, unsigned *status, cudaStream_t stream);

}  // namespace hgc
