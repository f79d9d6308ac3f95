// BinnedSelectKnn: host side of the search (packing, chunk bounding boxes, dispatch) and the
// op-level C entry.  The search kernel itself is in select_knn_kernel.cuh.
#include "common.cuh"
#include "select_knn.cuh"

// ranges longer than this many hits are scanned chunk-wise with box tests; grid size per SM
#ifndef HGC_KNN_LONG_RANGE
#define HGC_KNN_LONG_RANGE 96
#endif
#ifndef HGC_KNN_GRID_BLOCKS_PER_SM
#define HGC_KNN_GRID_BLOCKS_PER_SM 8
#endif

namespace hgc {
namespace {

#ifdef HGC_KNN_STATS
// work counters of the search kernel (instrumented builds only: make EXTRA=-DHGC_KNN_STATS)
__device__ unsigned long long g_knn_stats[96];
#endif

// [n_vert, n_coords] floats (optionally gathered through perm) -> zero-padded float4 records
__global__ void pack_points_kernel(const float *__restrict__ coords, int n_coords, int nv4,
                                   const int *__restrict__ perm, float4 *__restrict__ out, int n_vert)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)n_vert * nv4) return;
    const int i = (int)(t / nv4), u = (int)(t % nv4);
    const float *src = coords + (size_t)(perm ? perm[i] : i) * n_coords;
    float c[4];
#pragma unroll
    for (int k = 0; k < 4; k++) c[k] = (u * 4 + k < n_coords) ? src[u * 4 + k] : 0.f;
    out[t] = make_float4(c[0], c[1], c[2], c[3]);
}

// One warp per chunk of 32 consecutive records: component-wise min and max.
__global__ void __launch_bounds__(256)
chunk_aabb_kernel(const float4 *__restrict__ pts, int nv4, int n_vert, float4 *__restrict__ lo,
                  float4 *__restrict__ hi)
{
    const int lane = threadIdx.x & 31;
    const long long chunk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (chunk * 32 >= n_vert) return;
    const long long i = chunk * 32 + lane;
    for (int u = 0; u < nv4; u++) {
        float4 mn = make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
        float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        if (i < n_vert) mn = mx = pts[(size_t)i * nv4 + u];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn.x = fminf(mn.x, __shfl_xor_sync(0xffffffffu, mn.x, o));
            mn.y = fminf(mn.y, __shfl_xor_sync(0xffffffffu, mn.y, o));
            mn.z = fminf(mn.z, __shfl_xor_sync(0xffffffffu, mn.z, o));
            mn.w = fminf(mn.w, __shfl_xor_sync(0xffffffffu, mn.w, o));
            mx.x = fmaxf(mx.x, __shfl_xor_sync(0xffffffffu, mx.x, o));
            mx.y = fmaxf(mx.y, __shfl_xor_sync(0xffffffffu, mx.y, o));
            mx.z = fmaxf(mx.z, __shfl_xor_sync(0xffffffffu, mx.z, o));
            mx.w = fmaxf(mx.w, __shfl_xor_sync(0xffffffffu, mx.w, o));
        }
        if (lane == 0) {
            lo[(size_t)chunk * nv4 + u] = mn;
            hi[(size_t)chunk * nv4 + u] = mx;
        }
    }
}

}  // namespace

int pack_points(const float *coords, int n_coords, const int *perm, const KnnScratch &s, int n_vert,
                cudaStream_t stream)
{
    if (n_vert <= 0) return HGC_OK;
    const int nv4 = knn_nv4(n_coords);
    const long long total = (long long)n_vert * nv4;
    pack_points_kernel<<<div_up(total, 256), 256, 0, stream>>>(coords, n_coords, nv4, perm, s.pts, n_vert);
    HGC_LAUNCH_CHECK();
    chunk_aabb_kernel<<<div_up((long long)knn_chunks(n_vert), 8), 256, 0, stream>>>(s.pts, nv4, n_vert,
                                                                                    s.chunk_lo, s.chunk_hi);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

int launch_select_knn(const KnnScratch &s, int n_coords, const int *bin_idx, const int *dim_bin_idx,
                      const int *bin_boundaries, const int *n_bins, const float *bin_width,
                      const int *direction, int *out_idx, float *out_dist, const int *row_map,
                      const int *id_map, int n_vert, int K, int n_bin_dim, int n_bboundaries,
                      int tf_compat, bool use_dir, unsigned *status, cudaStream_t stream)
{
    if (n_vert <= 0) return HGC_OK;
    KnnArgs a;
    a.pts = s.pts; a.chunk_lo = s.chunk_lo; a.chunk_hi = s.chunk_hi;
    a.bin_idx = bin_idx; a.dim_bin_idx = dim_bin_idx; a.bin_boundaries = bin_boundaries;
    a.n_bins = n_bins; a.bin_width = bin_width; a.direction = direction;
    a.out_idx = out_idx; a.out_dist = out_dist; a.row_map = row_map; a.id_map = id_map;
    a.n_vert = n_vert; a.K = K; a.n_bboundaries = n_bboundaries; a.tf_compat = tf_compat;
    a.status = status;
    a.work_counter = status + 16;  // inside the 256 zeroed bytes that start every workspace
    a.long_range = HGC_KNN_LONG_RANGE;
    a.fetch = 1;
    a.blocks_per_sm = HGC_KNN_GRID_BLOCKS_PER_SM;
    a.stats = nullptr;
#ifdef HGC_KNN_STATS
    {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_knn_stats) == cudaSuccess) a.stats = static_cast<unsigned long long *>(p);
    }
#endif
    switch (knn_nv4(n_coords)) {
        case 1: return launch_knn_nv<1>(a, n_bin_dim, use_dir, stream);
        case 2: return launch_knn_nv<2>(a, n_bin_dim, use_dir, stream);
        case 3: return launch_knn_nv<3>(a, n_bin_dim, use_dir, stream);
        case 4: return launch_knn_nv<4>(a, n_bin_dim, use_dir, stream);
    }
    return HGC_ERR_UNSUPPORTED;
}

}  // namespace hgc

using namespace hgc;

#ifdef HGC_KNN_STATS
// Tuning aid: copies the search kernel's work counters (queries, candidates offered, accepted,
// list merges, boxes tested, chunks scanned, steps, then cycles: per query, in merges, in candidate
// steps, ...; from [16] on, per final shell 0..7: queries, candidates, cycles, accepted, cycles in merges /
// candidate steps / enumeration / box tests, steps, boxes; filled only by
// a build with -DHGC_KNN_STATS) to the host and clears them.
extern "C" int hgc_debug_knn_stats(unsigned long long *out96)
{
    HGC_CUDA_TRY(cudaDeviceSynchronize());
    HGC_CUDA_TRY(cudaMemcpyFromSymbol(out96, g_knn_stats, sizeof(unsigned long long) * 96));
    unsigned long long zero[96] = {0};
    HGC_CUDA_TRY(cudaMemcpyToSymbol(g_knn_stats, zero, sizeof(zero)));
    return HGC_OK;
}
#endif

namespace {
struct SizerW {
    Sizer s;
    template <typename T> T *take(size_t n) { s.take<T>(n); return nullptr; }
};
}  // namespace

extern "C" size_t hgc_binned_select_knn_workspace_bytes(int n_vert, int n_neigh, int n_coords, int n_bin_dim)
{
    (void)n_neigh; (void)n_bin_dim;
    SizerW w;
    knn_scratch_layout(w, n_vert, n_coords > 0 ? n_coords : 1);
    return w.s.used;
}

extern "C" int hgc_binned_select_knn(
        const float *d_coord, const int *d_bin_idx, const int *d_direction, const int *d_dim_bin_idx,
        const int *d_bin_boundaries, const int *d_n_bins, const float *d_bin_width,
        int *d_indices, float *d_dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // shape rules of the op (modules/compiled/binned_select_knn_kernel.cc:336-352)
    if (n_vert < 0 || n_neigh < 1 || n_bboundaries < 1) return HGC_ERR_INVALID_ARGUMENT;
    if (n_bin_dim < 2 || n_bin_dim > 5 || n_coords < 2) return HGC_ERR_INVALID_ARGUMENT;
    if (n_coords > 16 || n_neigh > 513) return HGC_ERR_UNSUPPORTED;
    if (n_vert == 0) return HGC_OK;
    if (!d_coord || !d_bin_idx || !d_dim_bin_idx || !d_bin_boundaries || !d_n_bins || !d_bin_width ||
        !d_indices || !d_dist || (use_direction && !d_direction))
        return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_binned_select_knn_workspace_bytes(n_vert, n_neigh, n_coords, n_bin_dim);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    const KnnScratch s = knn_scratch_layout(ws, n_vert, n_coords);
    if (int rc = pack_points(d_coord, n_coords, nullptr, s, n_vert, stream)) return rc;
    return launch_select_knn(s, n_coords, d_bin_idx, d_dim_bin_idx, d_bin_boundaries, d_n_bins,
                             d_bin_width, d_direction, d_indices, d_dist, nullptr, nullptr, n_vert,
                             n_neigh, n_bin_dim, n_bboundaries, tf_compat, use_direction != 0,
                             ws.status(), stream);
}
