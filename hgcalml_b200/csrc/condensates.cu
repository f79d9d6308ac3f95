// BinnedAssignToCondensates on the GPU (the reference has a CPU body only:
// modules/compiled/binned_assign_to_condensates_kernel.cc:23-241).
//
// The reference is a sequential greedy loop per event: take the not-yet-claimed high-beta hit with
// the largest beta (first among equals), make it the next condensate, let it claim the hits inside
// its radius, repeat.  The same result is produced here in three parallel steps:
//   1. priority sort  : the high-beta hits of each event are ordered by (beta descending, position
//                       ascending) with the stable counting sort of radix_sort.cu;
//   2. claim pass     : one block per event walks that order in windows of 1024 hits; a window is
//                       first tested against all condensates confirmed so far (parallel), then the
//                       survivors are resolved in order, each new condensate claiming the later
//                       survivors it covers.  A hit is a condensate exactly when no earlier
//                       condensate covers it, which is the greedy rule;
//   3. assignment     : every hit of the event is tested against the event's condensates in rank
//                       order (tiles of the list in shared memory): the first that covers it wins
//                       (assign_by_max_beta) or the reference's distance fold is applied.
// The reference finds a condensate's hits through the bins overlapping its bounding box and then
// applies an exact distance test; testing all condensates of the event gives the same set, so the
// bin inputs are accepted for interface compatibility and not read.
#include <cooperative_groups.h>
#include "common.cuh"

namespace hgc {
namespace {

constexpr int kMaxDims = 8;
constexpr int kClaimThreads = 1024;
constexpr int kAssignThreads = 256;
constexpr int kCondTile = 256;

struct CondList {        // per event e, entries [row_splits_h[e], row_splits_h[e] + count[e])
    float *centre;       // [n_h][dims]
    float *radius_sq;    // [n_h]
    int *subset_pos;     // [n_h]  position in the *_h arrays
    int *lonely;         // [n_h]  1: masked hit that only claims itself
    int *count;          // [num_rows]
};

__device__ __forceinline__ unsigned ordered_bits(float f)
{
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Sort key of a high-beta hit: 0 for hits the reference's pick loop takes in position order (it
// tests no_condensation_mask_h at index 0 or 1 only, binned_assign_to_condensates_kernel.cc:193),
// else 1 + descending beta.
__global__ void priority_keys_kernel(const float *__restrict__ beta_h, const int *__restrict__ mask_h,
                                     const int *__restrict__ row_splits_h, int num_rows, int n_h,
                                     int *__restrict__ beta_keys, int *__restrict__ event_keys)
{
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= n_h) return;
    const bool flagged = mask_h[a > 0 ? 1 : 0] != 0;  // n_h >= 2 whenever a > 0
    unsigned key = 0u;
    if (!flagged) {
        const unsigned desc = ~ordered_bits(beta_h[a]);
        key = desc == 0xffffffffu ? desc : desc + 1u;
    }
    beta_keys[a] = (int)key;
    int lo = 1, hi = num_rows + 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_splits_h[mid] <= a) lo = mid + 1; else hi = mid;
    }
    event_keys[a] = lo - 1;
}

__global__ void gather_int_kernel(const int *__restrict__ src, const int *__restrict__ idx,
                                  int *__restrict__ dst, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[idx[i]];
}

__global__ void init_outputs_kernel(int *__restrict__ status_h, int *__restrict__ alpha, int n_h,
                                    int *__restrict__ assignment, int *__restrict__ association, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_h) { status_h[i] = 0; alpha[i] = -1; }
    if (i < n) { assignment[i] = -1; association[i] = -1; }
}

__device__ __forceinline__ float centre_distsq(const float *c, const float *x, int dims)
{
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < kMaxDims; d++)
        if (d < dims) {
            const float t = __fsub_rn(c[d], x[d]);
            s = __fadd_rn(s, __fmul_rn(t, t));
        }
    return s;
}

// Step 2.  order[] lists, per event, the subset positions in priority order.
//
// A cluster of kClusterBlocks blocks works on one event and walks the priority order in windows of
// kWindow hits.  (a) Every block tests its 1024 hits of the window against the condensates confirmed
// in earlier windows and leaves a flag per hit.  (b) After a cluster barrier, block 0 resolves the
// survivors in order: the first open hit becomes the next condensate and closes the later survivors
// it covers.  (c) A second cluster barrier publishes the longer condensate list to all blocks.
// The barriers are the hardware cluster barrier; every block of a cluster runs the same number of
// windows, so none can be left waiting.
constexpr int kClusterBlocks = 8;
constexpr int kWindow = kClusterBlocks * kClaimThreads;
constexpr int kItems = kWindow / kClaimThreads;  // survivors a thread of block 0 looks after

__device__ __forceinline__ bool covers(const float *c, float r2, int lonely, int c_pos, const float *x, int dims,
                                       int x_pos, int x_mask)
{
    if (lonely) return c_pos == x_pos;
    return x_mask == 0 && centre_distsq(c, x, dims) <= r2;
}

__global__ void __cluster_dims__(kClusterBlocks, 1, 1) __launch_bounds__(kClaimThreads)
claim_kernel(int dims, const float *__restrict__ ccoords_h, const float *__restrict__ dist_h,
             const int *__restrict__ mask_h, const int *__restrict__ original_indices_h,
             const int *__restrict__ row_splits_h, const int *__restrict__ order,
             int *__restrict__ status_h, int *__restrict__ alpha_indices, int *__restrict__ open_flags,
             CondList cl)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_c[kCondTile][kMaxDims];
    __shared__ float s_r2[kCondTile];
    __shared__ int s_pos[kCondTile];
    __shared__ int s_lonely[kCondTile];
    __shared__ int s_first[32];
    __shared__ float s_new_c[kMaxDims];
    __shared__ float s_new_r2;
    __shared__ int s_new_pos, s_new_lonely;

    const int rank = (int)cluster.block_rank();
    const int e = blockIdx.x / kClusterBlocks;
    const int off = row_splits_h[e], n_h = row_splits_h[e + 1] - off;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    int *flags = open_flags + (size_t)e * kWindow;
    volatile int *count = cl.count + e;

    for (int w0 = 0; w0 < n_h; w0 += kWindow) {
        int n_cond = *count;  // published by block 0 before the barrier that ended the previous window

        // (a) this block's hits of the window against the confirmed condensates
        const int p = w0 + rank * kClaimThreads + t;
        const bool active = p < n_h;
        int a = 0, my_mask = 0;
        float x[kMaxDims];
        if (active) {
            a = order[off + p];
            my_mask = mask_h[a];
#pragma unroll
            for (int d = 0; d < kMaxDims; d++) x[d] = d < dims ? ccoords_h[(size_t)a * dims + d] : 0.f;
        }
        bool open = active;
        for (int c0 = 0; c0 < n_cond; c0 += kCondTile) {
            const int nt = min(kCondTile, n_cond - c0);
            __syncthreads();
            if (t < nt) {
                // written by block 0 on another SM during this launch: read past the (incoherent) L1
                for (int d = 0; d < dims; d++) s_c[t][d] = __ldcg(cl.centre + (size_t)(off + c0 + t) * dims + d);
                s_r2[t] = __ldcg(cl.radius_sq + off + c0 + t);
                s_pos[t] = __ldcg(cl.subset_pos + off + c0 + t);
                s_lonely[t] = __ldcg(cl.lonely + off + c0 + t);
            }
            __syncthreads();
            if (open) {
                for (int c = 0; c < nt; c++)
                    if (covers(s_c[c], s_r2[c], s_lonely[c], s_pos[c], x, dims, a, my_mask)) { open = false; break; }
            }
        }
        __stcg(flags + rank * kClaimThreads + t, open ? 1 : 0);
        __threadfence();
        cluster.sync();

        // (b) block 0: the survivors of the whole window, in priority order
        if (rank == 0) {
            unsigned open_bits = 0u;
#pragma unroll
            for (int q = 0; q < kItems; q++)
                if (__ldcg(flags + t * kItems + q)) open_bits |= 1u << q;
            for (int guard = 0; guard <= kWindow; guard++) {
                int first = open_bits ? t * kItems + __ffs(open_bits) - 1 : kWindow;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
                __syncthreads();
                if (lane == 0) s_first[warp] = first;
                __syncthreads();
                first = s_first[lane];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
                if (first >= kWindow) break;
                if (first / kItems == t) {
                    const int pos = order[off + w0 + first];
                    const float radius = dist_h[pos];
                    const int lonely = mask_h[pos] > 0;
                    for (int d = 0; d < dims; d++) {
                        const float v = ccoords_h[(size_t)pos * dims + d];
                        s_new_c[d] = v;
                        cl.centre[(size_t)(off + n_cond) * dims + d] = v;
                    }
                    s_new_r2 = __fmul_rn(radius, radius);
                    s_new_pos = pos;
                    s_new_lonely = lonely;
                    cl.radius_sq[off + n_cond] = __fmul_rn(radius, radius);
                    cl.subset_pos[off + n_cond] = pos;
                    cl.lonely[off + n_cond] = lonely;
                    status_h[pos] = 1;
                    alpha_indices[off + n_cond] = original_indices_h[pos];
                    open_bits &= ~(1u << (first - t * kItems));
                }
                __syncthreads();
                unsigned todo = open_bits;
                while (todo) {
                    const int q = __ffs(todo) - 1;
                    todo &= todo - 1;
                    if (t * kItems + q < first) continue;
                    const int pos = order[off + w0 + t * kItems + q];
                    float y[kMaxDims];
#pragma unroll
                    for (int d = 0; d < kMaxDims; d++) y[d] = d < dims ? ccoords_h[(size_t)pos * dims + d] : 0.f;
                    if (covers(s_new_c, s_new_r2, s_new_lonely, s_new_pos, y, dims, pos, mask_h[pos]))
                        open_bits &= ~(1u << q);
                }
                n_cond++;
            }
            __syncthreads();
            if (t == 0) *count = n_cond;
            __threadfence();
        }
        // (c) the longer list becomes visible to all blocks of the cluster
        cluster.sync();
    }
}

__global__ void condensate_totals_kernel(const int *__restrict__ count, int num_rows,
                                         int *__restrict__ n_condensates)
{
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int run = 0;
        n_condensates[0] = 0;
        for (int r = 0; r < num_rows; r++) { run += count[r]; n_condensates[r + 1] = run; }
    }
}

// Step 3.  A block covers 256 consecutive hits, which may straddle events.
__global__ void __launch_bounds__(kAssignThreads)
assign_kernel(int dims, const float *__restrict__ ccoords, const int *__restrict__ mask,
              const int *__restrict__ indices_to_filtered, const int *__restrict__ original_indices_h,
              const int *__restrict__ row_splits, const int *__restrict__ row_splits_h, int num_rows,
              int n_vert, bool by_max_beta, CondList cl, int *__restrict__ assignment,
              int *__restrict__ association)
{
    __shared__ float s_c[kCondTile][kMaxDims];
    __shared__ float s_r2[kCondTile];
    __shared__ int s_pos[kCondTile];
    __shared__ int s_lonely[kCondTile];

    const int v = blockIdx.x * kAssignThreads + threadIdx.x;
    const bool live = v < n_vert;
    float x[kMaxDims];
    int my_mask = 0, my_filtered = -1;
    if (live) {
#pragma unroll
        for (int d = 0; d < kMaxDims; d++) x[d] = d < dims ? ccoords[(size_t)v * dims + d] : 0.f;
        my_mask = mask[v];
        my_filtered = indices_to_filtered[v];
    }
    const int block_first = blockIdx.x * kAssignThreads;
    const int block_last = min(block_first + kAssignThreads, n_vert) - 1;
    // first event that ends after block_first
    int e = 0;
    {
        int lo = 1, hi = num_rows + 1;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (row_splits[mid] <= block_first) lo = mid + 1; else hi = mid;
        }
        e = lo - 1;
    }
    int best = -1, best_pos = -1;
    float min_distance = 10e20f;

    for (; e < num_rows && row_splits[e] <= block_last; e++) {
        const bool mine = live && v >= row_splits[e] && v < row_splits[e + 1];
        const int off = row_splits_h[e], n_cond = cl.count[e];
        bool done = !mine;
        for (int c0 = 0; c0 < n_cond; c0 += kCondTile) {
            const int nt = min(kCondTile, n_cond - c0);
            __syncthreads();
            if (threadIdx.x < nt) {
                const int t = threadIdx.x;
                for (int d = 0; d < dims; d++) s_c[t][d] = cl.centre[(size_t)(off + c0 + t) * dims + d];
                s_r2[t] = cl.radius_sq[off + c0 + t];
                s_pos[t] = cl.subset_pos[off + c0 + t];
                s_lonely[t] = cl.lonely[off + c0 + t];
            }
            __syncthreads();
            if (done) continue;
            for (int c = 0; c < nt; c++) {
                bool covered;
                float dsq = 0.f;
                if (s_lonely[c]) {
                    covered = s_pos[c] == my_filtered;
                    if (covered && !by_max_beta) dsq = centre_distsq(s_c[c], x, dims);
                } else {
                    dsq = centre_distsq(s_c[c], x, dims);
                    covered = my_mask == 0 && dsq <= s_r2[c];
                }
                if (!covered) continue;
                if (by_max_beta) {
                    best = c0 + c; best_pos = s_pos[c];
                    done = true;
                    break;
                }
                if (__fmul_rn(min_distance, s_r2[c]) >= dsq) {
                    best = c0 + c; best_pos = s_pos[c];
                    min_distance = dsq;
                }
            }
        }
    }
    if (live && best >= 0) {
        assignment[v] = best;
        association[v] = original_indices_h[best_pos];
    }
}

}  // namespace

// defined in radix_sort.cu
}  // namespace hgc

using namespace hgc;

namespace {
struct CondBuffers {
    int *beta_keys, *event_keys, *k1, *v1, *k2, *v2, *tk, *tv, *hist, *open_flags;
    CondList cl;
};
template <typename W>
void cond_layout(W &ws, int n_h, int num_rows, int dims, CondBuffers *out)
{
    const size_t n = n_h > 0 ? n_h : 0;
    CondBuffers b;
    b.beta_keys = ws.template take<int>(n);
    b.event_keys = ws.template take<int>(n);
    b.k1 = ws.template take<int>(n); b.v1 = ws.template take<int>(n);
    b.k2 = ws.template take<int>(n); b.v2 = ws.template take<int>(n);
    b.tk = ws.template take<int>(n); b.tv = ws.template take<int>(n);
    b.hist = ws.template take<int>(sort_hist_ints(n_h));
    b.cl.centre = ws.template take<float>(n * (dims > 0 ? dims : 1));
    b.cl.radius_sq = ws.template take<float>(n);
    b.cl.subset_pos = ws.template take<int>(n);
    b.cl.lonely = ws.template take<int>(n);
    b.cl.count = ws.template take<int>(num_rows > 0 ? num_rows : 0);
    b.open_flags = ws.template take<int>((size_t)(num_rows > 0 ? num_rows : 0) * kWindow);
    if (out) *out = b;
}
struct CondSizer {
    Sizer s;
    template <typename T> T *take(size_t n) { s.take<T>(n); return nullptr; }
};
}  // namespace

extern "C" size_t hgc_binned_assign_to_condensates_workspace_bytes(int n_vert, int n_vert_h, int num_rows,
                                                                   int dimensions)
{
    (void)n_vert;
    CondSizer w;
    cond_layout(w, n_vert_h, num_rows, dimensions, nullptr);
    return w.s.used;
}

extern "C" int hgc_binned_assign_to_condensates(
        int dimensions, int dimensions_binning,
        const float *d_ccoords_h, const float *d_dist_h, const float *d_beta_h,
        const int *d_no_condensation_mask_h,
        int *d_high_assigned_status_h,
        const int *d_original_indices_h, const int *d_row_splits_h,
        const float *d_ccoords, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_indices_to_filtered,
        int *d_assignment, int *d_association, int *d_n_condensates, int *d_alpha_indices,
        const int *d_bin_splits, const int *d_n_bins, const float *d_bin_widths,
        const int *d_row_splits, int num_rows, int n_vert, int n_vert_h, int assign_by_max_beta,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    (void)dimensions_binning; (void)d_dist; (void)d_bin_splits; (void)d_n_bins; (void)d_bin_widths;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dimensions < 1 || num_rows < 0 || n_vert < 0 || n_vert_h < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (dimensions > kMaxDims) return HGC_ERR_UNSUPPORTED;
    if (!d_n_condensates || !d_row_splits || !d_row_splits_h) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert > 0 && (!d_ccoords || !d_no_condensation_mask || !d_indices_to_filtered || !d_assignment ||
                       !d_association))
        return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert_h > 0 && (!d_ccoords_h || !d_dist_h || !d_beta_h || !d_no_condensation_mask_h ||
                         !d_high_assigned_status_h || !d_original_indices_h || !d_alpha_indices))
        return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_binned_assign_to_condensates_workspace_bytes(n_vert, n_vert_h, num_rows, dimensions);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    CondBuffers b;
    cond_layout(ws, n_vert_h, num_rows, dimensions, &b);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, sizeof(unsigned), stream));

    const int n_init = n_vert > n_vert_h ? n_vert : n_vert_h;
    if (n_init > 0) {
        init_outputs_kernel<<<div_up(n_init, 256), 256, 0, stream>>>(d_high_assigned_status_h, d_alpha_indices,
                                                                     n_vert_h, d_assignment, d_association, n_vert);
        HGC_LAUNCH_CHECK();
    }
    if (num_rows > 0) HGC_CUDA_TRY(cudaMemsetAsync(b.cl.count, 0, sizeof(int) * (size_t)num_rows, stream));
    if (n_vert_h > 0 && num_rows > 0) {
        priority_keys_kernel<<<div_up(n_vert_h, 256), 256, 0, stream>>>(d_beta_h, d_no_condensation_mask_h,
                                                                        d_row_splits_h, num_rows, n_vert_h,
                                                                        b.beta_keys, b.event_keys);
        HGC_LAUNCH_CHECK();
        // stable sort by priority, then stable sort by event: per event, priority order
        if (int rc = sort_pairs(b.beta_keys, nullptr, b.k1, b.v1, b.tk, b.tv, b.hist, n_vert_h, 32, stream)) return rc;
        gather_int_kernel<<<div_up(n_vert_h, 256), 256, 0, stream>>>(b.event_keys, b.v1, b.k1, n_vert_h);
        HGC_LAUNCH_CHECK();
        if (int rc = sort_pairs(b.k1, b.v1, b.k2, b.v2, b.tk, b.tv, b.hist, n_vert_h, bits_for(num_rows), stream)) return rc;
        claim_kernel<<<num_rows * kClusterBlocks, kClaimThreads, 0, stream>>>(
                dimensions, d_ccoords_h, d_dist_h, d_no_condensation_mask_h, d_original_indices_h, d_row_splits_h,
                b.v2, d_high_assigned_status_h, d_alpha_indices, b.open_flags, b.cl);
        HGC_LAUNCH_CHECK();
    }
    condensate_totals_kernel<<<1, 32, 0, stream>>>(b.cl.count, num_rows, d_n_condensates);
    HGC_LAUNCH_CHECK();
    if (n_vert > 0 && n_vert_h > 0 && num_rows > 0) {
        assign_kernel<<<div_up(n_vert, kAssignThreads), kAssignThreads, 0, stream>>>(
                dimensions, d_ccoords, d_no_condensation_mask, d_indices_to_filtered, d_original_indices_h,
                d_row_splits, d_row_splits_h, num_rows, n_vert, assign_by_max_beta != 0, b.cl, d_assignment,
                d_association);
        HGC_LAUNCH_CHECK();
    }
    return HGC_OK;
}
