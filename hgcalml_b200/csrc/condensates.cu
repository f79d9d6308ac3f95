// BinnedAssignToCondensates on the GPU (the reference has a CPU body only:
// modules/compiled/binned_assign_to_condensates_kernel.cc:23-241).
//
// The reference is a sequential greedy loop per event: take the not-yet-claimed high-beta hit with
// the largest beta (first among equals), make it the next condensate, let it claim the hits inside
// its radius, repeat.  The same result is produced here in three parallel steps:
//   1. priority sort  : the high-beta hits of each event are ordered by (beta descending, position
//                       ascending) with the stable counting sort of radix_sort.cu;
//   2. claim pass     : a cluster of 8 blocks per event walks that order in windows of 8192 hits;
//                       a window is first tested against all condensates confirmed so far
//                       (parallel), then the survivors are settled in order, 32 at a time, each
//                       new condensate closing the later survivors it covers.  A hit is a
//                       condensate exactly when no earlier condensate covers it, which is the
//                       greedy rule;
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
                                     const int *__restrict__ row_splits_h, int num_rows, int n_h_max,
                                     const int *__restrict__ n_h_dev,
                                     int *__restrict__ beta_keys, int *__restrict__ event_keys)
{
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    const int n_h = n_h_dev ? min(n_h_max, *n_h_dev) : n_h_max;
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
                                  int *__restrict__ dst, int n_max, const int *__restrict__ n_dev)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = n_dev ? min(n_max, *n_dev) : n_max;
    if (i < n) dst[i] = src[idx[i]];
}

__global__ void init_outputs_kernel(int *__restrict__ status_h, int *__restrict__ alpha, int n_h,
                                    int *__restrict__ assignment, int *__restrict__ association, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_h) { status_h[i] = 0; alpha[i] = -1; }
    if (i < n) { assignment[i] = -1; association[i] = -1; }
}

// Step 2.  order[] lists, per event, the subset positions in priority order.
//
// A cluster of kClusterBlocks blocks works on one event and walks the priority order in windows of
// kWindow hits, one hit per thread.
//  (a) Every thread tests its hit against the condensates confirmed in earlier windows.
//  (b) The hits still open are settled in batches of the first 32 open ones, in priority order: a
//      prefix sum over the cluster ranks the open hits; the batch goes through a small staging
//      area in global memory to every block; warp i of every block tests batch hit i against the
//      later hits of the batch and every thread then walks the batch in order -- a hit not covered
//      by an earlier condensate of the batch becomes a condensate.  Every thread drops its own hit
//      if one of the new condensates covers it.  (All open hits before a batch member are batch
//      members too, so a new condensate only ever meets later hits, as in the sequential loop.)
// All blocks take the same decisions from the same data, so only the condensate lists that later
// kernels read are published (by block 0).  The barriers are the hardware cluster barrier; every
// block of a cluster runs the same number of windows and batches, so none can be left waiting.
//
// A condensate is held as NR float4: its coordinates and, in the last slot, its squared radius (-1
// for a masked condensate, which covers nothing but itself): NR = 1 up to 3 dimensions, 2 up to 7,
// 3 for 8.
constexpr int kClusterBlocks = 8;
constexpr int kWindow = kClusterBlocks * kClaimThreads;
constexpr int kBatch = 32;
constexpr int kStageInts = 8 + kBatch * (3 * 4 + 2);  // block counts, batch records, positions, flags

template <int NR> struct Rec { float v[NR * 4]; };
template <int NR> __host__ __device__ constexpr int rec_dims() { return NR == 3 ? 8 : NR * 4 - 1; }
template <int NR> __host__ __device__ constexpr int rec_r2_slot() { return NR == 3 ? 8 : NR * 4 - 1; }

template <int NR>
__device__ __forceinline__ Rec<NR> load_rec_shared(const float4 *p)
{
    Rec<NR> r;
#pragma unroll
    for (int u = 0; u < NR; u++) {
        const float4 q = p[u];
        r.v[4 * u] = q.x; r.v[4 * u + 1] = q.y; r.v[4 * u + 2] = q.z; r.v[4 * u + 3] = q.w;
    }
    return r;
}

// Squared distance over the first `dims` slots: subtract, multiply, add, each rounded on its own, in
// coordinate order (the reference's loop, binned_assign_to_condensates_kernel.cc:88-91,103-106).
template <int NR>
__device__ __forceinline__ float rec_distsq(const Rec<NR> &c, const Rec<NR> &x, int dims)
{
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < rec_dims<NR>(); d++)
        if (d < dims) {
            const float t = __fsub_rn(c.v[d], x.v[d]);
            s = __fadd_rn(s, __fmul_rn(t, t));
        }
    return s;
}

template <int NR>
__global__ void __cluster_dims__(kClusterBlocks, 1, 1) __launch_bounds__(kClaimThreads)
claim_kernel(int dims, const float *__restrict__ ccoords_h, const float *__restrict__ dist_h,
             const int *__restrict__ mask_h, const int *__restrict__ original_indices_h,
             const int *__restrict__ row_splits_h, const int *__restrict__ order,
             int *__restrict__ status_h, int *__restrict__ alpha_indices, int *__restrict__ stage_all,
             CondList cl)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float4 s_rec[kCondTile][NR];
    __shared__ float4 s_b[kBatch][NR];
    __shared__ int s_b_pos[kBatch], s_b_flags[kBatch];  // flags: bit 0 = masked condensate, bit 1 = mask != 0
    __shared__ unsigned s_cov[kBatch];
    __shared__ int s_wcnt[32];

    const int rank = (int)cluster.block_rank();
    const int e = blockIdx.x / kClusterBlocks;
    const int off = row_splits_h[e], n_h = row_splits_h[e + 1] - off;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    int *stage_counts = stage_all + (size_t)e * kStageInts;
    float *stage_rec = reinterpret_cast<float *>(stage_counts + 8);
    int *stage_pos = stage_counts + 8 + kBatch * 12;
    int *stage_flags = stage_pos + kBatch;
    int n_cond = 0;

    for (int w0 = 0; w0 < n_h; w0 += kWindow) {
        const int p = w0 + rank * kClaimThreads + t;
        const bool active = p < n_h;
        int a = 0, my_mask = 0;
        Rec<NR> x;
#pragma unroll
        for (int d = 0; d < NR * 4; d++) x.v[d] = 0.f;
        if (active) {
            a = order[off + p];
            my_mask = mask_h[a];
#pragma unroll
            for (int d = 0; d < rec_dims<NR>(); d++)
                if (d < dims) x.v[d] = ccoords_h[(size_t)a * dims + d];
            const float radius = dist_h[a];
            x.v[rec_r2_slot<NR>()] = __fmul_rn(radius, radius);
        }
        bool open = active;

        // (a) against the condensates of earlier windows (written by block 0 on another SM during
        // this launch: read past the incoherent L1)
        for (int c0 = 0; c0 < n_cond; c0 += kCondTile) {
            const int nt = min(kCondTile, n_cond - c0);
            __syncthreads();
            if (t < nt) {
                Rec<NR> r;
#pragma unroll
                for (int d = 0; d < NR * 4; d++) r.v[d] = 0.f;
#pragma unroll
                for (int d = 0; d < rec_dims<NR>(); d++)
                    if (d < dims) r.v[d] = __ldcg(cl.centre + (size_t)(off + c0 + t) * dims + d);
                r.v[rec_r2_slot<NR>()] = __ldcg(cl.lonely + off + c0 + t) ? -1.f : __ldcg(cl.radius_sq + off + c0 + t);
#pragma unroll
                for (int u = 0; u < NR; u++)
                    s_rec[t][u] = make_float4(r.v[4 * u], r.v[4 * u + 1], r.v[4 * u + 2], r.v[4 * u + 3]);
            }
            __syncthreads();
            if (open && my_mask == 0) {
                for (int c = 0; c < nt; c++) {
                    const Rec<NR> r = load_rec_shared<NR>(s_rec[c]);
                    if (rec_distsq<NR>(r, x, dims) <= r.v[rec_r2_slot<NR>()]) { open = false; break; }
                }
            }
        }

        // (b) batches of the first kBatch open hits
        for (int guard = 0; guard <= kWindow; guard++) {
            const unsigned bal = __ballot_sync(0xffffffffu, open);
            // (the shared arrays of the previous round were last read before that round's cluster barriers)
            if (lane == 0) s_wcnt[warp] = __popc(bal);
            __syncthreads();
            const int wv = s_wcnt[lane];
            int wincl = wv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, wincl, o);
                if (lane >= o) wincl += v;
            }
            const int warp_base = __shfl_sync(0xffffffffu, wincl - wv, warp);
            const int blk_total = __shfl_sync(0xffffffffu, wincl, 31);
            if (t == 0) __stcg(stage_counts + rank, blk_total);
            __threadfence();
            cluster.sync();
            int cv = lane < kClusterBlocks ? __ldcg(stage_counts + lane) : 0;
            int cincl = cv;
#pragma unroll
            for (int o = 1; o < kClusterBlocks; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, cincl, o);
                if (lane >= o) cincl += v;
            }
            const int total = __shfl_sync(0xffffffffu, cincl, kClusterBlocks - 1);
            if (total == 0) break;  // the same in every block of the cluster
            const int blk_base = __shfl_sync(0xffffffffu, cincl - cv, rank);
            const int m = min(total, kBatch);
            const int my_r = blk_base + warp_base + __popc(bal & ((1u << lane) - 1u));
            if (open && my_r < kBatch) {
#pragma unroll
                for (int d = 0; d < NR * 4; d++) __stcg(stage_rec + my_r * 12 + d, x.v[d]);
                __stcg(stage_pos + my_r, a);
                __stcg(stage_flags + my_r, (my_mask > 0 ? 1 : 0) | (my_mask != 0 ? 2 : 0));
            }
            __threadfence();
            cluster.sync();
            if (t < m) {
                float v[NR * 4];
#pragma unroll
                for (int d = 0; d < NR * 4; d++) v[d] = __ldcg(stage_rec + t * 12 + d);
#pragma unroll
                for (int u = 0; u < NR; u++) s_b[t][u] = make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
                s_b_pos[t] = __ldcg(stage_pos + t);
                s_b_flags[t] = __ldcg(stage_flags + t);
            }
            __syncthreads();
            if (warp < m) {
                bool cov = false;
                if (lane < m && lane > warp && !(s_b_flags[warp] & 1) && !(s_b_flags[lane] & 2)) {
                    const Rec<NR> ci = load_rec_shared<NR>(s_b[warp]);
                    const Rec<NR> cj = load_rec_shared<NR>(s_b[lane]);
                    cov = rec_distsq<NR>(ci, cj, dims) <= ci.v[rec_r2_slot<NR>()];
                }
                const unsigned cm = __ballot_sync(0xffffffffu, cov);
                if (lane == 0) s_cov[warp] = cm;
            }
            __syncthreads();
            unsigned cond = 0u, dead = 0u;
            for (int i = 0; i < m; i++)
                if (!((dead >> i) & 1u)) {
                    cond |= 1u << i;
                    dead |= s_cov[i];
                }
            if (rank == 0 && warp == 0 && ((cond >> lane) & 1u)) {  // publish the new condensates, in order
                const int slot = off + n_cond + __popc(cond & ((1u << lane) - 1u));
                const int pos = s_b_pos[lane];
                const Rec<NR> c = load_rec_shared<NR>(s_b[lane]);
#pragma unroll
                for (int d = 0; d < rec_dims<NR>(); d++)
                    if (d < dims) cl.centre[(size_t)slot * dims + d] = c.v[d];
                cl.radius_sq[slot] = c.v[rec_r2_slot<NR>()];
                cl.subset_pos[slot] = pos;
                cl.lonely[slot] = s_b_flags[lane] & 1;
                status_h[pos] = 1;
                alpha_indices[slot] = original_indices_h[pos];
            }
            if (open) {
                if (my_r < kBatch) {
                    open = false;  // a batch member is a new condensate or covered by one
                } else if (my_mask == 0) {
                    for (unsigned cm = cond; cm; cm &= cm - 1u) {
                        const int i = __ffs(cm) - 1;
                        if (s_b_flags[i] & 1) continue;  // a masked condensate covers nothing but itself
                        const Rec<NR> c = load_rec_shared<NR>(s_b[i]);
                        if (rec_distsq<NR>(c, x, dims) <= c.v[rec_r2_slot<NR>()]) { open = false; break; }
                    }
                }
            }
            n_cond += __popc(cond);
        }
        // the lists block 0 wrote become visible to the other blocks with the fence and the cluster
        // barrier that end every round of (b), the last one included
    }
    if (rank == 0 && t == 0) cl.count[e] = n_cond;
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

// Step 3.  A block covers 256 consecutive hits, which may straddle events.  Condensates are staged in
// shared memory as in the claim pass (NR float4 each: coordinates and squared radius, -1 for a masked
// condensate).  A hit with a non-zero mask is covered by nothing but itself (if it is a masked
// condensate); those few hits look for their own entry in the position list instead.
template <int NR>
__global__ void __launch_bounds__(kAssignThreads)
assign_kernel(int dims, const float *__restrict__ ccoords, const int *__restrict__ mask,
              const int *__restrict__ indices_to_filtered, const int *__restrict__ original_indices_h,
              const int *__restrict__ row_splits, const int *__restrict__ row_splits_h, int num_rows,
              int n_vert, bool by_max_beta, CondList cl, int *__restrict__ assignment,
              int *__restrict__ association)
{
    __shared__ float4 s_rec[kCondTile][NR];
    __shared__ int s_pos[kCondTile];
    __shared__ int s_lonely[kCondTile];

    const int v = blockIdx.x * kAssignThreads + threadIdx.x;
    const bool live = v < n_vert;
    Rec<NR> x;
#pragma unroll
    for (int d = 0; d < NR * 4; d++) x.v[d] = 0.f;
    int my_mask = 0, my_filtered = -1;
    if (live) {
#pragma unroll
        for (int d = 0; d < rec_dims<NR>(); d++)
            if (d < dims) x.v[d] = ccoords[(size_t)v * dims + d];
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
    int best = -1, best_off = 0;
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
                Rec<NR> r;
#pragma unroll
                for (int d = 0; d < NR * 4; d++) r.v[d] = 0.f;
#pragma unroll
                for (int d = 0; d < rec_dims<NR>(); d++)
                    if (d < dims) r.v[d] = cl.centre[(size_t)(off + c0 + t) * dims + d];
                const int lonely = cl.lonely[off + c0 + t];
                r.v[rec_r2_slot<NR>()] = lonely ? -1.f : cl.radius_sq[off + c0 + t];
#pragma unroll
                for (int u = 0; u < NR; u++)
                    s_rec[t][u] = make_float4(r.v[4 * u], r.v[4 * u + 1], r.v[4 * u + 2], r.v[4 * u + 3]);
                s_pos[t] = cl.subset_pos[off + c0 + t];
                s_lonely[t] = lonely;
            }
            __syncthreads();
            if (done) continue;
            if (my_mask != 0) {
                // only a masked condensate at this very hit covers it
                for (int c = 0; c < nt; c++) {
                    if (!s_lonely[c] || s_pos[c] != my_filtered) continue;
                    if (by_max_beta) {
                        best = c0 + c; best_off = off;
                        done = true;
                        break;
                    }
                    const Rec<NR> r = load_rec_shared<NR>(s_rec[c]);
                    const float dsq = rec_distsq<NR>(r, x, dims);
                    if (__fmul_rn(min_distance, cl.radius_sq[off + c0 + c]) >= dsq) {
                        best = c0 + c; best_off = off;
                        min_distance = dsq;
                    }
                }
                continue;
            }
            for (int c = 0; c < nt; c++) {
                const Rec<NR> r = load_rec_shared<NR>(s_rec[c]);
                const float dsq = rec_distsq<NR>(r, x, dims);
                const float r2 = r.v[rec_r2_slot<NR>()];
                if (!(dsq <= r2)) continue;
                if (by_max_beta) {
                    best = c0 + c; best_off = off;
                    done = true;
                    break;
                }
                if (__fmul_rn(min_distance, r2) >= dsq) {
                    best = c0 + c; best_off = off;
                    min_distance = dsq;
                }
            }
        }
    }
    if (live && best >= 0) {
        assignment[v] = best;
        association[v] = original_indices_h[cl.subset_pos[best_off + best]];
    }
}

}  // namespace

// defined in radix_sort.cu
}  // namespace hgc

using namespace hgc;

namespace {
struct CondBuffers {
    int *beta_keys, *event_keys, *k1, *v1, *k2, *v2, *tk, *tv, *hist, *stage;
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
    b.stage = ws.template take<int>((size_t)(num_rows > 0 ? num_rows : 0) * kStageInts);
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

namespace hgc {
// The op with the number of high-beta hits either exact on the host (d_n_vert_h == nullptr) or in
// device memory (then n_vert_h is an upper bound that sizes workspace and launches).
int assign_to_condensates(
        int dimensions, int dimensions_binning,
        const float *d_ccoords_h, const float *d_dist_h, const float *d_beta_h,
        const int *d_no_condensation_mask_h,
        int *d_high_assigned_status_h,
        const int *d_original_indices_h, const int *d_row_splits_h,
        const float *d_ccoords, const float *d_dist, const int *d_no_condensation_mask,
        const int *d_indices_to_filtered,
        int *d_assignment, int *d_association, int *d_n_condensates, int *d_alpha_indices,
        const int *d_bin_splits, const int *d_n_bins, const float *d_bin_widths,
        const int *d_row_splits, int num_rows, int n_vert, int n_vert_h, const int *d_n_vert_h,
        int assign_by_max_beta, void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
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
                                                                        d_n_vert_h, b.beta_keys, b.event_keys);
        HGC_LAUNCH_CHECK();
        // stable sort by priority, then stable sort by event: per event, priority order
        if (int rc = sort_pairs(b.beta_keys, nullptr, b.k1, b.v1, b.tk, b.tv, b.hist, n_vert_h, 32, stream, d_n_vert_h)) return rc;
        gather_int_kernel<<<div_up(n_vert_h, 256), 256, 0, stream>>>(b.event_keys, b.v1, b.k1, n_vert_h, d_n_vert_h);
        HGC_LAUNCH_CHECK();
        if (int rc = sort_pairs(b.k1, b.v1, b.k2, b.v2, b.tk, b.tv, b.hist, n_vert_h, bits_for(num_rows), stream, d_n_vert_h)) return rc;
#define HGC_CLAIM(NR)                                                                                       \
    claim_kernel<NR><<<num_rows * kClusterBlocks, kClaimThreads, 0, stream>>>(                                \
            dimensions, d_ccoords_h, d_dist_h, d_no_condensation_mask_h, d_original_indices_h, d_row_splits_h, \
            b.v2, d_high_assigned_status_h, d_alpha_indices, b.stage, b.cl)
        if (dimensions <= 3) HGC_CLAIM(1);
        else if (dimensions <= 7) HGC_CLAIM(2);
        else HGC_CLAIM(3);
#undef HGC_CLAIM
        HGC_LAUNCH_CHECK();
    }
    condensate_totals_kernel<<<1, 32, 0, stream>>>(b.cl.count, num_rows, d_n_condensates);
    HGC_LAUNCH_CHECK();
    if (n_vert > 0 && n_vert_h > 0 && num_rows > 0) {
#define HGC_ASSIGN(NR)                                                                                         \
    assign_kernel<NR><<<div_up(n_vert, kAssignThreads), kAssignThreads, 0, stream>>>(                            \
            dimensions, d_ccoords, d_no_condensation_mask, d_indices_to_filtered, d_original_indices_h,          \
            d_row_splits, d_row_splits_h, num_rows, n_vert, assign_by_max_beta != 0, b.cl, d_assignment,         \
            d_association)
        if (dimensions <= 3) HGC_ASSIGN(1);
        else if (dimensions <= 7) HGC_ASSIGN(2);
        else HGC_ASSIGN(3);
#undef HGC_ASSIGN
        HGC_LAUNCH_CHECK();
    }
    return HGC_OK;
}
}  // namespace hgc

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
        void *workspace, size_t workspace_bytes, hgc_stream_t stream)
{
    return hgc::assign_to_condensates(
            dimensions, dimensions_binning, d_ccoords_h, d_dist_h, d_beta_h, d_no_condensation_mask_h,
            d_high_assigned_status_h, d_original_indices_h, d_row_splits_h, d_ccoords, d_dist,
            d_no_condensation_mask, d_indices_to_filtered, d_assignment, d_association, d_n_condensates,
            d_alpha_indices, d_bin_splits, d_n_bins, d_bin_widths, d_row_splits, num_rows, n_vert, n_vert_h,
            nullptr, assign_by_max_beta, workspace, workspace_bytes, stream);
}
