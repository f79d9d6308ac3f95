// BinnedSelectKnn: exact k nearest neighbours inside the query's event, by scanning shells of grid
// bins around the query's bin.
//
// One warp owns one query.  The bins of a shell are turned into ranges of consecutive hits (bins
// that are adjacent along the last binned dimension are contiguous in bin-sorted order), the ranges
// of a shell are laid end to end, and the 32 lanes walk that virtual array 32 candidates at a time,
// reading coordinates as packed float4.  The best K-1 candidates live in registers as a sorted list
// striped over the lanes (rank r in register r/32 of lane r%32), keyed by (distance bits, index) in
// one 64-bit word so ties fall to the lower index.  Candidates that beat the current K-th best are
// parked in a per-warp shared-memory buffer of 32; a full buffer is sorted with a warp-shuffle
// bitonic network and merged into the list.  The candidate set and the stop rule are those of the
// reference (modules/compiled/binned_select_knn_kernel.cc:110-192): shells d = 0,1,2,.. are scanned
// completely, and the search ends after a shell with no bin inside the grid or once the row is full
// and ((bw*d)*bw)*d exceeds the K-th best squared distance.  Distances use separately rounded
// subtract / multiply / add in coordinate order, so they are bit-identical to the CPU op
// (binned_select_knn_kernel.cc:19-29).
#include "common.cuh"
#include "select_knn.cuh"

namespace hgc {
namespace {

typedef unsigned long long u64;
constexpr u64 kInfKey = ~0ull;
constexpr int kKnnWarps = 8;
constexpr int kKnnThreads = kKnnWarps * kWarp;
constexpr int kQueriesPerBlock = 64;  // consecutive bin-sorted queries handled by one block

__device__ __forceinline__ u64 shfl64(u64 v, int src)
{
    return __shfl_sync(0xffffffffu, v, src);
}
__device__ __forceinline__ u64 shfl_xor64(u64 v, int m)
{
    return __shfl_xor_sync(0xffffffffu, v, m);
}
__device__ __forceinline__ u64 min64(u64 a, u64 b) { return a < b ? a : b; }
__device__ __forceinline__ u64 max64(u64 a, u64 b) { return a < b ? b : a; }

// Ascending bitonic sort of one value per lane.
__device__ __forceinline__ u64 warp_sort(u64 v, int lane)
{
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const u64 o = shfl_xor64(v, j);
            const bool up = (lane & k) == 0;      // k == 32: always ascending
            const bool low = (lane & j) == 0;
            v = (low == up) ? min64(v, o) : max64(v, o);
        }
    }
    return v;
}

// Sorts a bitonic sequence (one value per lane) ascending.
__device__ __forceinline__ u64 warp_bitonic_merge(u64 v, int lane)
{
#pragma unroll
    for (int j = 16; j > 0; j >>= 1) {
        const u64 o = shfl_xor64(v, j);
        v = ((lane & j) == 0) ? min64(v, o) : max64(v, o);
    }
    return v;
}

// Merges an ascending block `b` of 32 keys into the ascending striped list, keeping the smallest.
template <int L>
__device__ __forceinline__ void merge_into_list(u64 (&list)[L], u64 b, int lane)
{
#pragma unroll
    for (int r = 0; r < L; r++) {
        // Nothing in b can enter this or any later register when b's minimum is not below the
        // register's maximum... but later registers only hold larger keys, so test each in turn.
        const u64 reg_max = shfl64(list[r], 31);
        const u64 b_min = shfl64(b, 0);
        if (b_min >= reg_max) continue;
        const u64 rev = shfl64(b, 31 - lane);
        const u64 lo = min64(list[r], rev);
        const u64 hi = max64(list[r], rev);
        list[r] = warp_bitonic_merge(lo, lane);
        if (r + 1 < L) b = warp_bitonic_merge(hi, lane);
    }
}

// list[reg] for a runtime `reg`, without indexing the register array dynamically
template <int L>
__device__ __forceinline__ u64 list_reg(const u64 (&list)[L], int reg)
{
    u64 v = list[0];
#pragma unroll
    for (int r = 1; r < L; r++)
        if (r == reg) v = list[r];
    return v;
}

template <int NV4>
struct Point {
    float4 v[NV4];
};

template <int NV4>
__device__ __forceinline__ Point<NV4> load_point(const float4 *__restrict__ pts, int i)
{
    Point<NV4> p;
#pragma unroll
    for (int u = 0; u < NV4; u++) p.v[u] = __ldg(pts + (size_t)i * NV4 + u);
    return p;
}

// sum over coordinates of (a-b)^2, each operation rounded on its own, in coordinate order.  The
// zero padding of the last float4 adds +0 terms, which change nothing.
template <int NV4>
__device__ __forceinline__ float distsq(const Point<NV4> &a, const Point<NV4> &b)
{
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < NV4; u++) {
        float t;
        t = __fsub_rn(a.v[u].x, b.v[u].x); s = __fadd_rn(s, __fmul_rn(t, t));
        t = __fsub_rn(a.v[u].y, b.v[u].y); s = __fadd_rn(s, __fmul_rn(t, t));
        t = __fsub_rn(a.v[u].z, b.v[u].z); s = __fadd_rn(s, __fmul_rn(t, t));
        t = __fsub_rn(a.v[u].w, b.v[u].w); s = __fadd_rn(s, __fmul_rn(t, t));
    }
    return s;
}

struct KnnArgs {
    const float4 *pts;          // [n_vert][NV4] packed, bin-sorted
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
    unsigned *status;
};

template <int NV4, int L, int CB, bool USE_DIR>
__global__ void __launch_bounds__(kKnnThreads) select_knn_kernel(const KnnArgs a)
{
    __shared__ u64 s_buf[kKnnWarps][kWarp];
    __shared__ int s_start[kKnnWarps][kWarp];
    __shared__ int s_end[kKnnWarps][kWarp];  // inclusive prefix of the range lengths

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = a.K;
    const int want = K - 1;  // neighbours besides the query itself
    const float bw = a.bin_width[0];

    int nb[CB], stride[CB];
    {
        int s = 1;
#pragma unroll
        for (int d = CB - 1; d >= 0; d--) { nb[d] = a.n_bins[d]; stride[d] = s; s *= nb[d]; }
    }
    const int bins_per_event = stride[0] * nb[0];

    const int q_begin = blockIdx.x * kQueriesPerBlock;
    const int q_end = min(q_begin + kQueriesPerBlock, a.n_vert);

    for (int i = q_begin + warp; i < q_end; i += kKnnWarps) {
        const int out_row = a.row_map ? a.row_map[i] : i;
        const int self_id = a.id_map ? a.id_map[i] : i;
        int *row_idx = a.out_idx + (size_t)out_row * K;
        float *row_dist = a.out_dist + (size_t)out_row * K;

        u64 list[L];
#pragma unroll
        for (int r = 0; r < L; r++) list[r] = kInfKey;

        bool searching = true;
        if (USE_DIR) {
            const int dir = a.direction[i];
            if (dir == 0 || dir == 2) searching = false;  // may not have neighbours: defaults only
        }

        if (searching && want > 0) {
            const Point<NV4> q = load_point<NV4>(a.pts, i);
            int qb[CB];
#pragma unroll
            for (int d = 0; d < CB; d++) qb[d] = a.dim_bin_idx[(size_t)i * (CB + 1) + 1 + d];
            const int event_offset = bins_per_event * (a.bin_idx[i] / bins_per_event);

            const int thr_reg = (want - 1) / 32, thr_lane = (want - 1) % 32;
            u64 thr = kInfKey;  // key of the current K-th best; everything passes until the row is full
            int buffered = 0;

            // Shells 0 and 1 are always both scanned (the stop rule cannot fire at d = 0), so the
            // first pass covers the whole 3^CB cube; later passes cover one shell each.
            for (int d = 1;; d++) {
                // in-grid extent of the shell's bounding cube in the leading CB-1 dimensions
                int lo[CB], span[CB], cells = 1;
#pragma unroll
                for (int k = 0; k < CB - 1; k++) {
                    lo[k] = max(qb[k] - d, 0);
                    span[k] = min(qb[k] + d, nb[k] - 1) - lo[k] + 1;
                    cells *= span[k];
                }
                const int last_lo = qb[CB - 1] - d, last_hi = qb[CB - 1] + d;
                const int last_lo_c = max(last_lo, 0), last_hi_c = min(last_hi, nb[CB - 1] - 1);
                bool shell_in_grid = false;

                // two range slots per cell: a full row (surface cells, or every cell in the first
                // pass) or the two end bins of the row
                for (int base = 0; base < 2 * cells; base += kWarp) {
                    const int slot = base + lane;
                    int start = 0, len = 0;
                    bool slot_in_grid = false;
                    if (slot < 2 * cells) {
                        int c = slot >> 1, flat = 0;
                        bool surface = d == 1;
#pragma unroll
                        for (int k = CB - 2; k >= 0; k--) {
                            const int g = lo[k] + c % span[k];
                            c /= span[k];
                            flat += g * stride[k];
                            const int off = g - qb[k];
                            surface = surface || off == d || off == -d;
                        }
                        int b0 = -1, b1 = -1;
                        if (surface) {
                            if ((slot & 1) == 0) { b0 = last_lo_c; b1 = last_hi_c; }
                        } else if ((slot & 1) == 0) {
                            if (last_lo >= 0) b0 = b1 = last_lo;
                        } else {
                            if (last_hi < nb[CB - 1]) b0 = b1 = last_hi;
                        }
                        if (b0 >= 0 && b0 <= b1) {
                            const int g0 = event_offset + flat + b0, g1 = event_offset + flat + b1;
                            if (g1 < a.n_bboundaries - 1) {
                                slot_in_grid = true;
                                start = a.bin_boundaries[g0];
                                len = a.bin_boundaries[g1 + 1] - start;
                            } else {
                                flag_status(a.status, HGC_STATUS_FLAT_BIN_OVERFLOW);
                            }
                        }
                    }
                    shell_in_grid = shell_in_grid || __any_sync(0xffffffffu, slot_in_grid);
                    int incl = len;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int t = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += t;
                    }
                    const int total = __shfl_sync(0xffffffffu, incl, 31);
                    if (total == 0) continue;
                    __syncwarp();
                    s_start[warp][lane] = start - (incl - len);  // so that j = s_start[r] + v
                    s_end[warp][lane] = incl;
                    __syncwarp();

                    int r = 0;
                    for (int t0 = 0; t0 < total; t0 += kWarp) {
                        const int v = t0 + lane;
                        bool pass = false;
                        u64 key = kInfKey;
                        if (v < total) {
                            while (v >= s_end[warp][r]) r++;
                            const int j = s_start[warp][r] + v;
                            const Point<NV4> p = load_point<NV4>(a.pts, j);
                            const float ds = distsq<NV4>(q, p);
                            key = ((u64)__float_as_uint(ds) << 32) | (unsigned)j;
                            pass = j != i && key < thr;
                            if (USE_DIR && pass) {
                                const int dj = a.direction[j];
                                pass = !(dj == 1 || dj == 2);
                            }
                        }
                        unsigned m = __ballot_sync(0xffffffffu, pass);
                        if (m == 0u) continue;
                        if (buffered + __popc(m) > kWarp) {
                            __syncwarp();
                            u64 b = lane < buffered ? s_buf[warp][lane] : kInfKey;
                            b = warp_sort(b, lane);
                            merge_into_list<L>(list, b, lane);
                            thr = shfl64(list_reg<L>(list, thr_reg), thr_lane);
                            buffered = 0;
                            pass = pass && key < thr;
                            m = __ballot_sync(0xffffffffu, pass);
                            __syncwarp();
                        }
                        if (pass) s_buf[warp][buffered + __popc(m & ((1u << lane) - 1u))] = key;
                        buffered += __popc(m);
                    }
                }

                // end of shell: fold the parked candidates in, then apply the stop rule
                if (buffered > 0) {
                    __syncwarp();
                    u64 b = lane < buffered ? s_buf[warp][lane] : kInfKey;
                    b = warp_sort(b, lane);
                    merge_into_list<L>(list, b, lane);
                    thr = shfl64(list_reg<L>(list, thr_reg), thr_lane);
                    buffered = 0;
                    __syncwarp();
                }
                if (!shell_in_grid) break;
                if (thr != kInfKey) {
                    const float kth = __uint_as_float((unsigned)(thr >> 32));
                    const float df = (float)d;
                    const float reach = __fmul_rn(__fmul_rn(__fmul_rn(bw, df), bw), df);
                    if (reach > kth) break;
                }
                if (d > (1 << 20)) { flag_status(a.status, HGC_STATUS_ITERATION_CAP); break; }
            }
        }

        // write the row: slot 0 = the query, slots 1.. = list ranks 0.. (ascending)
        const int pad = a.tf_compat ? self_id : -1;
        if (lane == 0) { row_idx[0] = self_id; row_dist[0] = 0.f; }
#pragma unroll
        for (int r = 0; r < L; r++) {
            const int slot = 1 + r * 32 + lane;
            if (slot < K) {
                const u64 key = list[r];
                int id = pad;
                float ds = 0.f;
                if (key != kInfKey) {
                    const int j = (int)(unsigned)(key & 0xffffffffu);
                    id = a.id_map ? a.id_map[j] : j;
                    ds = __uint_as_float((unsigned)(key >> 32));
                }
                row_idx[slot] = id;
                row_dist[slot] = ds;
            }
        }
    }
}

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

template <int NV4, int L, int CB>
int launch_knn3(const KnnArgs &a, bool use_dir, cudaStream_t stream)
{
    const int blocks = div_up(a.n_vert, kQueriesPerBlock);
    if (use_dir) select_knn_kernel<NV4, L, CB, true><<<blocks, kKnnThreads, 0, stream>>>(a);
    else         select_knn_kernel<NV4, L, CB, false><<<blocks, kKnnThreads, 0, stream>>>(a);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

template <int NV4, int L>
int launch_knn2(const KnnArgs &a, int cb, bool use_dir, cudaStream_t stream)
{
    switch (cb) {
        case 2: return launch_knn3<NV4, L, 2>(a, use_dir, stream);
        case 3: return launch_knn3<NV4, L, 3>(a, use_dir, stream);
        case 4: return launch_knn3<NV4, L, 4>(a, use_dir, stream);
        case 5: return launch_knn3<NV4, L, 5>(a, use_dir, stream);
    }
    return HGC_ERR_UNSUPPORTED;
}

template <int NV4>
int launch_knn1(const KnnArgs &a, int cb, bool use_dir, cudaStream_t stream)
{
    const int want = a.K - 1;
    if (want <= 32) return launch_knn2<NV4, 1>(a, cb, use_dir, stream);
    if (want <= 64) return launch_knn2<NV4, 2>(a, cb, use_dir, stream);
    if (want <= 128) return launch_knn2<NV4, 4>(a, cb, use_dir, stream);
    if (want <= 256) return launch_knn2<NV4, 8>(a, cb, use_dir, stream);
    if (want <= 512) return launch_knn2<NV4, 16>(a, cb, use_dir, stream);
    return HGC_ERR_UNSUPPORTED;
}

}  // namespace

int knn_nv4(int n_coords) { return (n_coords + 3) / 4; }

int pack_points(const float *coords, int n_coords, const int *perm, float4 *out, int n_vert,
                cudaStream_t stream)
{
    if (n_vert <= 0) return HGC_OK;
    const int nv4 = knn_nv4(n_coords);
    const long long total = (long long)n_vert * nv4;
    pack_points_kernel<<<div_up(total, 256), 256, 0, stream>>>(coords, n_coords, nv4, perm, out, n_vert);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

int launch_select_knn(const float4 *pts, int n_coords, const int *bin_idx, const int *dim_bin_idx,
                      const int *bin_boundaries, const int *n_bins, const float *bin_width,
                      const int *direction, int *out_idx, float *out_dist, const int *row_map,
                      const int *id_map, int n_vert, int K, int n_bin_dim, int n_bboundaries,
                      int tf_compat, bool use_dir, unsigned *status, cudaStream_t stream)
{
    if (n_vert <= 0) return HGC_OK;
    KnnArgs a;
    a.pts = pts; a.bin_idx = bin_idx; a.dim_bin_idx = dim_bin_idx; a.bin_boundaries = bin_boundaries;
    a.n_bins = n_bins; a.bin_width = bin_width; a.direction = direction;
    a.out_idx = out_idx; a.out_dist = out_dist; a.row_map = row_map; a.id_map = id_map;
    a.n_vert = n_vert; a.K = K; a.n_bboundaries = n_bboundaries; a.tf_compat = tf_compat;
    a.status = status;
    switch (knn_nv4(n_coords)) {
        case 1: return launch_knn1<1>(a, n_bin_dim, use_dir, stream);
        case 2: return launch_knn1<2>(a, n_bin_dim, use_dir, stream);
        case 3: return launch_knn1<3>(a, n_bin_dim, use_dir, stream);
        case 4: return launch_knn1<4>(a, n_bin_dim, use_dir, stream);
    }
    return HGC_ERR_UNSUPPORTED;
}

}  // namespace hgc

using namespace hgc;

extern "C" size_t hgc_binned_select_knn_workspace_bytes(int n_vert, int n_neigh, int n_coords, int n_bin_dim)
{
    (void)n_neigh; (void)n_bin_dim;
    Sizer s;
    s.take<float4>((size_t)(n_vert > 0 ? n_vert : 0) * knn_nv4(n_coords > 0 ? n_coords : 1));
    return s.used;
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
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, sizeof(unsigned), stream));
    float4 *pts = ws.take<float4>((size_t)n_vert * knn_nv4(n_coords));
    if (int rc = pack_points(d_coord, n_coords, nullptr, pts, n_vert, stream)) return rc;
    return launch_select_knn(pts, n_coords, d_bin_idx, d_dim_bin_idx, d_bin_boundaries, d_n_bins,
                             d_bin_width, d_direction, d_indices, d_dist, nullptr, nullptr, n_vert,
                             n_neigh, n_bin_dim, n_bboundaries, tf_compat, use_direction != 0,
                             ws.status(), stream);
}
