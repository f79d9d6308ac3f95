// BinnedSelectKnn search kernel (device code; instantiated per coordinate width in select_knn_nv*.cu).
//
// One warp owns one query.  Work is organised around the reference's candidate set and stop rule
// (modules/compiled/binned_select_knn_kernel.cc:110-192): shells of grid bins at Chebyshev distance
// d = 0,1,2,.. around the query's bin are scanned completely; the search ends after a shell with no
// bin inside the grid, or once the row is full and ((bw*d)*bw)*d exceeds the K-th best squared
// distance.  Within that frame the kernel avoids work that cannot change the result:
//
//  * Bins that are adjacent along the last binned dimension are contiguous in bin-sorted order, so
//    a shell becomes a handful of index ranges.
//  * Every 32 consecutive bin-sorted hits form a chunk with a bounding box over all coordinates
//    (chunk_aabb_kernel).  Long ranges are scanned chunk by chunk, nearest box first, and a chunk
//    is skipped when the box's distance to the query already exceeds the current K-th best: with
//    the same unfused subtract/multiply/add sequence as the point distance, rounding is monotone,
//    so no point of the chunk can have a smaller computed distance than the box.
//  * Short ranges (sparse regions) are laid end to end and walked 64 candidates at a time, two per
//    lane, so that two coordinate loads are in flight per lane.
//  * From the second shell on, bins whose distance to the query's bin already puts them beyond the
//    K-th best are left out of the ranges (the shells are cubes, the K-th best cuts a ball).
//
// The best K-1 candidates live in registers as a sorted list striped over the lanes (rank r in
// register r/32 of lane r%32), keyed by (distance bits, index) in one 64-bit word so that ties
// fall to the lower index.  Candidates that beat the current K-th best are parked in a per-warp
// shared-memory buffer of 64 slots; as soon as 32 are parked they are sorted with a warp-shuffle
// bitonic network and merged into the list, and the rest is filtered against the new K-th best.  Distances are computed with separately rounded operations in coordinate
// order, so they are bit-identical to the CPU op (binned_select_knn_kernel.cc:19-29).
#pragma once
#include "common.cuh"
#include "select_knn.cuh"

namespace hgc {

// A candidate is one 64-bit word: squared-distance bits in the high half, hit index in the low
// half, so that ordering the words orders by (distance, index).  The word is held as a double:
// for non-negative floats in the high half the IEEE-754 order of the doubles equals the order of
// the 64-bit integers (distances are never NaN), and a 64-bit comparison then is one FP64
// instruction instead of a chain of integer compares on the (half-rate, saturated) integer pipe.
typedef double knn_key;
#define HGC_KNN_INF_KEY 1.7976931348623157e308  /* DBL_MAX: above every real key, even distance = +inf */
#ifdef HGC_KNN_STATS
#define HGC_STAT(x) x
#else
#define HGC_STAT(x)
#endif
#ifndef HGC_KNN_FLUSH_AT
#define HGC_KNN_FLUSH_AT 32
#endif
#ifndef HGC_KNN_BINPRUNE
#define HGC_KNN_BINPRUNE 1
#endif
#ifndef HGC_KNN_OFFER2
#define HGC_KNN_OFFER2 1
#endif
static_assert(HGC_KNN_FLUSH_AT >= 1 && HGC_KNN_FLUSH_AT <= 32,
              "a candidate step parks up to 32 keys on top of fewer than HGC_KNN_FLUSH_AT in a 64-slot buffer");
// Resident blocks per SM the kernel is compiled for.  8 blocks of 256 threads leave 32 registers per thread,
// so part of the state spills to (L1-resident) local memory; measured on the 64-event batch that is still
// faster than fewer warps with everything in registers (ms per step at 3 / 4 / 5 / 6 / 7 / 8 blocks:
// 102.0 / 91.7 / 91.4 / 88.8 / 88.0 / 87.8): the kernel is a chain of dependent shuffles and loads, and more
// warps hide more of their latency.
#ifndef HGC_KNN_MIN_BLOCKS
#define HGC_KNN_MIN_BLOCKS 8
#endif
constexpr int kKnnWarps = 8;
constexpr int kKnnThreads = kKnnWarps * kWarp;

__device__ __forceinline__ knn_key make_key(float distsq, int j)
{
    return __hiloint2double((int)__float_as_uint(distsq), j);
}
__device__ __forceinline__ float key_distsq(knn_key k) { return __int_as_float(__double2hiint(k)); }
__device__ __forceinline__ int key_index(knn_key k) { return __double2loint(k); }

__device__ __forceinline__ knn_key shfl_key(knn_key v, int src) { return __shfl_sync(0xffffffffu, v, src); }
__device__ __forceinline__ knn_key shfl_xor_key(knn_key v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }

// Keeps the smaller of (v, o) when `lower`, else the larger.
__device__ __forceinline__ knn_key cmp_exchange(knn_key v, knn_key o, bool lower)
{
    return ((v < o) == lower) ? v : o;
}

// Ascending bitonic sort of one key per lane.  Each merge starts with the mirrored partner, so
// every step is "the lower lane keeps the smaller key" and only five lane-bit tests are needed.
__device__ __forceinline__ knn_key warp_sort(knn_key v, int lane)
{
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
        v = cmp_exchange(v, shfl_xor_key(v, k - 1), (lane & (k >> 1)) == 0);
#pragma unroll
        for (int j = k >> 2; j > 0; j >>= 1) v = cmp_exchange(v, shfl_xor_key(v, j), (lane & j) == 0);
    }
    return v;
}

// Ascending sort of one 32-bit word per lane (same network).
__device__ __forceinline__ unsigned warp_sort_u32(unsigned v, int lane)
{
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
        unsigned o = __shfl_xor_sync(0xffffffffu, v, k - 1);
        v = ((lane & (k >> 1)) == 0) ? min(v, o) : max(v, o);
#pragma unroll
        for (int j = k >> 2; j > 0; j >>= 1) {
            o = __shfl_xor_sync(0xffffffffu, v, j);
            v = ((lane & j) == 0) ? min(v, o) : max(v, o);
        }
    }
    return v;
}

// Sorts a bitonic sequence (one key per lane) ascending.
__device__ __forceinline__ knn_key warp_bitonic_merge(knn_key v, int lane)
{
#pragma unroll
    for (int j = 16; j > 0; j >>= 1) v = cmp_exchange(v, shfl_xor_key(v, j), (lane & j) == 0);
    return v;
}

// Merges an ascending block `b` of 32 keys into the ascending striped list, keeping the smallest.
template <int L>
__device__ __forceinline__ void merge_into_list(knn_key (&list)[L], knn_key b, int lane)
{
#pragma unroll
    for (int r = 0; r < L; r++) {
        // a register whose largest key is not above b's smallest stays as it is
        const knn_key reg_max = shfl_key(list[r], 31);
        const knn_key b_min = shfl_key(b, 0);
        if (b_min >= reg_max) continue;
        const knn_key rev = shfl_xor_key(b, 31);
        const bool keep = list[r] < rev;
        const knn_key lo = keep ? list[r] : rev;
        const knn_key hi = keep ? rev : list[r];
        list[r] = warp_bitonic_merge(lo, lane);
        if (r + 1 < L) b = warp_bitonic_merge(hi, lane);
    }
}

// list[reg] for a runtime `reg`, without indexing the register array dynamically
template <int L>
__device__ __forceinline__ knn_key list_reg(const knn_key (&list)[L], int reg)
{
    knn_key v = list[0];
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
__device__ __forceinline__ Point<NV4> load_point(const float4 *__restrict__ pts, size_t i)
{
    Point<NV4> p;
#pragma unroll
    for (int u = 0; u < NV4; u++) p.v[u] = __ldg(pts + i * NV4 + u);
    return p;
}

// sum over coordinates of (a-b)^2, each operation rounded on its own, in coordinate order.  The
// zero padding of the last float4 adds +0 terms, which change nothing.
// Packed float32x2 subtract / multiply (two individually rounded float32 operations per instruction).
__device__ __forceinline__ float2 sub2(float ax, float ay, float bx, float by)
{
    float2 r;
    asm("{ .reg .b64 ra, rb, rr; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; sub.rn.f32x2 rr, ra, rb; "
        "mov.b64 {%0,%1}, rr; }"
        : "=f"(r.x), "=f"(r.y) : "f"(ax), "f"(ay), "f"(bx), "f"(by));
    return r;
}
__device__ __forceinline__ float2 sqr2(float2 a)
{
    float2 r;
    asm("{ .reg .b64 ra, rr; mov.b64 ra, {%2,%3}; mul.rn.f32x2 rr, ra, ra; mov.b64 {%0,%1}, rr; }"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y));
    return r;
}

template <int NV4>
__device__ __forceinline__ float distsq(const Point<NV4> &a, const Point<NV4> &b)
{
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < NV4; u++) {
        const float2 q01 = sqr2(sub2(a.v[u].x, a.v[u].y, b.v[u].x, b.v[u].y));
        const float2 q23 = sqr2(sub2(a.v[u].z, a.v[u].w, b.v[u].z, b.v[u].w));
        s = __fadd_rn(s, q01.x);
        s = __fadd_rn(s, q01.y);
        s = __fadd_rn(s, q23.x);
        s = __fadd_rn(s, q23.y);
    }
    return s;
}

// Squared distance from q to the box [lo, hi], with the operation sequence of distsq: a lower
// bound of the computed distance to any point inside the box.
__device__ __forceinline__ float gap1(float q, float lo, float hi)
{
    return fmaxf(fmaxf(__fsub_rn(lo, q), __fsub_rn(q, hi)), 0.f);
}
template <int NV4>
__device__ __forceinline__ float box_distsq(const Point<NV4> &q, const float4 *__restrict__ lo,
                                            const float4 *__restrict__ hi, size_t chunk)
{
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < NV4; u++) {
        const float4 l = __ldg(lo + chunk * NV4 + u), h = __ldg(hi + chunk * NV4 + u);
        float g;
        g = gap1(q.v[u].x, l.x, h.x); s = __fadd_rn(s, __fmul_rn(g, g));
        g = gap1(q.v[u].y, l.y, h.y); s = __fadd_rn(s, __fmul_rn(g, g));
        g = gap1(q.v[u].z, l.z, h.z); s = __fadd_rn(s, __fmul_rn(g, g));
        g = gap1(q.v[u].w, l.w, h.w); s = __fadd_rn(s, __fmul_rn(g, g));
    }
    return s;
}

template <int NV4, int L, bool USE_DIR>
struct Query {
    knn_key list[L];
    knn_key thr;        // key of the current K-th best; everything passes until the row is full
    int buffered;
    int thr_reg, thr_lane, lane, self;
    Point<NV4> q;
    knn_key *buf;   // this warp's shared buffer of 64 parked keys
#ifdef HGC_KNN_STATS
    unsigned n_offered, n_accepted, n_flushes, n_steps;  // work counters (tuning aid)
    long long t_flush, t_offer;
#endif
    const float4 *pts;
    const int *direction;

    __device__ __forceinline__ float kth() const
    {
        return thr == HGC_KNN_INF_KEY ? INFINITY : key_distsq(thr);
    }
    // Folds the first 32 parked keys into the list; later ones that still beat the new K-th best
    // move to the front of the buffer.
    __device__ __forceinline__ void flush()
    {
        HGC_STAT(const long long t0 = clock64());
        __syncwarp();
        knn_key b = lane < buffered ? buf[lane] : HGC_KNN_INF_KEY;
        const knn_key rest = (lane + kWarp < buffered) ? buf[lane + kWarp] : HGC_KNN_INF_KEY;
        b = warp_sort(b, lane);
        merge_into_list<L>(list, b, lane);
        thr = shfl_key(list_reg<L>(list, thr_reg), thr_lane);
        const bool keep = rest < thr;
        const unsigned m = __ballot_sync(0xffffffffu, keep);
        if (keep) buf[__popc(m & ((1u << lane) - 1u))] = rest;
        buffered = __popc(m);
        HGC_STAT(n_flushes++);
        __syncwarp();
        HGC_STAT(t_flush += clock64() - t0);
    }
    // One candidate per lane (or none).  Uniform control flow: call with all 32 lanes.
    __device__ __forceinline__ void offer(bool valid, int j)
    {
        HGC_STAT(const long long t0 = clock64(); const long long f0 = t_flush);
        offer_inner(valid, j);
        HGC_STAT(t_offer += (clock64() - t0) - (t_flush - f0));
    }
    // Two candidates per lane: both coordinate loads are issued before either is used, so their
    // latencies overlap (candidates of sparse regions come from many short ranges and miss L1).
    __device__ __forceinline__ void offer2(bool valid0, int j0, bool valid1, int j1)
    {
        HGC_STAT(const long long t0 = clock64(); const long long f0 = t_flush);
        const Point<NV4> p0 = load_point<NV4>(pts, (size_t)(valid0 ? j0 : self));
        const Point<NV4> p1 = load_point<NV4>(pts, (size_t)(valid1 ? j1 : self));
        offer_loaded(valid0, j0, p0);
        if (__any_sync(0xffffffffu, valid1)) offer_loaded(valid1, j1, p1);
        HGC_STAT(t_offer += (clock64() - t0) - (t_flush - f0));
    }
    __device__ __forceinline__ void offer_inner(bool valid, int j)
    {
        offer_loaded(valid, j, load_point<NV4>(pts, (size_t)(valid ? j : self)));
    }
    __device__ __forceinline__ void offer_loaded(bool valid, int j, const Point<NV4> &p)
    {
        bool pass = false;
        knn_key key = HGC_KNN_INF_KEY;
        if (valid) {
            const float ds = distsq<NV4>(q, p);
            key = make_key(ds, j);
            pass = j != self && key < thr;
            if (USE_DIR && pass) {
                const int dj = direction[j];
                pass = !(dj == 1 || dj == 2);
            }
        }
        HGC_STAT(n_steps++);
        HGC_STAT(n_offered += __popc(__ballot_sync(0xffffffffu, valid)));
        const unsigned m = __ballot_sync(0xffffffffu, pass);
        if (m == 0u) return;
        // fewer than 32 keys are parked on entry, so these at most 32 more always fit into the 64 slots
        if (pass) buf[buffered + __popc(m & ((1u << lane) - 1u))] = key;
        buffered += __popc(m);
        HGC_STAT(n_accepted += __popc(m));
        if (buffered >= HGC_KNN_FLUSH_AT) flush();
    }
};

template <int NV4, int L, int CB, bool USE_DIR>
__global__ void __launch_bounds__(kKnnThreads, HGC_KNN_MIN_BLOCKS) select_knn_kernel(const KnnArgs a)
{
    __shared__ knn_key s_buf[kKnnWarps][2 * kWarp];
    __shared__ int s_start[kKnnWarps][kWarp];
    __shared__ int s_end[kKnnWarps][kWarp];  // inclusive prefix of range lengths / chunk counts
    __shared__ int s_rbeg[kKnnWarps][kWarp], s_rend[kKnnWarps][kWarp];

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

    // Warps fetch queries one at a time from one global counter: queries differ a lot in cost (dense
    // shower vs sparse noise), and a fixed assignment leaves warps idle at the end of a block.  The
    // counter also spreads neighbouring queries over all SMs, so that every SM always holds a mix of
    // issue-bound (dense) and latency-bound (sparse) searches; giving a block runs of 16..256
    // consecutive queries instead, so that its warps share candidate chunks in L1, was measured 25-35 %
    // slower on the 200k-hit events.
    for (;;) {
    {
    int run_begin = 0;
    if (lane == 0) run_begin = (int)atomicAdd(a.work_counter, (unsigned)a.fetch);
    run_begin = __shfl_sync(0xffffffffu, run_begin, 0);
    if (run_begin >= a.n_vert) break;
    const int run_end = min(run_begin + a.fetch, a.n_vert);
    for (int i = run_begin; i < run_end; i++) {
        const int out_row = a.row_map ? a.row_map[i] : i;
        const int self_id = a.id_map ? a.id_map[i] : i;
        int *row_idx = a.out_idx + (size_t)out_row * K;
        float *row_dist = a.out_dist + (size_t)out_row * K;

        Query<NV4, L, USE_DIR> Q;
#pragma unroll
        for (int r = 0; r < L; r++) Q.list[r] = HGC_KNN_INF_KEY;
        Q.thr = HGC_KNN_INF_KEY;
        Q.buffered = 0;
        HGC_STAT(Q.n_offered = Q.n_accepted = Q.n_flushes = Q.n_steps = 0; Q.t_flush = Q.t_offer = 0; const long long t_query0 = clock64());
        HGC_STAT(int st_dfinal = 0; unsigned st_boxes = 0; unsigned st_chunks = 0; long long t_enum = 0; long long t_box = 0; long long t_out = 0);
        Q.lane = lane;
        Q.self = i;
        Q.buf = s_buf[warp];
        Q.pts = reinterpret_cast<const float4 *>(a.pts);
        Q.direction = a.direction;
        Q.thr_reg = want > 0 ? (want - 1) / 32 : 0;
        Q.thr_lane = want > 0 ? (want - 1) % 32 : 0;

        bool searching = true;
        if (USE_DIR) {
            const int dir = a.direction[i];
            if (dir == 0 || dir == 2) searching = false;  // may not have neighbours: defaults only
        }

        if (searching && want > 0) {
            Q.q = load_point<NV4>(Q.pts, (size_t)i);
            int qb[CB];
#pragma unroll
            for (int d = 0; d < CB; d++) qb[d] = a.dim_bin_idx[(size_t)i * (CB + 1) + 1 + d];
            const int event_offset = bins_per_event * (a.bin_idx[i] / bins_per_event);

            // Shells 0 and 1 are always both scanned (the stop rule cannot fire at d = 0), so the
            // first pass covers the whole 3^CB cube; later passes cover one shell each.
            for (int d = 1;; d++) {
                HGC_STAT(st_dfinal = d);
                // in-grid extent of the shell's bounding cube in the leading CB-1 dimensions
                int lo[CB], span[CB], cells = 1, centre = 0;
                float inv_span[CB];
#pragma unroll
                for (int k = 0; k < CB - 1; k++) {
                    lo[k] = max(qb[k] - d, 0);
                    span[k] = min(qb[k] + d, nb[k] - 1) - lo[k] + 1;
                    inv_span[k] = __frcp_rn((float)span[k]);
                    centre = centre * span[k] + (qb[k] - lo[k]);
                    cells *= span[k];
                }
                const int last_lo = qb[CB - 1] - d, last_hi = qb[CB - 1] + d;
                const int last_lo_c = max(last_lo, 0), last_hi_c = min(last_hi, nb[CB - 1] - 1);
                bool shell_in_grid = false;

                // two range slots per cell: a full row (surface cells, or every cell in the first
                // pass) or the two end bins of the row.  Cells are visited starting at the query's
                // own row, which tightens the K-th best early.
                for (int base = 0; base < 2 * cells; base += kWarp) {
                    HGC_STAT(const long long te0 = clock64());
                    const int slot = base + lane;
                    int start = 0, len = 0;
                    bool slot_in_grid = false;
                    if (slot < 2 * cells) {
                        int c = (slot >> 1) + centre, flat = 0;
                        if (c >= cells) c -= cells;
                        bool surface = d == 1;
                        float lead_lb = 0.f;  // lower bound of the squared distance from the leading dimensions
#pragma unroll
                        for (int k = CB - 2; k >= 0; k--) {
                            int quot;
                            if (cells <= 4096) {
                                // exact for these sizes: (c + 0.5) / span is at least 0.5/61 away from an integer
                                quot = (int)(((float)c + 0.5f) * inv_span[k]);
                            } else {
                                quot = c / span[k];
                            }
                            const int g = lo[k] + (c - quot * span[k]);
                            c = quot;
                            flat += g * stride[k];
                            const int off = g - qb[k];
                            surface = surface || off == d || off == -d;
                            const float gap = fmaxf((float)abs(off) - 1.01f, 0.f) * bw;
                            lead_lb += gap * gap;
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
                            const int g1 = event_offset + flat + b1;
                            if (g1 < a.n_bboundaries - 1) {
                                slot_in_grid = true;
                                // Beyond the first pass, bins that cannot hold anything closer than the
                                // K-th best are left out.  A hit whose bin is |o| bins from the query's
                                // in one dimension is more than (|o| - 1) bin widths away in it (the
                                // 0.01 bins and the factor on the K-th best absorb the rounding of the
                                // bin arithmetic and of the distances); along the last dimension the
                                // row is cut to the bins the remaining room allows.
                                if (HGC_KNN_BINPRUNE && d >= 2 && Q.thr != HGC_KNN_INF_KEY) {
                                    const float room = Q.kth() * 1.00001f - lead_lb;
                                    if (room < 0.f) {
                                        b1 = b0 - 1;
                                    } else if (room < 1e30f) {
                                        const int omax = (int)(sqrtf(room) / bw + 1.02f);
                                        b0 = max(b0, qb[CB - 1] - omax);
                                        b1 = min(b1, qb[CB - 1] + omax);
                                    }
                                }
                                if (b0 <= b1) {
                                    start = a.bin_boundaries[event_offset + flat + b0];
                                    len = a.bin_boundaries[event_offset + flat + b1 + 1] - start;
                                }
                            } else {
                                flag_status(a.status, HGC_STATUS_FLAT_BIN_OVERFLOW);
                            }
                        }
                    }
                    shell_in_grid = shell_in_grid || __any_sync(0xffffffffu, slot_in_grid);

                    HGC_STAT(t_enum += clock64() - te0);
                    // ---- long ranges: their chunks, all rows together, nearest bounding box first ----
                    const bool is_long = len > a.long_range;
                    if (__any_sync(0xffffffffu, is_long)) {
                        const int n_chunks = is_long ? ((start + len - 1) >> 5) - (start >> 5) + 1 : 0;
                        int cincl = n_chunks;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const int t = __shfl_up_sync(0xffffffffu, cincl, o);
                            if (lane >= o) cincl += t;
                        }
                        const int total_chunks = __shfl_sync(0xffffffffu, cincl, 31);
                        __syncwarp();
                        s_start[warp][lane] = (start >> 5) - (cincl - n_chunks);  // chunk = s_start[r] + v
                        s_end[warp][lane] = cincl;
                        s_rbeg[warp][lane] = start;
                        s_rend[warp][lane] = start + len;
                        __syncwarp();
                        int r = 0;
                        for (int v0 = 0; v0 < total_chunks; v0 += kWarp) {
                            HGC_STAT(const long long tb0 = clock64());
                            const int v = v0 + lane;
                            int chunk = 0, r_begin = 0, r_end = 0;
                            // order word: box distance with its 5 lowest mantissa bits replaced by the lane
                            // (rounding a non-negative float down keeps it a lower bound)
                            unsigned order_key = 0xffffffffu;
                            if (v < total_chunks) {
                                while (v >= s_end[warp][r]) r++;
                                chunk = s_start[warp][r] + v;
                                r_begin = s_rbeg[warp][r];
                                r_end = s_rend[warp][r];
                                const float lb = box_distsq<NV4>(Q.q, a.chunk_lo, a.chunk_hi, (size_t)chunk);
                                if (lb <= Q.kth()) order_key = (__float_as_uint(lb) & ~31u) | (unsigned)lane;
                            }
                            HGC_STAT(st_boxes += min(total_chunks - v0, kWarp));
                            const int alive = __popc(__ballot_sync(0xffffffffu, order_key != 0xffffffffu));
                            if (alive == 0) continue;
                            order_key = warp_sort_u32(order_key, lane);
                            HGC_STAT(t_box += clock64() - tb0);
                            for (int n = 0; n < alive; n++) {
                                const unsigned ok = __shfl_sync(0xffffffffu, order_key, n);
                                if (__uint_as_float(ok & ~31u) > Q.kth()) break;  // sorted: the remaining boxes are farther still
                                const int src = (int)(ok & 31u);
                                const int c = __shfl_sync(0xffffffffu, chunk, src);
                                const int rb = __shfl_sync(0xffffffffu, r_begin, src);
                                const int re = __shfl_sync(0xffffffffu, r_end, src);
                                HGC_STAT(st_chunks++);
                                const int j = (c << 5) + lane;
                                Q.offer(j >= rb && j < re, j);
                            }
                        }
                    }

                    // ---- short ranges: laid end to end, 32 candidates per step ----
                    const int slen = len > a.long_range ? 0 : len;
                    int incl = slen;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int t = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += t;
                    }
                    const int total = __shfl_sync(0xffffffffu, incl, 31);
                    if (total == 0) continue;
                    __syncwarp();
                    s_start[warp][lane] = start - (incl - slen);  // so that j = s_start[r] + v
                    s_end[warp][lane] = incl;
                    __syncwarp();
                    int r = 0;
                    for (int t0 = 0; t0 < total; t0 += (HGC_KNN_OFFER2 ? 2 : 1) * kWarp) {
                        const int v0 = t0 + lane, v1 = HGC_KNN_OFFER2 ? t0 + kWarp + lane : total;
                        int j0 = 0, j1 = 0;
                        if (v0 < total) {
                            while (v0 >= s_end[warp][r]) r++;
                            j0 = s_start[warp][r] + v0;
                        }
                        if (v1 < total) {
                            while (v1 >= s_end[warp][r]) r++;
                            j1 = s_start[warp][r] + v1;
                        }
                        Q.offer2(v0 < total, j0, v1 < total, j1);
                    }
                }

                // end of shell: fold the parked candidates in, then apply the stop rule
                while (Q.buffered > 0) Q.flush();
                if (!shell_in_grid) break;
                if (Q.thr != HGC_KNN_INF_KEY) {
                    const float df = (float)d;
                    const float reach = __fmul_rn(__fmul_rn(__fmul_rn(bw, df), bw), df);
                    if (reach > Q.kth()) break;
                }
                if (d > (1 << 20)) { flag_status(a.status, HGC_STATUS_ITERATION_CAP); break; }
            }
        }

        HGC_STAT(const long long to0 = clock64());
        // write the row: slot 0 = the query, slots 1.. = list ranks 0.. (ascending)
        const int pad = a.tf_compat ? self_id : -1;
        if (lane == 0) { row_idx[0] = self_id; row_dist[0] = 0.f; }
#pragma unroll
        for (int r = 0; r < L; r++) {
            const int slot = 1 + r * 32 + lane;
            if (slot < K) {
                const knn_key key = Q.list[r];
                int id = pad;
                float ds = 0.f;
                if (key != HGC_KNN_INF_KEY) {
                    const int j = key_index(key);
                    id = a.id_map ? a.id_map[j] : j;
                    ds = key_distsq(key);
                }
                row_idx[slot] = id;
                row_dist[slot] = ds;
            }
        }
#ifdef HGC_KNN_STATS
        t_out = clock64() - to0;
        if (a.stats && lane == 0) {
            atomicAdd(&a.stats[0], 1ull);
            atomicAdd(&a.stats[1], (unsigned long long)Q.n_offered);
            atomicAdd(&a.stats[2], (unsigned long long)Q.n_accepted);
            atomicAdd(&a.stats[3], (unsigned long long)Q.n_flushes);
            atomicAdd(&a.stats[4], (unsigned long long)st_boxes);
            atomicAdd(&a.stats[5], (unsigned long long)st_chunks);
            atomicAdd(&a.stats[6], (unsigned long long)Q.n_steps);
            atomicAdd(&a.stats[7], (unsigned long long)(to0 - t_query0));
            atomicAdd(&a.stats[8], (unsigned long long)Q.t_flush);
            atomicAdd(&a.stats[9], (unsigned long long)Q.t_offer);
            atomicAdd(&a.stats[10], (unsigned long long)t_enum);
            atomicAdd(&a.stats[11], (unsigned long long)t_box);
            atomicAdd(&a.stats[12], (unsigned long long)t_out);
            {   // by the shell the search ended in (1..7, 7 = seven or more): queries, candidates, cycles
                const int db = st_dfinal < 7 ? st_dfinal : 7;
                atomicAdd(&a.stats[16 + db], 1ull);
                atomicAdd(&a.stats[24 + db], (unsigned long long)Q.n_offered);
                atomicAdd(&a.stats[32 + db], (unsigned long long)(to0 - t_query0));
                atomicAdd(&a.stats[40 + db], (unsigned long long)Q.n_accepted);
                atomicAdd(&a.stats[48 + db], (unsigned long long)Q.t_flush);
                atomicAdd(&a.stats[56 + db], (unsigned long long)Q.t_offer);
                atomicAdd(&a.stats[64 + db], (unsigned long long)t_enum);
                atomicAdd(&a.stats[72 + db], (unsigned long long)t_box);
                atomicAdd(&a.stats[80 + db], (unsigned long long)Q.n_steps);
                atomicAdd(&a.stats[88 + db], (unsigned long long)st_boxes);
            }
        }
#endif
    }
    }
    }
}

template <int NV4, int L, int CB>
int launch_knn3(const KnnArgs &a, bool use_dir, cudaStream_t stream)
{
    const int blocks = min(div_up(a.n_vert, kKnnWarps * a.fetch), sm_count() * a.blocks_per_sm);
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
int launch_knn_nv(const KnnArgs &a, int cb, bool use_dir, cudaStream_t stream)
{
    const int want = a.K - 1;
    if (want <= 32) return launch_knn2<NV4, 1>(a, cb, use_dir, stream);
    if (want <= 64) return launch_knn2<NV4, 2>(a, cb, use_dir, stream);
    if (want <= 128) return launch_knn2<NV4, 4>(a, cb, use_dir, stream);
    if (want <= 256) return launch_knn2<NV4, 8>(a, cb, use_dir, stream);
    if (want <= 512) return launch_knn2<NV4, 16>(a, cb, use_dir, stream);
    return HGC_ERR_UNSUPPORTED;
}

}  // namespace hgc
