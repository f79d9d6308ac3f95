// Atomic-free, stable counting sort of (bin key, hit index) pairs, one 8-bit digit per pass.
//
// Each pass is a counting sort on one digit:
//   1. digit_count_kernel   : every block counts the digits of its tile (per-warp counters,
//                             warp peers found with __match_any_sync, no atomics)
//   2. scan_*_kernel        : exclusive scan of the [digit][block] table (digit-major, so a
//                             digit's blocks are contiguous and block order = input order);
//                             long tables are scanned tile-wise by many blocks
//   3. digit_scatter_kernel : every block recomputes the rank of each item inside its
//                             (warp, digit) run and scatters to its final place.
// A warp owns a contiguous run of its block's tile and walks it 32 items at a time, so equal
// keys keep their input order (the stability that bin-sorted hit order relies on).
#include "common.cuh"

namespace hgc {

namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / kWarp;
constexpr int kRounds = 8;                                   // 32-item rounds per warp
constexpr int kItemsPerWarp = kRounds * kWarp;               // 256
constexpr int kTile = kItemsPerWarp * kSortWarps;            // 2048 items per block
constexpr int kDigits = 256;

__device__ __forceinline__ int digit_of(int key, int shift) { return (key >> shift) & (kDigits - 1); }

__global__ void __launch_bounds__(kSortThreads)
digit_count_kernel(const int *__restrict__ keys, int n_max, const int *__restrict__ n_dev, int shift,
                   int *__restrict__ block_hist, int n_blocks)
{
    // the number of items may sit in device memory (then n_max only sized the grid and the tables)
    const int n = n_dev ? min(n_max, *n_dev) : n_max;
    __shared__ int counts[kSortWarps][kDigits];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int d = threadIdx.x; d < kSortWarps * kDigits; d += kSortThreads) (&counts[0][0])[d] = 0;
    __syncthreads();

    const int warp_base = blockIdx.x * kTile + warp * kItemsPerWarp;
#pragma unroll
    for (int r = 0; r < kRounds; r++) {
        const int i = warp_base + r * kWarp + lane;
        const bool valid = i < n;
        const unsigned active = __ballot_sync(0xffffffffu, valid);
        if (valid) {
            const int dg = digit_of(keys[i], shift);
            const unsigned peers = __match_any_sync(active, dg);
            if ((peers & ((1u << lane) - 1u)) == 0u) counts[warp][dg] += __popc(peers);
        }
        __syncwarp();
    }
    __syncthreads();
    const int dg = threadIdx.x;  // kSortThreads == kDigits
    int total = 0;
#pragma unroll
    for (int w = 0; w < kSortWarps; w++) total += counts[w][dg];
    block_hist[(size_t)dg * n_blocks + blockIdx.x] = total;
}

// Single-block exclusive scan over `len` ints, in place.
__global__ void __launch_bounds__(1024) scan_hist_kernel(int *__restrict__ data, int len)
{
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < len; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < len ? data[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int s = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, s, o);
                if (lane >= o) s += t;
            }
            warp_sums[lane] = s;  // inclusive over warps
        }
        __syncthreads();
        const int carry = carry_s;
        const int warp_excl = warp == 0 ? 0 : warp_sums[warp - 1];
        if (i < len) data[i] = carry + warp_excl + incl - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = carry + warp_excl + incl;
        __syncthreads();
    }
}

// Exclusive scan of a long table in three steps: every block scans its own tile of kScanTile ints
// and records the tile total, one block scans the totals (scan_hist_kernel), the totals are added back.
constexpr int kScanTile = 4096;

__global__ void __launch_bounds__(1024) scan_tiles_kernel(int *__restrict__ data, int len, int *__restrict__ tile_sums)
{
    __shared__ int warp_sums[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int base = blockIdx.x * kScanTile + threadIdx.x * 4;
    int v[4];
#pragma unroll
    for (int q = 0; q < 4; q++) v[q] = base + q < len ? data[base + q] : 0;
    const int mine = v[0] + v[1] + v[2] + v[3];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int s = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += t;
        }
        warp_sums[lane] = s;
    }
    __syncthreads();
    int run = (warp == 0 ? 0 : warp_sums[warp - 1]) + incl - mine;
#pragma unroll
    for (int q = 0; q < 4; q++) {
        if (base + q < len) data[base + q] = run;
        run += v[q];
    }
    if (threadIdx.x == 1023) tile_sums[blockIdx.x] = warp_sums[31];
}

__global__ void add_tile_offsets_kernel(int *__restrict__ data, int len, const int *__restrict__ tile_sums)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < len) data[i] += tile_sums[i / kScanTile];
}

__global__ void __launch_bounds__(kSortThreads)
digit_scatter_kernel(const int *__restrict__ keys_in, const int *__restrict__ vals_in,
                     int *__restrict__ keys_out, int *__restrict__ vals_out, int n_max,
                     const int *__restrict__ n_dev, int shift, const int *__restrict__ block_offsets, int n_blocks)
{
    const int n = n_dev ? min(n_max, *n_dev) : n_max;
    __shared__ int counts[kSortWarps][kDigits];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int d = threadIdx.x; d < kSortWarps * kDigits; d += kSortThreads) (&counts[0][0])[d] = 0;
    __syncthreads();

    int key[kRounds], val[kRounds], rank[kRounds];
    const int warp_base = blockIdx.x * kTile + warp * kItemsPerWarp;
#pragma unroll
    for (int r = 0; r < kRounds; r++) {
        const int i = warp_base + r * kWarp + lane;
        const bool valid = i < n;
        const unsigned active = __ballot_sync(0xffffffffu, valid);
        rank[r] = 0;
        key[r] = 0;
        val[r] = 0;
        if (valid) {
            key[r] = keys_in[i];
            val[r] = vals_in ? vals_in[i] : i;
            const int dg = digit_of(key[r], shift);
            const unsigned peers = __match_any_sync(active, dg);
            const unsigned before = peers & ((1u << lane) - 1u);
            const int seen = counts[warp][dg];  // run length of this digit in earlier rounds
            rank[r] = seen + __popc(before);
            __syncwarp(active);
            if (before == 0u) counts[warp][dg] = seen + __popc(peers);
        }
        __syncwarp();
    }
    __syncthreads();
    {
        const int dg = threadIdx.x;
        int running = block_offsets[(size_t)dg * n_blocks + blockIdx.x];
#pragma unroll
        for (int w = 0; w < kSortWarps; w++) {
            const int c = counts[w][dg];
            counts[w][dg] = running;
            running += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRounds; r++) {
        const int i = warp_base + r * kWarp + lane;
        if (i < n) {
            const int dst = counts[warp][digit_of(key[r], shift)] + rank[r];
            keys_out[dst] = key[r];
            vals_out[dst] = val[r];
        }
    }
}

// One thread per table entry: bounds[b] = number of keys below b = first position whose key is >= b
// (keys are ascending; keys >= n_bins are sentinels that count for no bin).  A binary search per
// entry costs log2(n) cached loads and no thread ever fills a run of empty bins by itself.
__global__ void boundaries_kernel(const int *__restrict__ keys, int n, int *__restrict__ bounds,
                                  int n_bins)
{
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b > n_bins) return;
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (keys[mid] < b) lo = mid + 1; else hi = mid;
    }
    bounds[b] = lo;
}

__global__ void fill_int_kernel(int *__restrict__ p, int n, int v)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

}  // namespace

size_t sort_hist_ints(int n)
{
    const size_t table = (size_t)kDigits * (size_t)div_up(n > 0 ? n : 1, kTile);
    return table + scan_scratch_ints((int)table);  // digit table + its tile totals
}

size_t scan_scratch_ints(int len) { return (size_t)div_up(len > 0 ? len : 1, kScanTile) + 1; }

int exclusive_scan_ints(int *data, int len, int *tile_sums, cudaStream_t stream)
{
    if (len <= 0) return HGC_OK;
    if (len <= 4 * kScanTile) {
        scan_hist_kernel<<<1, 1024, 0, stream>>>(data, len);
        HGC_LAUNCH_CHECK();
        return HGC_OK;
    }
    const int n_tiles = div_up(len, kScanTile);
    scan_tiles_kernel<<<n_tiles, 1024, 0, stream>>>(data, len, tile_sums);
    HGC_LAUNCH_CHECK();
    scan_hist_kernel<<<1, 1024, 0, stream>>>(tile_sums, n_tiles);
    HGC_LAUNCH_CHECK();
    add_tile_offsets_kernel<<<div_up(len, 256), 256, 0, stream>>>(data, len, tile_sums);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

int sort_pairs(const int *keys_in, const int *vals_in, int *keys_out, int *vals_out,
               int *keys_tmp, int *vals_tmp, int *block_hist, int n, int key_bits,
               cudaStream_t stream, const int *n_dev)
{
    if (n <= 0) return HGC_OK;
    const int passes = key_bits <= 0 ? 1 : (key_bits + 7) / 8;
    const int n_blocks = div_up(n, kTile);
    // Choose the ping-pong start so that the last pass lands in keys_out / vals_out.
    int *kbuf[2] = {keys_out, keys_tmp};
    int *vbuf[2] = {vals_out, vals_tmp};
    int dst = (passes & 1) ? 0 : 1;
    const int *src_k = keys_in;
    const int *src_v = vals_in;
    for (int p = 0; p < passes; p++) {
        const int shift = 8 * p;
        digit_count_kernel<<<n_blocks, kSortThreads, 0, stream>>>(src_k, n, n_dev, shift, block_hist, n_blocks);
        HGC_LAUNCH_CHECK();
        const int table = kDigits * n_blocks;
        if (int rc = exclusive_scan_ints(block_hist, table, block_hist + table, stream)) return rc;
        digit_scatter_kernel<<<n_blocks, kSortThreads, 0, stream>>>(src_k, src_v, kbuf[dst], vbuf[dst], n, n_dev,
                                                                    shift, block_hist, n_blocks);
        HGC_LAUNCH_CHECK();
        src_k = kbuf[dst];
        src_v = vbuf[dst];
        dst ^= 1;
    }
    return HGC_OK;
}

int boundaries_from_sorted_keys(const int *sorted_keys, int n, int *bin_boundaries, int n_bins,
                                cudaStream_t stream)
{
    if (n <= 0) {
        fill_int_kernel<<<div_up(n_bins + 1, 256), 256, 0, stream>>>(bin_boundaries, n_bins + 1, 0);
    } else {
        boundaries_kernel<<<div_up(n_bins + 1, 256), 256, 0, stream>>>(sorted_keys, n, bin_boundaries, n_bins);
    }
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

}  // namespace hgc
