// Shared host/device helpers of the hgcalml_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/hgcalml_b200.h"

namespace hgc {

constexpr int kWarp = 32;
constexpr size_t kAlign = 256;

inline size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

// Bump allocator over the caller's workspace.  The first kAlign bytes hold the status word.
struct Carver {
    char *base;
    size_t used;
    explicit Carver(void *p) : base(static_cast<char *>(p)), used(kAlign) {}
    template <typename T> T *take(size_t n) {
        T *r = reinterpret_cast<T *>(base + used);
        used += align_up(n * sizeof(T));
        return r;
    }
    unsigned *status() const { return reinterpret_cast<unsigned *>(base); }
};

// The same arithmetic without a base pointer, for the *_workspace_bytes queries.
struct Sizer {
    size_t used = kAlign;
    template <typename T> void take(size_t n) { used += align_up(n * sizeof(T)); }
};

void set_cuda_error(cudaError_t e);

#define HGC_CUDA_TRY(expr)                                  \
    do {                                                    \
        cudaError_t hgc_e_ = (expr);                        \
        if (hgc_e_ != cudaSuccess) {                        \
            ::hgc::set_cuda_error(hgc_e_);                  \
            return HGC_ERR_CUDA;                            \
        }                                                   \
    } while (0)

void count_launch();
// Multiprocessors of the calling thread's current device (asked for once per device); sizes persistent grids.
int sm_count();
#define HGC_LAUNCH_CHECK()                   \
    do {                                     \
        ::hgc::count_launch();               \
        HGC_CUDA_TRY(cudaGetLastError());    \
    } while (0)

inline int check_workspace(const void *ws, size_t have, size_t need) {
    if (need == 0) return HGC_OK;
    if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) % kAlign) != 0 || have < need)
        return HGC_ERR_WORKSPACE;
    return HGC_OK;
}

inline int div_up(long long a, long long b) { return (int)((a + b - 1) / b); }

__device__ __forceinline__ void flag_status(unsigned *status, unsigned bit) {
    // Idempotent bit set; a plain racy store of the same value would do, atomicOr keeps other bits.
    if (status) atomicOr(status, bit);
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// ---- internal device-wide primitives (radix_sort.cu) ---------------------------------------

// Stable LSD radix sort of (key, value) pairs on keys in [0, 2^key_bits).  No atomics: per-warp
// digit counters combined by scans, so the result is deterministic.  values_in == nullptr means
// value i = i.  Sorted data ends up in keys_out / vals_out; keys_tmp / vals_tmp are ping-pong
// buffers of n ints each, block_hist has sort_hist_ints(n) ints.  With n_dev (device memory) the
// number of items is min(n, *n_dev): n then only sizes the launches and the tables, so that a count
// produced on the device needs no round trip to the host.
size_t sort_hist_ints(int n);
int sort_pairs(const int *keys_in, const int *vals_in, int *keys_out, int *vals_out,
               int *keys_tmp, int *vals_tmp, int *block_hist, int n, int key_bits,
               cudaStream_t stream, const int *n_dev = nullptr);

// Exclusive prefix sum of `len` ints in place; tile_sums needs scan_scratch_ints(len) ints.
size_t scan_scratch_ints(int len);
int exclusive_scan_ints(int *data, int len, int *tile_sums, cudaStream_t stream);

// bin_boundaries[b] = first position in the ascending key array whose key is >= b, for b in
// [0, n_bins]; keys >= n_bins (sentinels) sort last and are not counted.
int boundaries_from_sorted_keys(const int *sorted_keys, int n, int *bin_boundaries, int n_bins,
                                cudaStream_t stream);

inline int bits_for(long long max_value) {
    int b = 1;
    while ((1LL << b) <= max_value) b++;
    return b;
}

}  // namespace hgc
