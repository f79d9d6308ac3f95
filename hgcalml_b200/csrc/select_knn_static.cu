// BinnedSelectKnn without a caller-provided workspace: the scratch the search needs (one status
// word and the packed coordinates) lives in a fixed array inside the library's device image.
#include <mutex>

#include "common.cuh"
#include "select_knn.cuh"

namespace {

constexpr int kStaticMaxVert = HGC_STATIC_KNN_MAX_VERT;
constexpr int kStaticMaxCoords = HGC_STATIC_KNN_MAX_COORDS;
constexpr int kMaxDevices = 64;
// status word + packed points + two bounding-box arrays (one box per 32 hits), each 256-byte aligned
constexpr size_t kStaticBytes = hgc::kAlign + (size_t)kStaticMaxVert * sizeof(float4) +
                                2 * ((size_t)kStaticMaxVert / 32) * sizeof(float4);

// Every GPU that loads the library carries this array until the process exits (4.25 MiB + 256 B).
// All calls on a device share it and it keeps the previous call's contents.
static __device__ __align__(256) unsigned char g_knn_scratch[kStaticBytes];

// In host code `g_knn_scratch` is only a handle for the runtime, not a device address; the real
// address is asked for once per device, with that device current, and remembered here.  (It stays
// valid for the life of the device's primary context, i.e. until a cudaDeviceReset.)
std::mutex g_mutex;
void *g_device_ptr[kMaxDevices] = {nullptr};

int scratch_for_current_device(void **out)
{
    int dev = -1;
    HGC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return HGC_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_device_ptr[dev] == nullptr) {
        void *p = nullptr;
        HGC_CUDA_TRY(cudaGetSymbolAddress(&p, g_knn_scratch));
        g_device_ptr[dev] = p;
    }
    *out = g_device_ptr[dev];
    return HGC_OK;
}

}  // namespace

using namespace hgc;

extern "C" int hgc_binned_select_knn_static(
        const float *d_coord, const int *d_bin_idx, const int *d_direction, const int *d_dim_bin_idx,
        const int *d_bin_boundaries, const int *d_n_bins, const float *d_bin_width,
        int *d_indices, float *d_dist,
        int n_vert, int n_neigh, int n_coords, int n_bin_dim, int n_bboundaries,
        int tf_compat, int use_direction, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_vert < 0 || n_neigh < 1 || n_bboundaries < 1) return HGC_ERR_INVALID_ARGUMENT;
    if (n_bin_dim < 2 || n_bin_dim > 5 || n_coords < 2) return HGC_ERR_INVALID_ARGUMENT;
    if (n_neigh > 513) return HGC_ERR_UNSUPPORTED;
    // the fixed scratch bounds the problem size
    if (n_vert > kStaticMaxVert || n_coords > kStaticMaxCoords) return HGC_ERR_STATIC_SCRATCH_TOO_SMALL;
    if (n_vert == 0) return HGC_OK;
    if (!d_coord || !d_bin_idx || !d_dim_bin_idx || !d_bin_boundaries || !d_n_bins || !d_bin_width ||
        !d_indices || !d_dist || (use_direction && !d_direction))
        return HGC_ERR_INVALID_ARGUMENT;

    void *scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    Carver ws(scratch);
    // the status word must start at zero; packed points and boxes are rewritten for all n_vert hits
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    const KnnScratch s = knn_scratch_layout(ws, n_vert, n_coords);
    if (int rc = pack_points(d_coord, n_coords, nullptr, s, n_vert, stream)) return rc;
    return launch_select_knn(s, n_coords, d_bin_idx, d_dim_bin_idx, d_bin_boundaries, d_n_bins,
                             d_bin_width, d_direction, d_indices, d_dist, nullptr, nullptr, n_vert,
                             n_neigh, n_bin_dim, n_bboundaries, tf_compat, use_direction != 0,
                             ws.status(), stream);
}

extern "C" int hgc_binned_select_knn_static_status(hgc_stream_t stream_, unsigned *status_out)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!status_out) return HGC_ERR_INVALID_ARGUMENT;
    void *scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    // the status word is the first word of the scratch (Carver::status)
    HGC_CUDA_TRY(cudaMemcpyAsync(status_out, scratch, sizeof(unsigned), cudaMemcpyDeviceToHost, stream));
    HGC_CUDA_TRY(cudaStreamSynchronize(stream));
    return *status_out ? HGC_ERR_DEVICE_STATUS : HGC_OK;
}
