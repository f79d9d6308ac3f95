// Error reporting, the workspace status word, and IndexReplacer.
#include <atomic>
#include "common.cuh"

namespace hgc {

static thread_local cudaError_t t_last_cuda_error = cudaSuccess;

void set_cuda_error(cudaError_t e) { t_last_cuda_error = e; }

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int sm_count()
{
    constexpr int kMaxDevices = 64, kDefault = 148;  // 148: B200, used only if the query fails
    static std::atomic<int> cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kDefault;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kDefault;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

namespace {

// replaced[i] = replacements[to_be_replaced[i]]; negative entries pass through; entries beyond
// the table stay unwritten (modules/compiled/index_replacer_kernel.cc:28-41).
__global__ void index_replacer_kernel(const int *__restrict__ to_be_replaced,
                                      const int *__restrict__ replacements, int *__restrict__ replaced,
                                      int n, int n_replacements, unsigned *status)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = to_be_replaced[i];
    if (r < 0) replaced[i] = r;
    else if (r < n_replacements) replaced[i] = replacements[r];
    else flag_status(status, HGC_STATUS_INDEX_OUT_OF_RANGE);
}

}  // namespace
}  // namespace hgc

using namespace hgc;

extern "C" const char *hgc_strerror(int code)
{
    switch (code) {
        case HGC_OK: return "ok";
        case HGC_ERR_INVALID_ARGUMENT: return "invalid argument";
        case HGC_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case HGC_ERR_UNSUPPORTED: return "outside the limits of this library";
        case HGC_ERR_CUDA: return "CUDA runtime error";
        case HGC_ERR_DEVICE_STATUS: return "device status word is non-zero";
        case HGC_ERR_STATIC_SCRATCH_TOO_SMALL: return "problem exceeds the built-in scratch of this entry point";
    }
    return "unknown error code";
}

extern "C" const char *hgc_last_cuda_error(void) { return cudaGetErrorString(t_last_cuda_error); }

extern "C" int hgc_version(void) { return 100; }

extern "C" unsigned long long hgc_launch_count(void) { return hgc::g_launches.load(); }

extern "C" int hgc_workspace_status(const void *workspace, hgc_stream_t stream_, unsigned *status_out)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!workspace || !status_out) return HGC_ERR_INVALID_ARGUMENT;
    unsigned s = 0;
    HGC_CUDA_TRY(cudaMemcpyAsync(&s, workspace, sizeof(unsigned), cudaMemcpyDeviceToHost, stream));
    HGC_CUDA_TRY(cudaStreamSynchronize(stream));
    *status_out = s;
    return s ? HGC_ERR_DEVICE_STATUS : HGC_OK;
}

extern "C" int hgc_index_replacer(
        const int *d_to_be_replaced, const int *d_replacements, int *d_replaced,
        int n_to_be_replaced, int n_replacements, unsigned *d_status, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_to_be_replaced < 0 || n_replacements < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (n_to_be_replaced == 0) return HGC_OK;
    if (!d_to_be_replaced || !d_replaced || (n_replacements > 0 && !d_replacements))
        return HGC_ERR_INVALID_ARGUMENT;
    index_replacer_kernel<<<div_up(n_to_be_replaced, 256), 256, 0, stream>>>(
            d_to_be_replaced, d_replacements, d_replaced, n_to_be_replaced, n_replacements, d_status);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}
