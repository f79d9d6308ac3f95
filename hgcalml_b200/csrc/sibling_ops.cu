// Two small ops that live on the same neighbour tables as the main path and are used by the
// graph-condensation layers: LocalDistance and PushKnn.
#include "common.cuh"
#include "incoming.cuh"

namespace hgc {
namespace {

// Squared distance from hit i to its listed neighbour; 0 for padding and for the hit itself
// (modules/compiled/local_distance_kernel.cc:22-70).  Unfused operations in coordinate order.
__global__ void local_distance_kernel(const int *__restrict__ nidx, const float *__restrict__ coords,
                                      float *__restrict__ dist, int C, int n_in, long long n_edges, int K)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_edges) return;
    const int i = (int)(e / K);
    const int j = nidx[e];
    float s = 0.f;
    if (j >= 0 && j < n_in && j != i) {
        for (int c = 0; c < C; c++) {
            const float t = __fsub_rn(coords[(size_t)i * C + c], coords[(size_t)j * C + c]);
            s = __fadd_rn(s, __fmul_rn(t, t));
        }
    }
    dist[e] = s;
}

// out[m,f] = sum over the edges (i,k) that point at m, in (i,k) order, of feat[i,f] * w[i,k]
// (modules/compiled/push_knn_kernel.cc:35-71; the reference's GPU kernel scatters with atomicAdd,
// push_knn_kernel.cu.cc:61).  One warp per target hit, lanes over the features.
__global__ void __launch_bounds__(256)
push_knn_kernel(const float *__restrict__ weights, const float *__restrict__ feat,
                const int *__restrict__ bounds, const int *__restrict__ sedges, float *__restrict__ out,
                int n_vert, int K, int F)
{
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (m >= n_vert) return;
    const int e_begin = bounds[m], e_end = bounds[m + 1];
    for (int f = lane; f < F; f += 32) {
        float acc = 0.f;
        for (int p = e_begin; p < e_end; p++) {
            const int e = sedges[p];
            const int i = e / K;
            acc = __fadd_rn(acc, __fmul_rn(feat[(size_t)i * F + f], weights[e]));
        }
        out[(size_t)m * F + f] = acc;
    }
}

// PushKnnGrad (modules/compiled/push_knn_grad_kernel.cc:22-95): both parts are gathers.
// feat_grad[i,f] = sum_k grad[m_k,f] * w[i,k]: one warp per hit, lanes over the features, k in order.
__global__ void __launch_bounds__(256)
push_grad_features_kernel(const float *__restrict__ grad, const float *__restrict__ weights,
                          const int *__restrict__ nidx, float *__restrict__ feat_grad, int n_vert, int K, int F)
{
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= n_vert) return;
    for (int f = lane; f < F; f += 32) {
        float acc = 0.f;
        for (int k = 0; k < K; k++) {
            const int m = nidx[(size_t)i * K + k];
            if (m < 0 || m >= n_vert) continue;
            acc = __fadd_rn(acc, __fmul_rn(grad[(size_t)m * F + f], weights[(size_t)i * K + k]));
        }
        feat_grad[(size_t)i * F + f] = acc;
    }
}

// w_grad[i,k] = sum_f grad[m_k,f] * feat[i,f]: one thread per (hit, slot), f in order.
__global__ void __launch_bounds__(256)
push_grad_weights_kernel(const float *__restrict__ grad, const float *__restrict__ feat,
                         const int *__restrict__ nidx, float *__restrict__ w_grad, long long n_edges,
                         int n_vert, int K, int F)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_edges) return;
    const int m = nidx[e];
    float acc = 0.f;
    if (m >= 0 && m < n_vert) {
        const int i = (int)(e / K);
        for (int f = 0; f < F; f++)
            acc = __fadd_rn(acc, __fmul_rn(__ldg(grad + (size_t)m * F + f), feat[(size_t)i * F + f]));
    }
    w_grad[e] = acc;
}

}  // namespace
}  // namespace hgc

using namespace hgc;

extern "C" int hgc_push_knn_grad(
        const float *d_grad, const float *d_weights, const float *d_feat, const int *d_idxs,
        float *d_feat_grad, float *d_w_grad, int n_vert, int n_neigh, int n_feat, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_vert < 0 || n_neigh < 0 || n_feat < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert == 0) return HGC_OK;
    const long long ne = (long long)n_vert * n_neigh;
    if (n_feat > 0 && (!d_grad || !d_feat || !d_feat_grad)) return HGC_ERR_INVALID_ARGUMENT;
    if (ne > 0 && (!d_weights || !d_idxs || !d_w_grad)) return HGC_ERR_INVALID_ARGUMENT;
    if (n_feat > 0) {
        push_grad_features_kernel<<<div_up(n_vert, 8), 256, 0, stream>>>(d_grad, d_weights, d_idxs, d_feat_grad,
                                                                        n_vert, n_neigh, n_feat);
        HGC_LAUNCH_CHECK();
    }
    if (ne > 0) {
        push_grad_weights_kernel<<<div_up(ne, 256), 256, 0, stream>>>(d_grad, d_feat, d_idxs, d_w_grad, ne, n_vert,
                                                                     n_neigh, n_feat);
        HGC_LAUNCH_CHECK();
    }
    return HGC_OK;
}

extern "C" int hgc_local_distance(
        const int *d_neigh_idxs, const float *d_coords, float *d_distances,
        int n_coords, int n_in_vert, int n_out_vert, int n_neigh, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_coords < 0 || n_in_vert < 0 || n_out_vert < 0 || n_neigh < 0 || n_out_vert > n_in_vert)
        return HGC_ERR_INVALID_ARGUMENT;
    const long long ne = (long long)n_out_vert * n_neigh;
    if (ne == 0) return HGC_OK;
    if (!d_neigh_idxs || !d_distances || (n_coords > 0 && !d_coords)) return HGC_ERR_INVALID_ARGUMENT;
    local_distance_kernel<<<div_up(ne, 256), 256, 0, stream>>>(d_neigh_idxs, d_coords, d_distances, n_coords,
                                                              n_in_vert, ne, n_neigh);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

extern "C" int hgc_push_knn(
        const float *d_weights, const float *d_feat, const int *d_idxs, float *d_out_feat,
        int n_vert, int n_neigh, int n_feat, void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n_vert < 0 || n_neigh < 0 || n_feat < 0) return HGC_ERR_INVALID_ARGUMENT;
    if ((long long)n_vert * n_neigh >= (1LL << 31) - 4096) return HGC_ERR_UNSUPPORTED;
    if (n_vert == 0 || n_feat == 0) return HGC_OK;
    if (!d_feat || !d_out_feat || (n_neigh > 0 && (!d_weights || !d_idxs))) return HGC_ERR_INVALID_ARGUMENT;
    if (n_neigh == 0) {
        HGC_CUDA_TRY(cudaMemsetAsync(d_out_feat, 0, sizeof(float) * (size_t)n_vert * n_feat, stream));
        return HGC_OK;
    }
    const size_t need = hgc_knn_grad_workspace_bytes(n_vert, n_neigh);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    const Incoming b = incoming_layout(ws, n_vert, n_neigh);
    if (int rc = build_incoming(d_idxs, n_vert, n_neigh, b, stream)) return rc;
    push_knn_kernel<<<div_up(n_vert, 8), 256, 0, stream>>>(d_weights, d_feat, b.bounds, b.sedges, d_out_feat,
                                                          n_vert, n_neigh, n_feat);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}
