// Backward ops of the neighbour path: AccumulateKnnGrad and SelectKnnGrad.
//
// Both ops push gradients from a hit to its neighbours.  The reference's GPU kernels do that with
// float atomicAdd (modules/compiled/accumulate_knn_grad_kernel.cu.cc:102,
// select_knn_grad_kernel.cu.cc:139), so their sums depend on scheduling.  Here the neighbour lists
// are transposed first: the (hit, slot) edges are ordered by their target with the stable counting
// sort of radix_sort.cu, which gives every hit the list of edges that point at it, in ascending
// (hit, slot) order.  Each target then sums its incoming contributions itself, in that fixed
// order -- no atomics, run-to-run identical, and for AccumulateKnnGrad the same order as the
// reference's CPU loop, so the result is bit-identical to it.
#include "common.cuh"
#include "incoming.cuh"
#include "../../include/hgcalml_b200.h"

namespace hgc {
namespace {

__global__ void edge_target_keys_kernel(const int *__restrict__ nidx, long long n_edges, int n_vert,
                                        int *__restrict__ keys)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_edges) return;
    const int m = nidx[e];
    keys[e] = (m >= 0 && m < n_vert) ? m : n_vert;  // sentinel: sorts last, belongs to no hit
}

// ---- AccumulateKnnGrad: gradient w.r.t. the features ------------------------------------------
// One warp per target hit m; lanes stride over the features, so the rows of grad_out and of the
// arg-max table are read coalesced.  Follows modules/compiled/accumulate_knn_grad_kernel.cc:36-99.
template <int FPL>  // features per lane: lane, lane+32, ..
__global__ void __launch_bounds__(256)
acc_grad_features_kernel(const float *__restrict__ grad_out, const float *__restrict__ weights,
                         const int *__restrict__ max_idx, const int *__restrict__ nidx,
                         const int *__restrict__ bounds, const int *__restrict__ sedges,
                         float *__restrict__ grad_feat, int n_vert, int K, int F, int G, bool mean_and_max,
                         const int *__restrict__ order)
{
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (slot >= n_vert) return;
    const int m = order ? order[slot] : slot;  // processing order only: every target is visited once
    const int e_begin = bounds[m], e_end = bounds[m + 1];
    const float kf = (float)K;
    constexpr int U = 4;  // edges whose rows are requested together (the sum still runs edge by edge)
    for (int f0 = 0; f0 < F; f0 += 32 * FPL) {
        float acc[FPL];
#pragma unroll
        for (int u = 0; u < FPL; u++) acc[u] = 0.f;
        for (int pw = e_begin; pw < e_end; pw += 32) {
            // the warp fetches 32 edges and their weights at once, then hands them round by shuffle
            const int my_p = pw + lane;
            const int my_e = my_p < e_end ? sedges[my_p] : 0;
            const float my_w = my_p < e_end ? weights[my_e] : 0.f;
            const int n_here = min(32, e_end - pw);
            for (int q0 = 0; q0 < n_here; q0 += U) {
                int ii[U];
                float ww[U], g[U][FPL];
                int am[U][FPL];
#pragma unroll
                for (int q = 0; q < U; q++) {
                    const int src = min(q0 + q, n_here - 1);
                    const int e = __shfl_sync(0xffffffffu, my_e, src);
                    ww[q] = __shfl_sync(0xffffffffu, my_w, src);
                    ii[q] = e / K;
#pragma unroll
                    for (int u = 0; u < FPL; u++) {
                        const int f = f0 + u * 32 + lane;
                        g[q][u] = 0.f;
                        am[q][u] = -1;
                        if (f < F) {
                            g[q][u] = grad_out[(size_t)ii[q] * G + f];
                            if (mean_and_max) am[q][u] = max_idx[(size_t)ii[q] * F + f];
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < U; q++) {
                    if (q0 + q >= n_here) break;  // uniform
                    const int i = ii[q];
                    const float w = ww[q];
                    bool counts_for_max = true;
                    if (i == m) {
                        // the hit is its own neighbour: only its first occurrence in the row counts for the max
                        const int k = __shfl_sync(0xffffffffu, my_e, q0 + q) - i * K;
                        bool earlier = false;
                        for (int kk = lane; kk < k; kk += 32) earlier = earlier || nidx[(size_t)i * K + kk] == i;
                        counts_for_max = !__any_sync(0xffffffffu, earlier);
                    }
#pragma unroll
                    for (int u = 0; u < FPL; u++) {
                        const int f = f0 + u * 32 + lane;
                        if (f < F) {
                            const float mean_part = __fmul_rn(__fdiv_rn(g[q][u], kf), w);
                            float max_part = 0.f;
                            if (mean_and_max && counts_for_max && am[q][u] == m)
                                max_part = __fmul_rn(grad_out[(size_t)i * G + F + f], w);
                            acc[u] = __fadd_rn(acc[u], __fadd_rn(mean_part, max_part));
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < FPL; u++) {
            const int f = f0 + u * 32 + lane;
            if (f < F) grad_feat[(size_t)m * F + f] = acc[u];
        }
    }
}

// ---- AccumulateKnnGrad: gradient w.r.t. the weights --------------------------------------------
// One thread per (hit, slot); the sum over the features runs in order
// (modules/compiled/accumulate_knn_grad_kernel.cc:101-163).
__global__ void __launch_bounds__(256)
acc_grad_weights_kernel(const float *__restrict__ grad_out, const float *__restrict__ feat,
                        const int *__restrict__ max_idx, const int *__restrict__ nidx,
                        float *__restrict__ grad_w, long long n_edges, int n_vert, int K, int F, int G,
                        bool mean_and_max, bool vec4, const int *__restrict__ order)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_edges) return;
    const int row = (int)(t / K);
    const int i = order ? order[row] : row;  // processing order only
    const long long e = (long long)i * K + (t - (long long)row * K);
    const int m = nidx[e];
    if (m < 0 || m >= n_vert) { grad_w[e] = 0.f; return; }
    const float *g = grad_out + (size_t)i * G;
    const float *x = feat + (size_t)m * F;
    const int *am = max_idx + (size_t)i * F;
    float mean_part = 0.f, max_part = 0.f;
    if (vec4) {
        // rows are 16-byte aligned: four features per load, summed in feature order all the same
        for (int f = 0; f < F; f += 4) {
            const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + f));
            const float4 gv = *reinterpret_cast<const float4 *>(g + f);
            mean_part = __fadd_rn(mean_part, __fmul_rn(gv.x, xv.x));
            mean_part = __fadd_rn(mean_part, __fmul_rn(gv.y, xv.y));
            mean_part = __fadd_rn(mean_part, __fmul_rn(gv.z, xv.z));
            mean_part = __fadd_rn(mean_part, __fmul_rn(gv.w, xv.w));
            if (mean_and_max) {
                const int4 av = *reinterpret_cast<const int4 *>(am + f);
                if (av.x == m || av.y == m || av.z == m || av.w == m) {
                    const float4 hv = *reinterpret_cast<const float4 *>(g + F + f);
                    if (av.x == m) max_part = __fadd_rn(max_part, __fmul_rn(hv.x, xv.x));
                    if (av.y == m) max_part = __fadd_rn(max_part, __fmul_rn(hv.y, xv.y));
                    if (av.z == m) max_part = __fadd_rn(max_part, __fmul_rn(hv.z, xv.z));
                    if (av.w == m) max_part = __fadd_rn(max_part, __fmul_rn(hv.w, xv.w));
                }
            }
        }
    } else {
        for (int f = 0; f < F; f++) {
            const float xf = __ldg(x + f);
            mean_part = __fadd_rn(mean_part, __fmul_rn(g[f], xf));
            if (mean_and_max && am[f] == m) max_part = __fadd_rn(max_part, __fmul_rn(g[F + f], xf));
        }
    }
    // the reference scales by the double 1./(float)K
    mean_part = (float)__dmul_rn((double)mean_part, 1.0 / (double)(float)K);
    grad_w[e] = __fadd_rn(mean_part, max_part);
}

// ---- SelectKnnGrad ------------------------------------------------------------------------------
// One thread per (hit, coordinate): its own part first, in the reference's mixed float/double
// arithmetic (modules/compiled/select_knn_grad_kernel.cu.cc:81-118), then the parts pushed to it by
// the hits that list it as a neighbour (:120-165), in (hit, slot) order instead of atomics.
__global__ void __launch_bounds__(256)
select_grad_kernel(const float *__restrict__ grad_dist, const int *__restrict__ nidx,
                   const float *__restrict__ coord, const int *__restrict__ bounds,
                   const int *__restrict__ sedges, float *__restrict__ grad_coord, int n_vert, int K, int C)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)n_vert * C) return;
    const int m = (int)(t / C), c = (int)(t - (long long)m * C);
    const float xm = coord[t];
    float val = 0.f;
    for (int k = 0; k < K; k++) {
        const int j = nidx[(size_t)m * K + k];
        if (j < 0 || j >= n_vert) continue;
        const float g = grad_dist[(size_t)m * K + k];
        const float d = __fsub_rn(coord[(size_t)j * C + c], xm);
        // separately rounded double operations, as the host compiler evaluates the reference expression
        val = (float)__dsub_rn((double)val, __dmul_rn(__dmul_rn(2.0, (double)g), (double)d));
    }
    for (int p = bounds[m]; p < bounds[m + 1]; p++) {
        const int e = sedges[p];
        const int i = e / K;
        const float d = __fsub_rn(xm, coord[(size_t)i * C + c]);
        const float add = (float)__dmul_rn(__dmul_rn(2.0, (double)grad_dist[e]), (double)d);
        val = __fadd_rn(val, add);
    }
    grad_coord[t] = val;
}

}  // namespace

int build_incoming(const int *nidx, int n_vert, int n_neigh, const Incoming &b, cudaStream_t stream)
{
    const long long ne = (long long)n_vert * n_neigh;
    edge_target_keys_kernel<<<div_up(ne, 256), 256, 0, stream>>>(nidx, ne, n_vert, b.keys);
    HGC_LAUNCH_CHECK();
    if (int rc = sort_pairs(b.keys, nullptr, b.skeys, b.sedges, b.tkeys, b.tvals, b.hist, (int)ne,
                            bits_for(n_vert), stream))
        return rc;
    return boundaries_from_sorted_keys(b.skeys, (int)ne, b.bounds, n_vert, stream);
}

}  // namespace hgc

using namespace hgc;

extern "C" size_t hgc_knn_grad_workspace_bytes(int n_vert, int n_neigh)
{
    IncomingSizer w;
    incoming_layout(w, n_vert, n_neigh);
    return w.s.used;
}

static int check_edge_count(int n_vert, int n_neigh)
{
    if (n_vert < 0 || n_neigh < 0) return HGC_ERR_INVALID_ARGUMENT;
    if ((long long)n_vert * n_neigh >= (1LL << 31) - 4096) return HGC_ERR_UNSUPPORTED;
    return HGC_OK;
}

extern "C" int hgc_accumulate_knn_grad(
        const float *d_grad_from_out_features, const float *d_distances, const float *d_feat,
        const int *d_max_feat_indices, const int *d_neigh_indices,
        float *d_out_grad_distances, float *d_out_grad_features,
        int n_vert, int n_neigh, int n_feat, int n_grad_from_out_feat, int n_moments, int mean_and_max,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    return hgc_accumulate_knn_grad_ordered(d_grad_from_out_features, d_distances, d_feat, d_max_feat_indices,
                                           d_neigh_indices, d_out_grad_distances, d_out_grad_features, n_vert,
                                           n_neigh, n_feat, n_grad_from_out_feat, n_moments, mean_and_max,
                                           nullptr, workspace, workspace_bytes, stream_);
}

extern "C" int hgc_accumulate_knn_grad_ordered(
        const float *d_grad_from_out_features, const float *d_distances, const float *d_feat,
        const int *d_max_feat_indices, const int *d_neigh_indices,
        float *d_out_grad_distances, float *d_out_grad_features,
        int n_vert, int n_neigh, int n_feat, int n_grad_from_out_feat, int n_moments, int mean_and_max,
        const int *d_order, void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    (void)n_moments;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_edge_count(n_vert, n_neigh)) return rc;
    if (n_feat < 0 || n_grad_from_out_feat != (mean_and_max ? 2 * n_feat : n_feat)) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert == 0) return HGC_OK;
    if (n_feat > 0 && (!d_grad_from_out_features || !d_feat || !d_out_grad_features ||
                       (mean_and_max && !d_max_feat_indices)))
        return HGC_ERR_INVALID_ARGUMENT;
    if (n_neigh > 0 && (!d_distances || !d_neigh_indices || !d_out_grad_distances)) return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_knn_grad_workspace_bytes(n_vert, n_neigh);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    const Incoming b = incoming_layout(ws, n_vert, n_neigh);
    if (n_neigh == 0) {
        if (n_feat > 0)
            HGC_CUDA_TRY(cudaMemsetAsync(d_out_grad_features, 0, sizeof(float) * (size_t)n_vert * n_feat, stream));
        return HGC_OK;
    }
    if (int rc = build_incoming(d_neigh_indices, n_vert, n_neigh, b, stream)) return rc;
    if (n_feat > 0) {
#define HGC_FEAT(FPL)                                                                               \
    acc_grad_features_kernel<FPL><<<div_up(n_vert, 8), 256, 0, stream>>>(                           \
            d_grad_from_out_features, d_distances, d_max_feat_indices, d_neigh_indices, b.bounds, b.sedges, \
            d_out_grad_features, n_vert, n_neigh, n_feat, n_grad_from_out_feat, mean_and_max != 0, d_order)
        if (n_feat <= 32) HGC_FEAT(1);
        else if (n_feat <= 64) HGC_FEAT(2);
        else HGC_FEAT(4);
#undef HGC_FEAT
        HGC_LAUNCH_CHECK();
    }
    const long long ne = (long long)n_vert * n_neigh;
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec4 = n_feat % 4 == 0 && aligned16(d_feat) && aligned16(d_grad_from_out_features) &&
                      (!mean_and_max || aligned16(d_max_feat_indices));
    acc_grad_weights_kernel<<<div_up(ne, 256), 256, 0, stream>>>(
            d_grad_from_out_features, d_feat, d_max_feat_indices, d_neigh_indices, d_out_grad_distances, ne,
            n_vert, n_neigh, n_feat, n_grad_from_out_feat, mean_and_max != 0, vec4, d_order);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

extern "C" int hgc_select_knn_grad(
        const float *d_grad_dist, const int *d_indices, const float *d_dist, const float *d_coord,
        float *d_grad_coord, int n_vert, int n_neigh, int n_coords,
        void *workspace, size_t workspace_bytes, hgc_stream_t stream_)
{
    (void)d_dist;  // an input of the op that its kernels never read
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_edge_count(n_vert, n_neigh)) return rc;
    if (n_coords < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert == 0 || n_coords == 0) return HGC_OK;
    if (!d_coord || !d_grad_coord || (n_neigh > 0 && (!d_grad_dist || !d_indices))) return HGC_ERR_INVALID_ARGUMENT;
    const size_t need = hgc_knn_grad_workspace_bytes(n_vert, n_neigh);
    if (int rc = check_workspace(workspace, workspace_bytes, need)) return rc;
    Carver ws(workspace);
    HGC_CUDA_TRY(cudaMemsetAsync(ws.status(), 0, kAlign, stream));
    const Incoming b = incoming_layout(ws, n_vert, n_neigh);
    if (n_neigh == 0) {
        HGC_CUDA_TRY(cudaMemsetAsync(d_grad_coord, 0, sizeof(float) * (size_t)n_vert * n_coords, stream));
        return HGC_OK;
    }
    if (int rc = build_incoming(d_indices, n_vert, n_neigh, b, stream)) return rc;
    const long long total = (long long)n_vert * n_coords;
    select_grad_kernel<<<div_up(total, 256), 256, 0, stream>>>(d_grad_dist, d_indices, d_coord, b.bounds, b.sedges,
                                                              d_grad_coord, n_vert, n_neigh, n_coords);
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}
