// AccumulateKnn: weighted neighbour mean and max (and arg-max) in one pass over the K neighbours.
//
// A group of LPH lanes owns one hit; each lane owns VPL float4 feature columns, so a neighbour row
// of F floats is fetched with one 16-byte load per lane (F=64: 16 lanes, two hits per warp).  The
// group loads the hit's K indices and weights coalesced, LPH at a time, and broadcasts them with
// shuffles; feature rows of a whole chunk are requested before the arithmetic starts, so many
// independent gathers are in flight.  Sums run over the slots in order with separately rounded
// multiply and add, which makes the mean bit-identical to the CPU op
// (modules/compiled/accumulate_knn_kernel.cc:48-81); the max is reset by slot 0 and later slots win
// ties, as there.
#include "common.cuh"

namespace hgc {
namespace {

constexpr int kAccThreads = 256;

template <int LPH, int VPL, bool EXP, bool WITH_ARG>
__global__ void __launch_bounds__(kAccThreads)
accumulate_vec_kernel(const float *__restrict__ weights, const float4 *__restrict__ feat,
                      const int *__restrict__ idxs, float *__restrict__ out, int *__restrict__ out_arg,
                      int n_vert, int K, int F4, int n_out_feat, bool mean_and_max,
                      const int *__restrict__ order, float scale)
{
    constexpr int kGroupsPerBlock = kAccThreads / LPH;
    constexpr int CH = LPH < 8 ? LPH : 8;  // neighbour rows requested before the arithmetic starts
    const int gl = threadIdx.x % LPH;      // lane inside the group
    const int group_in_block = threadIdx.x / LPH;
    const float inv_count = (float)K;

    for (long long g = (long long)blockIdx.x * kGroupsPerBlock + group_in_block;;
         g += (long long)gridDim.x * kGroupsPerBlock) {
        // whole warps leave together: a warp's groups are consecutive g
        const long long warp_first = g - (group_in_block % (kWarp / LPH));
        if (warp_first >= n_vert) break;
        const bool live = g < n_vert;
        const int v = live ? (order ? order[g] : (int)g) : 0;

        float4 sum[VPL], best[VPL];
        int4 arg[VPL];
#pragma unroll
        for (int u = 0; u < VPL; u++) {
            sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            best[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            arg[u] = make_int4(0, 0, 0, 0);
        }

        for (int c0 = 0; c0 < K; c0 += LPH) {
            int my_j = -1;
            float my_w = 0.f;
            if (live && c0 + gl < K) {
                my_j = idxs[(size_t)v * K + c0 + gl];
                my_w = weights[(size_t)v * K + c0 + gl];
                if (EXP) my_w = expf(-__fmul_rn(scale, my_w));
                if (my_j >= n_vert) my_j = -1;
            }
#pragma unroll
            for (int s0 = 0; s0 < LPH; s0 += CH) {
                int j[CH];
                float w[CH];
                float4 f[CH][VPL];
#pragma unroll
                for (int kk = 0; kk < CH; kk++) {
                    j[kk] = __shfl_sync(0xffffffffu, my_j, s0 + kk, LPH);
                    w[kk] = __shfl_sync(0xffffffffu, my_w, s0 + kk, LPH);
#pragma unroll
                    for (int u = 0; u < VPL; u++) {
                        const int vec = gl + u * LPH;
                        f[kk][u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (j[kk] >= 0 && vec < F4) f[kk][u] = __ldg(feat + (size_t)j[kk] * F4 + vec);
                    }
                }
#pragma unroll
                for (int kk = 0; kk < CH; kk++) {
                    if (j[kk] < 0) continue;
                    const bool first = (c0 + s0 + kk) == 0;
#pragma unroll
                    for (int u = 0; u < VPL; u++) {
#define HGC_ACC(comp)                                                           \
    {                                                                           \
        const float t = __fmul_rn(f[kk][u].comp, w[kk]);                        \
        sum[u].comp = __fadd_rn(sum[u].comp, t);                                \
        if (t >= best[u].comp || first) {                                       \
            best[u].comp = t;                                                   \
            if (WITH_ARG) arg[u].comp = j[kk];                                  \
        }                                                                       \
    }
                        HGC_ACC(x) HGC_ACC(y) HGC_ACC(z) HGC_ACC(w)
#undef HGC_ACC
                    }
                }
            }
        }

        if (live) {
#pragma unroll
            for (int u = 0; u < VPL; u++) {
                const int vec = gl + u * LPH;
                if (vec >= F4) continue;
                float4 m;
                m.x = __fdiv_rn(sum[u].x, inv_count);
                m.y = __fdiv_rn(sum[u].y, inv_count);
                m.z = __fdiv_rn(sum[u].z, inv_count);
                m.w = __fdiv_rn(sum[u].w, inv_count);
                float4 *row = reinterpret_cast<float4 *>(out + (size_t)v * n_out_feat);
                row[vec] = m;
                if (mean_and_max) {
                    row[F4 + vec] = best[u];
                    if (WITH_ARG) reinterpret_cast<int4 *>(out_arg + (size_t)v * F4 * 4)[vec] = arg[u];
                }
            }
        }
    }
}

// Any feature count / alignment: one warp per hit, lanes stride over the features.
template <bool EXP>
__global__ void __launch_bounds__(kAccThreads)
accumulate_scalar_kernel(const float *__restrict__ weights, const float *__restrict__ feat,
                         const int *__restrict__ idxs, float *__restrict__ out, int *__restrict__ out_arg,
                         int n_vert, int K, int F, int n_out_feat, bool mean_and_max,
                         const int *__restrict__ order, float scale)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_block = kAccThreads / kWarp;
    for (long long g = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); g < n_vert;
         g += (long long)gridDim.x * warps_per_block) {
        const int v = order ? order[g] : (int)g;
        for (int f = lane; f < F; f += kWarp) {
            float sum = 0.f, best = 0.f;
            int arg = 0;
            for (int s = 0; s < K; s++) {
                const int j = idxs[(size_t)v * K + s];
                if (j < 0 || j >= n_vert) continue;
                float w = weights[(size_t)v * K + s];
                if (EXP) w = expf(-__fmul_rn(scale, w));
                const float t = __fmul_rn(feat[(size_t)j * F + f], w);
                sum = __fadd_rn(sum, t);
                if (t >= best || s == 0) { best = t; arg = j; }
            }
            out[(size_t)v * n_out_feat + f] = __fdiv_rn(sum, (float)K);
            if (mean_and_max) {
                out[(size_t)v * n_out_feat + F + f] = best;
                if (out_arg) out_arg[(size_t)v * F + f] = arg;
            }
        }
    }
}

template <int LPH, int VPL>
int launch_vec(bool exp_w, bool with_arg, const float *w, const float *feat, const int *idxs, float *out,
               int *out_arg, int n_vert, int K, int F4, int n_out, bool mm, const int *order,
               float scale, cudaStream_t stream)
{
    const int groups_per_block = kAccThreads / LPH;
    long long blocks = div_up(n_vert, groups_per_block);
    const long long cap = (long long)kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    const float4 *f4 = reinterpret_cast<const float4 *>(feat);
#define HGC_GO(E, A)                                                                              \
    accumulate_vec_kernel<LPH, VPL, E, A><<<(int)blocks, kAccThreads, 0, stream>>>(               \
            w, f4, idxs, out, out_arg, n_vert, K, F4, n_out, mm, order, scale)
    if (exp_w) { if (with_arg) HGC_GO(true, true); else HGC_GO(true, false); }
    else       { if (with_arg) HGC_GO(false, true); else HGC_GO(false, false); }
#undef HGC_GO
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

int accumulate_dispatch(bool exp_w, const float *w, const float *feat, const int *idxs, float *out,
                        int *out_arg, int n_vert, int K, int F, int n_out, int mean_and_max,
                        const int *order, float scale, cudaStream_t stream)
{
    if (n_vert < 0 || K < 0 || F < 0) return HGC_ERR_INVALID_ARGUMENT;
    if (n_out != (mean_and_max ? 2 * F : F)) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert == 0 || F == 0) return HGC_OK;
    if (!feat || !out || (K > 0 && (!w || !idxs))) return HGC_ERR_INVALID_ARGUMENT;
    const bool mm = mean_and_max != 0;
    const bool with_arg = mm && out_arg != nullptr;
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec_ok = (F % 4 == 0) && F <= 512 && aligned16(feat) && aligned16(out) &&
                        (!with_arg || aligned16(out_arg));
    if (!vec_ok) {
        long long blocks = div_up(n_vert, kAccThreads / kWarp);
        const long long cap = (long long)kNumSMs * 32;
        if (blocks > cap) blocks = cap;
        if (exp_w)
            accumulate_scalar_kernel<true><<<(int)blocks, kAccThreads, 0, stream>>>(
                    w, feat, idxs, out, with_arg ? out_arg : nullptr, n_vert, K, F, n_out, mm, order, scale);
        else
            accumulate_scalar_kernel<false><<<(int)blocks, kAccThreads, 0, stream>>>(
                    w, feat, idxs, out, with_arg ? out_arg : nullptr, n_vert, K, F, n_out, mm, order, scale);
        HGC_LAUNCH_CHECK();
        return HGC_OK;
    }
    const int F4 = F / 4;
#define HGC_VEC(L, V) return launch_vec<L, V>(exp_w, with_arg, w, feat, idxs, out, out_arg, n_vert, K, F4, n_out, mm, order, scale, stream)
    if (F4 <= 4) HGC_VEC(4, 1);
    if (F4 <= 8) HGC_VEC(8, 1);
    if (F4 <= 16) HGC_VEC(16, 1);
    if (F4 <= 32) HGC_VEC(32, 1);
    if (F4 <= 64) HGC_VEC(32, 2);
    HGC_VEC(32, 4);
#undef HGC_VEC
}

}  // namespace
}  // namespace hgc

extern "C" int hgc_accumulate_knn(
        const float *d_weights, const float *d_feat, const int *d_idxs,
        float *d_out_feat, int *d_out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int n_moments, int mean_and_max,
        hgc_stream_t stream)
{
    (void)n_moments;  // read and ignored by the reference too (accumulate_knn_kernel.cc:44)
    return hgc::accumulate_dispatch(false, d_weights, d_feat, d_idxs, d_out_feat, d_out_maxidxs, n_vert,
                                    n_neigh, n_feat, n_out_feat, mean_and_max, nullptr, 1.f,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int hgc_accumulate_knn_exp(
        const float *d_distances, const float *d_feat, const int *d_idxs,
        float *d_out_feat, int *d_out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int mean_and_max,
        float distance_scale, const int *d_order, hgc_stream_t stream)
{
    return hgc::accumulate_dispatch(true, d_distances, d_feat, d_idxs, d_out_feat, d_out_maxidxs, n_vert,
                                    n_neigh, n_feat, n_out_feat, mean_and_max, d_order, distance_scale,
                                    static_cast<cudaStream_t>(stream));
}
