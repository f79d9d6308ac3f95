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

#ifndef HGC_ACC_CH16
#define HGC_ACC_CH16 4
#endif
#ifndef HGC_ACC_MINB16
#define HGC_ACC_MINB16 4
#endif
#ifndef HGC_ACC_THREADS
#define HGC_ACC_THREADS 256
#endif
#ifndef HGC_ACC_TILE
#define HGC_ACC_TILE 512
#endif
constexpr int kAccThreads = HGC_ACC_THREADS;
constexpr int kAccTile = HGC_ACC_TILE;  // consecutive hits a block processes before it jumps to its next tile

// Packed float32x2 arithmetic (two independent, individually rounded float32 operations per
// instruction on sm_100): same results as scalar __fmul_rn / __fadd_rn, half the issue slots.
__device__ __forceinline__ float2 mul2(float2 a, float2 b)
{
    float2 r;
    asm("{ .reg .b64 ra, rb, rr; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; mul.rn.f32x2 rr, ra, rb; "
        "mov.b64 {%0,%1}, rr; }"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b)
{
    float2 r;
    asm("{ .reg .b64 ra, rb, rr; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; add.rn.f32x2 rr, ra, rb; "
        "mov.b64 {%0,%1}, rr; }"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}

template <int LPH, int VPL, int CH, int MINB, bool EXP, bool WITH_ARG>
__global__ void __launch_bounds__(kAccThreads, (MINB * 256 / kAccThreads) > 0 ? (MINB * 256 / kAccThreads) : 1)
accumulate_vec_kernel(const float *__restrict__ weights, const float4 *__restrict__ feat,
                      const int *__restrict__ idxs, float *__restrict__ out, int *__restrict__ out_arg,
                      int n_vert, int K, int ldk, int F4, int n_out_feat, bool mean_and_max,
                      const int *__restrict__ order, float scale, bool sub_self)
{
    constexpr int kGroupsPerBlock = kAccThreads / LPH;
    static_assert(LPH % CH == 0 || CH > LPH, "chunking");
    constexpr int CHN = CH < LPH ? CH : LPH;  // neighbour rows requested before the arithmetic starts
    const int gl = threadIdx.x % LPH;         // lane inside the group
    const int group_in_block = threadIdx.x / LPH;
    const unsigned group_mask = LPH == 32 ? 0xffffffffu : (((1u << LPH) - 1u) << ((threadIdx.x & 31) / LPH * LPH));
    const float inv_count = (float)K;

    // A block walks tiles of kAccTile consecutive hits (of the processing order), kGroupsPerBlock at a
    // time: with a spatially coherent order the neighbour rows of one step are still in L1 for the next.
    constexpr int kStepsPerTile = kAccTile / kGroupsPerBlock;
    const long long n_tiles = ((long long)n_vert + kAccTile - 1) / kAccTile;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x)
    for (int step = 0; step < kStepsPerTile; step++) {
        const long long g0 = tile * kAccTile + (long long)step * kGroupsPerBlock;
        if (g0 >= n_vert) break;  // uniform over the block
        const long long g = g0 + group_in_block;
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

        // indices / weights of the next LPH slots are requested one chunk ahead of their use
        int next_j = -1;
        float next_w = 0.f;
        if (live && gl < K) {
            next_j = idxs[(size_t)v * ldk + gl];
            next_w = weights[(size_t)v * ldk + gl];
        }
        for (int c0 = 0; c0 < K; c0 += LPH) {
            int my_j = next_j;
            float my_w = next_w;
            next_j = -1;
            next_w = 0.f;
            if (live && c0 + LPH + gl < K) {
                next_j = idxs[(size_t)v * ldk + c0 + LPH + gl];
                next_w = weights[(size_t)v * ldk + c0 + LPH + gl];
            }
            if (my_j >= 0) {
                if (EXP) my_w = expf(-__fmul_rn(scale, my_w));
                if (my_j >= n_vert) my_j = -1;
            }
            // A chunk of LPH valid neighbours (the common case) runs without per-neighbour tests.
            const bool dense = (__ballot_sync(0xffffffffu, my_j >= 0) & group_mask) == group_mask;
            if (dense) {
                if (c0 == 0) {
                    // slot 0 is valid, so it resets the running maximum: start below everything
#pragma unroll
                    for (int u = 0; u < VPL; u++) best[u] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                }
#pragma unroll
                for (int s0 = 0; s0 < LPH; s0 += CHN) {
                    int j[CHN];
                    float w[CHN];
                    float4 f[CHN][VPL];
#pragma unroll
                    for (int kk = 0; kk < CHN; kk++) {
                        j[kk] = __shfl_sync(0xffffffffu, my_j, s0 + kk, LPH);
                        w[kk] = __shfl_sync(0xffffffffu, my_w, s0 + kk, LPH);
#pragma unroll
                        for (int u = 0; u < VPL; u++) {
                            const int vec = gl + u * LPH;
                            f[kk][u] = __ldg(feat + (size_t)j[kk] * F4 + (vec < F4 ? vec : 0));
                        }
                    }
#pragma unroll
                    for (int kk = 0; kk < CHN; kk++) {
                        const float2 w2 = make_float2(w[kk], w[kk]);
#pragma unroll
                        for (int u = 0; u < VPL; u++) {
                            const float2 t01 = mul2(make_float2(f[kk][u].x, f[kk][u].y), w2);
                            const float2 t23 = mul2(make_float2(f[kk][u].z, f[kk][u].w), w2);
                            const float2 s01 = add2(make_float2(sum[u].x, sum[u].y), t01);
                            const float2 s23 = add2(make_float2(sum[u].z, sum[u].w), t23);
                            sum[u] = make_float4(s01.x, s01.y, s23.x, s23.y);
#define HGC_MAX(comp, t)                                  \
    if ((t) >= best[u].comp) {                            \
        best[u].comp = (t);                               \
        if (WITH_ARG) arg[u].comp = j[kk];                \
    }
                            HGC_MAX(x, t01.x) HGC_MAX(y, t01.y) HGC_MAX(z, t23.x) HGC_MAX(w, t23.y)
#undef HGC_MAX
                        }
                    }
                }
                continue;
            }
            // chunk with padding (-1) or out-of-range ids: neighbour by neighbour
            for (int kk = 0; kk < LPH; kk++) {
                const int j = __shfl_sync(0xffffffffu, my_j, kk, LPH);
                const float w = __shfl_sync(0xffffffffu, my_w, kk, LPH);
                if (j < 0) continue;
                const bool first = (c0 + kk) == 0;
#pragma unroll
                for (int u = 0; u < VPL; u++) {
                    const int vec = gl + u * LPH;
                    const float4 f = __ldg(feat + (size_t)j * F4 + (vec < F4 ? vec : 0));
#define HGC_ACC(comp)                                                           \
    {                                                                           \
        const float t = __fmul_rn(f.comp, w);                                   \
        sum[u].comp = __fadd_rn(sum[u].comp, t);                                \
        if (t >= best[u].comp || first) {                                       \
            best[u].comp = t;                                                   \
            if (WITH_ARG) arg[u].comp = j;                                      \
        }                                                                       \
    }
                    HGC_ACC(x) HGC_ACC(y) HGC_ACC(z) HGC_ACC(w)
#undef HGC_ACC
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
                float4 mx = best[u];
                if (sub_self) {
                    // the hit's own row is taken off the mean and the max (one rounding each)
                    const float4 own = __ldg(feat + (size_t)v * F4 + vec);
                    m = make_float4(__fsub_rn(m.x, own.x), __fsub_rn(m.y, own.y), __fsub_rn(m.z, own.z), __fsub_rn(m.w, own.w));
                    mx = make_float4(__fsub_rn(mx.x, own.x), __fsub_rn(mx.y, own.y), __fsub_rn(mx.z, own.z), __fsub_rn(mx.w, own.w));
                }
                float4 *row = reinterpret_cast<float4 *>(out + (size_t)v * n_out_feat);
                __stcs(row + vec, m);  // results are written once and not read again by this kernel
                if (mean_and_max) {
                    __stcs(row + F4 + vec, mx);
                    if (WITH_ARG) __stcs(reinterpret_cast<int4 *>(out_arg + (size_t)v * F4 * 4) + vec, arg[u]);
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
                         int n_vert, int K, int ldk, int F, int n_out_feat, bool mean_and_max,
                         const int *__restrict__ order, float scale, bool sub_self)
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
                const int j = idxs[(size_t)v * ldk + s];
                if (j < 0 || j >= n_vert) continue;
                float w = weights[(size_t)v * ldk + s];
                if (EXP) w = expf(-__fmul_rn(scale, w));
                const float t = __fmul_rn(feat[(size_t)j * F + f], w);
                sum = __fadd_rn(sum, t);
                if (t >= best || s == 0) { best = t; arg = j; }
            }
            float mean = __fdiv_rn(sum, (float)K);
            if (sub_self) {
                const float own = feat[(size_t)v * F + f];
                mean = __fsub_rn(mean, own);
                best = __fsub_rn(best, own);
            }
            out[(size_t)v * n_out_feat + f] = mean;
            if (mean_and_max) {
                out[(size_t)v * n_out_feat + F + f] = best;
                if (out_arg) out_arg[(size_t)v * F + f] = arg;
            }
        }
    }
}

template <int LPH, int VPL, int CH, int MINB>
int launch_vec(bool exp_w, bool with_arg, const float *w, const float *feat, const int *idxs, float *out,
               int *out_arg, int n_vert, int K, int ldk, int F4, int n_out, bool mm, const int *order,
               float scale, bool sub_self, cudaStream_t stream)
{
    long long blocks = div_up(n_vert, kAccTile);
    const long long cap = (long long)kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    const float4 *f4 = reinterpret_cast<const float4 *>(feat);
#define HGC_GO(E, A)                                                                              \
    accumulate_vec_kernel<LPH, VPL, CH, MINB, E, A><<<(int)blocks, kAccThreads, 0, stream>>>(     \
            w, f4, idxs, out, out_arg, n_vert, K, ldk, F4, n_out, mm, order, scale, sub_self)
    if (exp_w) { if (with_arg) HGC_GO(true, true); else HGC_GO(true, false); }
    else       { if (with_arg) HGC_GO(false, true); else HGC_GO(false, false); }
#undef HGC_GO
    HGC_LAUNCH_CHECK();
    return HGC_OK;
}

// ldk: row stride of the weight and index arrays (>= K); ld_out: row stride of the output.
int accumulate_dispatch(bool exp_w, const float *w, const float *feat, const int *idxs, float *out,
                        int *out_arg, int n_vert, int K, int ldk, int F, int ld_out, int mean_and_max,
                        const int *order, float scale, bool sub_self, cudaStream_t stream)
{
    if (n_vert < 0 || K < 0 || F < 0 || ldk < K) return HGC_ERR_INVALID_ARGUMENT;
    if (ld_out < (mean_and_max ? 2 * F : F)) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert == 0 || F == 0) return HGC_OK;
    if (!feat || !out || (K > 0 && (!w || !idxs))) return HGC_ERR_INVALID_ARGUMENT;
    const int n_out = ld_out;
    const bool mm = mean_and_max != 0;
    const bool with_arg = mm && out_arg != nullptr;
    auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec_ok = (F % 4 == 0) && (ld_out % 4 == 0) && F <= 512 && aligned16(feat) && aligned16(out) &&
                        (!with_arg || aligned16(out_arg));
    if (!vec_ok) {
        long long blocks = div_up(n_vert, kAccThreads / kWarp);
        const long long cap = (long long)kNumSMs * 32;
        if (blocks > cap) blocks = cap;
        if (exp_w)
            accumulate_scalar_kernel<true><<<(int)blocks, kAccThreads, 0, stream>>>(
                    w, feat, idxs, out, with_arg ? out_arg : nullptr, n_vert, K, ldk, F, n_out, mm, order, scale, sub_self);
        else
            accumulate_scalar_kernel<false><<<(int)blocks, kAccThreads, 0, stream>>>(
                    w, feat, idxs, out, with_arg ? out_arg : nullptr, n_vert, K, ldk, F, n_out, mm, order, scale, sub_self);
        HGC_LAUNCH_CHECK();
        return HGC_OK;
    }
    const int F4 = F / 4;
#define HGC_VEC(L, V, C, M) return launch_vec<L, V, C, M>(exp_w, with_arg, w, feat, idxs, out, out_arg, n_vert, K, ldk, F4, n_out, mm, order, scale, sub_self, stream)
    if (F4 <= 4) HGC_VEC(4, 1, 4, 3);
    if (F4 <= 8) HGC_VEC(8, 1, 4, 3);
    // F = 64: 16 lanes per hit, 4 rows in flight, 4 blocks per SM (64 registers), tiles of 512 hits:
    // measured best on the 64-event batch of {rows in flight / blocks per SM: 8/2, 8/3, 4/3, 4/4, 4/5, 2/4,
    // 2/5, 2/6} and of tiles of 64..2048 hits.  (On a batch of 8 events run back to back, 5 blocks per SM
    // and tiles of 256 looked 6 % faster; on the full batch they are 5 % slower.)
    if (F4 <= 16) HGC_VEC(16, 1, HGC_ACC_CH16, HGC_ACC_MINB16);
    if (F4 <= 32) HGC_VEC(32, 1, 4, 3);
    if (F4 <= 64) HGC_VEC(32, 2, 4, 2);
    HGC_VEC(32, 4, 2, 1);
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
    if (n_out_feat != (mean_and_max ? 2 * n_feat : n_feat)) return HGC_ERR_INVALID_ARGUMENT;
    return hgc::accumulate_dispatch(false, d_weights, d_feat, d_idxs, d_out_feat, d_out_maxidxs, n_vert,
                                    n_neigh, n_neigh, n_feat, n_out_feat, mean_and_max, nullptr, 1.f, false,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int hgc_accumulate_knn_exp(
        const float *d_distances, const float *d_feat, const int *d_idxs,
        float *d_out_feat, int *d_out_maxidxs,
        int n_vert, int n_neigh, int n_feat, int n_out_feat, int mean_and_max,
        float distance_scale, const int *d_order, hgc_stream_t stream)
{
    if (n_out_feat != (mean_and_max ? 2 * n_feat : n_feat)) return HGC_ERR_INVALID_ARGUMENT;
    return hgc::accumulate_dispatch(true, d_distances, d_feat, d_idxs, d_out_feat, d_out_maxidxs, n_vert,
                                    n_neigh, n_neigh, n_feat, n_out_feat, mean_and_max, d_order, distance_scale,
                                    false, static_cast<cudaStream_t>(stream));
}

extern "C" int hgc_gravnet_collect(
        const float *d_distances, const int *d_idxs, int ld_neigh, int first_slot, int n_neigh,
        const float *d_feat, float *d_out, int ld_out, int *d_out_maxidxs,
        int n_vert, int n_feat, float distance_scale, int subtract_self, const int *d_order,
        hgc_stream_t stream)
{
    if (first_slot < 0 || n_neigh < 0 || ld_neigh < first_slot + n_neigh) return HGC_ERR_INVALID_ARGUMENT;
    if (n_vert > 0 && n_neigh > 0 && (!d_distances || !d_idxs)) return HGC_ERR_INVALID_ARGUMENT;
    return hgc::accumulate_dispatch(true, d_distances ? d_distances + first_slot : nullptr, d_feat,
                                    d_idxs ? d_idxs + first_slot : nullptr, d_out, d_out_maxidxs, n_vert,
                                    n_neigh, ld_neigh, n_feat, ld_out, 1, d_order, distance_scale,
                                    subtract_self != 0, static_cast<cudaStream_t>(stream));
}
