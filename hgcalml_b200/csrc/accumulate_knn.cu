// AccumulateKnn: weighted neighbour mean and max (and arg-max) in one pass over the K neighbours.
//
// A group of LPH lanes owns one hit; each lane owns VPL float4 feature columns, so a neighbour row
// of F floats is fetched with VPL 16-byte loads per lane (F=64: 8 lanes x 2 loads, four hits per
// warp; the eight lanes of a quarter warp read one 128-byte line per load, which is what the L1
// data stage moves per cycle).  The group loads the hit's K indices and weights coalesced, LPH at a
// time, and broadcasts them with shuffles; the feature rows of a chunk are requested before the
// arithmetic starts, so many independent gathers are in flight.  Sums run over the slots in order
// with separately rounded multiply and add (packed two per instruction), which makes the mean
// bit-identical to the CPU op (modules/compiled/accumulate_knn_kernel.cc:48-81).  The max is reset
// by slot 0 and later slots win ties, as there; it is taken two slots at a time with the
// three-input max, and the arg-max is kept as the SLOT of the last neighbour that equals the new
// maximum (a float, updated with multiply-adds so that it costs no compare/select pair per
// product); the neighbour id is looked up once at the end.
#include "common.cuh"

namespace hgc {
namespace {

#ifndef HGC_ACC_TILE_STEPS
#define HGC_ACC_TILE_STEPS 8
#endif
// consecutive steps (of THREADS/LPH hits each) a block processes before it jumps to its next tile
constexpr int kAccTileSteps = HGC_ACC_TILE_STEPS;
constexpr int kAccThreads = 256;  // block size of the scalar fallback

typedef unsigned long long f32x2;  // two float32 in one 64-bit register

// Packed float32x2 arithmetic (two independent, individually rounded float32 operations per
// instruction on sm_100): same results as scalar __fmul_rn / __fadd_rn, half the issue slots.
__device__ __forceinline__ f32x2 pack2(float a, float b)
{
    f32x2 r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &a, float &b)
{
    asm("mov.b64 {%0,%1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// max(a, b, c) in one instruction (sm_100); a NaN operand is ignored, as by the CPU op's `>=`.
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// 1.0f where a == b, else 0.0f
__device__ __forceinline__ float set_eq(float a, float b)
{
    float r;
    asm("set.eq.f32.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// EXACT: the row has exactly LPH * VPL float4 (then the row width is a compile-time constant and no
// lane is idle).
template <int LPH, int VPL, int CH, int THREADS, int MINB, bool EXP, bool WITH_ARG, bool EXACT>
__global__ void __launch_bounds__(THREADS, MINB)
accumulate_vec_kernel(const float *__restrict__ weights, const float4 *__restrict__ feat,
                      const int *__restrict__ idxs, float *__restrict__ out, int *__restrict__ out_arg,
                      int n_vert, int K, int ldk, int F4_arg, int n_out_feat, bool mean_and_max,
                      const int *__restrict__ order, float scale, bool sub_self)
{
    const int F4 = EXACT ? LPH * VPL : F4_arg;
    constexpr int G = THREADS / LPH;  // hits a block works on at a time
    constexpr int NP = VPL * 2;       // packed pairs per lane per row
    constexpr int NE = VPL * 4;       // floats per lane per row
    static_assert(LPH % CH == 0 && CH % 2 == 0, "rows are requested CH at a time and processed in pairs");
    const int gl = threadIdx.x % LPH;  // lane inside the group
    const int grp = threadIdx.x / LPH;
    const float inv_count = (float)K;
    // float4 column of this lane's u-th vector; lanes beyond the row read column 0 and store nothing
    int col[VPL];
#pragma unroll
    for (int u = 0; u < VPL; u++) col[u] = (EXACT || (gl + u * LPH) < F4) ? (gl + u * LPH) : 0;

    // A block walks tiles of kAccTileSteps * G consecutive hits (of the processing order), G at a
    // time, and the grid moves over the batch tile by tile: with a spatially coherent order the
    // neighbour rows of one step are still in L1 for the next, and all blocks work inside one
    // window of the batch at any time.
    const long long total_steps = ((long long)n_vert + G - 1) / G;
    const long long n_tiles = (total_steps + kAccTileSteps - 1) / kAccTileSteps;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x)
    for (int ts = 0; ts < kAccTileSteps; ts++) {
        const long long step = tile * kAccTileSteps + ts;
        if (step >= total_steps) break;  // uniform over the block
        const long long g = step * G + grp;
        const bool live = g < n_vert;
        const int v = live ? (order ? order[g] : (int)g) : 0;

        f32x2 sum[NP], argslot[NP];  // argslot: slot of the running arg-max as a float, -1 = none yet
        float best[NE];
#pragma unroll
        for (int e = 0; e < NP; e++) { sum[e] = 0ull; argslot[e] = pack2(-1.f, -1.f); }
#pragma unroll
        for (int e = 0; e < NE; e++) best[e] = 0.f;

        // indices / weights of the next LPH slots are requested one chunk ahead of their use; they
        // are read once, so they should not displace feature rows from L1
        int next_j = -1;
        float next_w = 0.f;
        if (live && gl < K) {
            next_j = __ldcs(idxs + (size_t)v * ldk + gl);
            next_w = __ldcs(weights + (size_t)v * ldk + gl);
        }
        for (int c0 = 0; c0 < K; c0 += LPH) {
            int my_j = next_j;
            float my_w = next_w;
            next_j = -1;
            next_w = 0.f;
            if (live && c0 + LPH + gl < K) {
                next_j = __ldcs(idxs + (size_t)v * ldk + c0 + LPH + gl);
                next_w = __ldcs(weights + (size_t)v * ldk + c0 + LPH + gl);
            }
            if (my_j >= 0) {
                if (EXP) my_w = expf(-__fmul_rn(scale, my_w));
                if (my_j >= n_vert) my_j = -1;
            }
            // A chunk in which every hit of the warp has LPH valid neighbours (the common case) runs
            // without per-neighbour tests.  The decision is taken for the whole warp, so every
            // shuffle below is executed by all 32 lanes together.
            const bool dense = __all_sync(0xffffffffu, my_j >= 0);
            if (dense) {
                if (c0 == 0) {
                    // slot 0 is valid, so it resets the running maximum: start below everything
#pragma unroll
                    for (int e = 0; e < NE; e++) best[e] = -INFINITY;
                }
                const float cf = (float)c0;
#pragma unroll
                for (int s0 = 0; s0 < LPH; s0 += CH) {
                    f32x2 f[CH][NP];
                    float w[CH];
#pragma unroll
                    for (int kk = 0; kk < CH; kk++) {
                        const int j = __shfl_sync(0xffffffffu, my_j, s0 + kk, LPH);
                        w[kk] = __shfl_sync(0xffffffffu, my_w, s0 + kk, LPH);
#pragma unroll
                        for (int u = 0; u < VPL; u++) {
                            const float4 *p = feat + (size_t)j * F4 + col[u];
                            asm volatile("ld.global.nc.v2.b64 {%0,%1}, [%2];"
                                         : "=l"(f[kk][2 * u]), "=l"(f[kk][2 * u + 1]) : "l"(p));
                        }
                    }
#pragma unroll
                    for (int kk = 0; kk < CH; kk += 2) {
                        const f32x2 w0 = pack2(w[kk], w[kk]), w1 = pack2(w[kk + 1], w[kk + 1]);
                        const float sf0 = cf + (float)(s0 + kk), sf1 = cf + (float)(s0 + kk + 1);
                        const f32x2 slot0 = pack2(sf0, sf0), slot1 = pack2(sf1, sf1);
#pragma unroll
                        for (int e = 0; e < NP; e++) {
                            const f32x2 t0 = mul2(f[kk][e], w0);
                            const f32x2 t1 = mul2(f[kk + 1][e], w1);
                            sum[e] = add2(add2(sum[e], t0), t1);
                            float t0x, t0y, t1x, t1y;
                            unpack2(t0, t0x, t0y);
                            unpack2(t1, t1x, t1y);
                            // maximum over (running, slot, slot + 1); a slot takes the arg-max when its
                            // product equals that maximum, the later slot last: the same winner as
                            // testing `product >= running maximum` slot by slot
                            const float bx = max3(best[2 * e], t0x, t1x);
                            const float by = max3(best[2 * e + 1], t0y, t1y);
                            best[2 * e] = bx;
                            best[2 * e + 1] = by;
                            if (WITH_ARG) {
                                const f32x2 m0 = pack2(set_eq(t0x, bx), set_eq(t0y, by));
                                const f32x2 m1 = pack2(set_eq(t1x, bx), set_eq(t1y, by));
                                f32x2 a = argslot[e];
                                a = fma2(m0, sub2(slot0, a), a);  // a = m ? slot : a, exact for these small integers
                                a = fma2(m1, sub2(slot1, a), a);
                                argslot[e] = a;
                            }
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
                const float sf = (float)(c0 + kk);
#pragma unroll
                for (int u = 0; u < VPL; u++) {
                    const float4 fv = __ldg(feat + (size_t)j * F4 + col[u]);
                    const float fc[4] = {fv.x, fv.y, fv.z, fv.w};
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        float sx, sy, ax, ay;
                        unpack2(sum[2 * u + h], sx, sy);
                        unpack2(argslot[2 * u + h], ax, ay);
                        const float tx = __fmul_rn(fc[2 * h], w), ty = __fmul_rn(fc[2 * h + 1], w);
                        sx = __fadd_rn(sx, tx);
                        sy = __fadd_rn(sy, ty);
                        if (tx >= best[4 * u + 2 * h] || first) { best[4 * u + 2 * h] = tx; ax = sf; }
                        if (ty >= best[4 * u + 2 * h + 1] || first) { best[4 * u + 2 * h + 1] = ty; ay = sf; }
                        sum[2 * u + h] = pack2(sx, sy);
                        argslot[2 * u + h] = pack2(ax, ay);
                    }
                }
            }
        }

        if (live) {
#pragma unroll
            for (int u = 0; u < VPL; u++) {
                const int vec = gl + u * LPH;
                if (!EXACT && vec >= F4) continue;
                float sx, sy, sz, sw;
                unpack2(sum[2 * u], sx, sy);
                unpack2(sum[2 * u + 1], sz, sw);
                float4 m = make_float4(__fdiv_rn(sx, inv_count), __fdiv_rn(sy, inv_count),
                                       __fdiv_rn(sz, inv_count), __fdiv_rn(sw, inv_count));
                float4 mx = make_float4(best[4 * u], best[4 * u + 1], best[4 * u + 2], best[4 * u + 3]);
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
                    if (WITH_ARG) {
                        // slot -> neighbour id; no slot ever took the maximum: 0, the CPU op's initial value
                        float a0, a1, a2, a3;
                        unpack2(argslot[2 * u], a0, a1);
                        unpack2(argslot[2 * u + 1], a2, a3);
                        const int *ir = idxs + (size_t)v * ldk;
                        int4 a;
                        a.x = a0 < 0.f ? 0 : ir[(int)a0];
                        a.y = a1 < 0.f ? 0 : ir[(int)a1];
                        a.z = a2 < 0.f ? 0 : ir[(int)a2];
                        a.w = a3 < 0.f ? 0 : ir[(int)a3];
                        __stcs(reinterpret_cast<int4 *>(out_arg + (size_t)v * F4 * 4) + vec, a);
                    }
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

template <int LPH, int VPL, int CH, int THREADS, int MINB>
int launch_vec(bool exp_w, bool with_arg, const float *w, const float *feat, const int *idxs, float *out,
               int *out_arg, int n_vert, int K, int ldk, int F4, int n_out, bool mm, const int *order,
               float scale, bool sub_self, cudaStream_t stream)
{
    constexpr int G = THREADS / LPH;
    const long long n_tiles = div_up(div_up(n_vert, G), kAccTileSteps);
    // one block per tile up to 32 blocks per SM (blocks beyond that walk several tiles): measured faster on
    // the 64-event batch than a grid of resident blocks only, which keeps the SMs less evenly loaded
    long long blocks = (long long)sm_count() * 32;
    if (blocks > n_tiles) blocks = n_tiles;
    const float4 *f4 = reinterpret_cast<const float4 *>(feat);
#define HGC_GO(E, A, X)                                                                                    \
    accumulate_vec_kernel<LPH, VPL, CH, THREADS, MINB, E, A, X><<<(int)blocks, THREADS, 0, stream>>>(      \
            w, f4, idxs, out, out_arg, n_vert, K, ldk, F4, n_out, mm, order, scale, sub_self)
#define HGC_GO2(E, A) do { if (F4 == LPH * VPL) HGC_GO(E, A, true); else HGC_GO(E, A, false); } while (0)
    if (exp_w) { if (with_arg) HGC_GO2(true, true); else HGC_GO2(true, false); }
    else       { if (with_arg) HGC_GO2(false, true); else HGC_GO2(false, false); }
#undef HGC_GO2
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
        const long long cap = (long long)sm_count() * 32;
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
#define HGC_VEC(L, V, C, T, M) return launch_vec<L, V, C, T, M>(exp_w, with_arg, w, feat, idxs, out, out_arg, n_vert, K, ldk, F4, n_out, mm, order, scale, sub_self, stream)
    // lanes per hit x float4 per lane, rows in flight, block size, blocks per SM
    if (F4 <= 4) HGC_VEC(4, 1, 4, 1024, 1);  // measured at F = 16: 2.55 ms against 3.12 ms with 4 blocks of 256 (6.4 M hits)
    if (F4 <= 8) HGC_VEC(8, 1, 4, 256, 4);
    // F = 64: one block of 768 threads per SM works on 96 consecutive hits at a time (measured best on the
    // 64-event batch: the rows those hits share are found in L1)
    if (F4 <= 16) HGC_VEC(8, 2, 4, 768, 1);
    if (F4 <= 32) HGC_VEC(16, 2, 4, 768, 1);
    if (F4 <= 64) HGC_VEC(32, 2, 4, 768, 1);
    HGC_VEC(32, 4, 2, 512, 1);
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
