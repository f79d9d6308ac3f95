/* Uses the library from plain C: no Python, no torch, no TensorFlow -- only the CUDA runtime for device
 * memory.  One event of N hits in 3-D, wrapper-level kNN (hgc_binned_select_knn_ragged), then
 * hgc_accumulate_knn_exp on the result; both are checked on the host against a brute-force loop with the
 * same float32 operation order.  Exit code 0 = all rows agree.
 *
 *   gcc -std=c11 -O2 -Iinclude tests/c_abi/knn_from_c.c -o knn_from_c \
 *       -Lhgcalml_b200 -lhgcalml_b200 -L/usr/local/cuda/lib64 -lcudart -lm -Wl,-rpath,$PWD/hgcalml_b200
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <cuda_runtime_api.h>
#include "hgcalml_b200.h"

#define N 3000
#define C 3
#define K 12
#define F 8

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 2; } } while (0)
#define HK(x) do { int r_ = (x); if (r_ != HGC_OK) { fprintf(stderr, "%s: %s (%s)\n", #x, hgc_strerror(r_), hgc_last_cuda_error()); return 3; } } while (0)

static unsigned rng_state = 12345u;
static float uniform01(void) { rng_state = rng_state * 1664525u + 1013904223u; return (float)(rng_state >> 8) / 16777216.0f; }

static float distsq(const float *a, const float *b)
{
    float s = 0.f;
    for (int c = 0; c < C; c++) { const float d = a[c] - b[c]; s += d * d; }  /* compile without -ffast-math */
    return s;
}

int main(void)
{
    static float coords[N * C], feats[N * F], dist[N * K], out[N * 2 * F];
    static int idx[N * K], row_splits[2] = {0, N};
    for (int i = 0; i < N * C; i++) coords[i] = uniform01();
    for (int i = 0; i < N * F; i++) feats[i] = uniform01() - 0.5f;

    float *d_coords, *d_feats, *d_dist, *d_out;
    int *d_rs, *d_idx, *d_sorting;
    void *d_ws;
    const size_t ws_bytes = hgc_binned_select_knn_ragged_workspace_bytes(N, K, C, 2, 0, 3);
    CK(cudaMalloc((void **)&d_coords, sizeof coords));
    CK(cudaMalloc((void **)&d_feats, sizeof feats));
    CK(cudaMalloc((void **)&d_dist, sizeof dist));
    CK(cudaMalloc((void **)&d_out, sizeof out));
    CK(cudaMalloc((void **)&d_rs, sizeof row_splits));
    CK(cudaMalloc((void **)&d_idx, sizeof idx));
    CK(cudaMalloc((void **)&d_sorting, sizeof(int) * N));
    CK(cudaMalloc(&d_ws, ws_bytes));
    CK(cudaMemcpy(d_coords, coords, sizeof coords, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_feats, feats, sizeof feats, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_rs, row_splits, sizeof row_splits, cudaMemcpyHostToDevice));

    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    HK(hgc_binned_select_knn_ragged(d_coords, d_rs, NULL, d_idx, d_dist, d_sorting, N, K, C, 2, 0, 3, 0, 0,
                                    d_ws, ws_bytes, stream));
    unsigned status = 0;
    HK(hgc_workspace_status(d_ws, stream, &status));
    HK(hgc_accumulate_knn_exp(d_dist, d_feats, d_idx, d_out, NULL, N, K, F, 2 * F, 1, 10.f, d_sorting, stream));
    CK(cudaStreamSynchronize(stream));
    CK(cudaMemcpy(idx, d_idx, sizeof idx, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dist, d_dist, sizeof dist, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(out, d_out, sizeof out, cudaMemcpyDeviceToHost));

    int bad = 0;
    for (int i = 0; i < N && bad < 5; i++) {
        /* brute force: the K-1 smallest distances to other hits, ascending (distance, index) */
        if (idx[i * K] != i || dist[i * K] != 0.f) { printf("row %d: slot 0 is not the hit itself\n", i); bad++; continue; }
        float prev_d = -1.f; int prev_j = -1;
        for (int k = 1; k < K; k++) {
            float best = INFINITY; int best_j = -1;
            for (int j = 0; j < N; j++) {
                if (j == i) continue;
                const float d = distsq(coords + i * C, coords + j * C);
                if ((d > prev_d || (d == prev_d && j > prev_j)) && (d < best || (d == best && j < best_j))) { best = d; best_j = j; }
            }
            if (idx[i * K + k] != best_j || dist[i * K + k] != best) {
                printf("row %d slot %d: got (%d, %g), brute force (%d, %g)\n", i, k, idx[i * K + k], dist[i * K + k], best_j, best);
                bad++;
                break;
            }
            prev_d = best; prev_j = best_j;
        }
        /* accumulated mean and max of exp(-10 d) * feature, 1e-5 relative to the summed terms */
        for (int f = 0; f < F; f++) {
            float sum = 0.f, mx = 0.f, scale = 0.f;
            for (int k = 0; k < K; k++) {
                const float t = expf(-(10.f * dist[i * K + k])) * feats[idx[i * K + k] * F + f];
                sum += t; scale += fabsf(t);
                if (k == 0 || t >= mx) mx = t;
            }
            const float mean = sum / (float)K;
            if (fabsf(out[i * 2 * F + f] - mean) > 1e-5f * (scale / K + fabsf(mean)) + 1e-12f ||
                fabsf(out[i * 2 * F + F + f] - mx) > 1e-5f * fabsf(mx) + 1e-12f) {
                printf("row %d feature %d: got (%g, %g), host (%g, %g)\n", i, f, out[i * 2 * F + f], out[i * 2 * F + F + f], mean, mx);
                bad++;
                break;
            }
        }
    }
    printf("%s: %d hits, K=%d, library version %d, %llu kernel launches\n", bad ? "MISMATCH" : "ok", N, K, hgc_version(),
           hgc_launch_count());
    return bad ? 1 : 0;
}
