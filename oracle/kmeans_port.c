/* Test infrastructure, not product code.
 *
 * CPU restatement (plain C, FP32, no FMA contraction: build with -ffp-contract=off) of the two
 * host-side loops of the reference's Centroid Accumulator.  Only tests/, the smoke check and
 * bench.py's cpu_baseline / reference arm may load this library; the product path never does.
 *
 * Pinned against the reference itself: tests/test_oracle_golden.py runs oracle/_ref/centroid-merge
 * (the unmodified reference CLI) on the same snapshot files and requires byte-identical output.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Lloyd k-means over N vectors of dimension D.
 * Follows src/centroid/centroid_accumulator.cpp:114-157:
 *   - k = min(k, N)                                   (:115)
 *   - centres start as vectors[(i*N)/k]               (:121-123)
 *   - at most 50 iterations; assignments start at 0   (:125-126)
 *   - distance is a sequential `d += v*v` over i      (:132-136)
 *   - strict `<` so the lowest index wins ties        (:137)
 *   - stop before the update when nothing changed     (:141)
 *   - update = sequential sum in n order, then `v /= count`; empty clusters stay all-zero (:144-156)
 * Returns the number of assignment passes executed. `centers` is [k*D], `assign` is [N]. */
static int lloyd(const float* vectors, int N, int D, int k, int max_iters, float* centers, int* assign);

int ta_oracle_kmeans(const float* vectors, int N, int D, int k, int max_iters,
                     float* centers, int* assign, int* k_out)
{
    if (k > N) k = N;
    *k_out = k;
    for (int i = 0; i < k; i++)
        memcpy(centers + (size_t)i * D, vectors + (size_t)(((long)i * N) / k) * D, sizeof(float) * D);
    return lloyd(vectors, N, D, k, max_iters, centers, assign);
}

/* The same Lloyd passes from caller-chosen starting centres vectors[init_idx[i]] (the seeded
 * k-means++ extension; no reference counterpart). */
int ta_oracle_kmeans_from(const float* vectors, int N, int D, int k, int max_iters, const int* init_idx,
                          float* centers, int* assign)
{
    for (int i = 0; i < k; i++)
        memcpy(centers + (size_t)i * D, vectors + (size_t)init_idx[i] * D, sizeof(float) * D);
    return lloyd(vectors, N, D, k, max_iters, centers, assign);
}

static int lloyd(const float* vectors, int N, int D, int k, int max_iters, float* centers, int* assign)
{
    for (int n = 0; n < N; n++) assign[n] = 0;
    int* counts = (int*)malloc(sizeof(int) * (k > 0 ? k : 1));
    int iters = 0;
    for (int iter = 0; iter < max_iters; iter++) {
        iters++;
        int changed = 0;
        for (int n = 0; n < N; n++) {
            float best_d = 1e38f;
            int best_k = 0;
            const float* x = vectors + (size_t)n * D;
            for (int ki = 0; ki < k; ki++) {
                const float* c = centers + (size_t)ki * D;
                float d = 0.f;
                for (int i = 0; i < D; i++) {
                    float v = x[i] - c[i];
                    d += v * v;
                }
                if (d < best_d) { best_d = d; best_k = ki; }
            }
            if (assign[n] != best_k) { assign[n] = best_k; changed = 1; }
        }
        if (!changed) break;
        for (int ki = 0; ki < k; ki++) counts[ki] = 0;
        memset(centers, 0, sizeof(float) * (size_t)k * D);
        for (int n = 0; n < N; n++) {
            int ki = assign[n];
            float* c = centers + (size_t)ki * D;
            const float* x = vectors + (size_t)n * D;
            for (int i = 0; i < D; i++) c[i] += x[i];
            counts[ki]++;
        }
        for (int ki = 0; ki < k; ki++)
            if (counts[ki] > 0) {
                float* c = centers + (size_t)ki * D;
                /* `v /= counts[ki]`: float divided by int, i.e. by (float)count */
                for (int i = 0; i < D; i++) c[i] /= (float)counts[ki];
            }
    }
    free(counts);
    return iters;
}

/* Intended accumulation, src/centroid/centroid_accumulator.cpp:54-69 fed the [BT,D] data its
 * header documents: gnorm_t = sqrt(sum_d g[t,d]^2) (sequential FP32), acc[d] += h[t,d]*gnorm_t,
 * weight += gnorm_t.  h and g are FP32 arrays holding BF16-representable values. */
void ta_oracle_centroid_intended(const float* h, const float* g, int BT, int D,
                                 float* acc, float* weight)
{
    float w = *weight;
    for (int t = 0; t < BT; t++) {
        float gn = 0.f;
        for (int d = 0; d < D; d++) { float v = g[(size_t)t * D + d]; gn += v * v; }
        gn = sqrtf(gn);
        for (int d = 0; d < D; d++) acc[d] += h[(size_t)t * D + d] * gn;
        w += gn;
    }
    *weight = w;
}

/* What the shipped trainer actually computes: src/trainer/adapt_trainer.cu:215-231 up-casts both
 * tensors to F32 and CentroidAccumulator::accumulate (:45-48) then re-reads those F32 buffers
 * through a BF16 pointer.  Each F32 that came from a BF16 has zero low 16 bits, so the BF16
 * stream seen is 0, x0, 0, x1, ... and only the first BT*D/2 floats are consumed.  This applies
 * the same loop (:54-69) to that reinterpreted stream. */
void ta_oracle_centroid_asbuilt(const float* h, const float* g, int BT, int D,
                                float* acc, float* weight)
{
    float w = *weight;
    for (int u = 0; u < BT; u++) {
        float gn = 0.f;
        for (int d = 0; d < D; d++) {
            /* element (u, d) of the reinterpreted stream: flat bf16 index j = u*D + d */
            size_t j = (size_t)u * D + d;
            float v = (j & 1) ? g[j >> 1] : 0.f;
            gn += v * v;
        }
        gn = sqrtf(gn);
        for (int d = 0; d < D; d++) {
            size_t j = (size_t)u * D + d;
            float v = (j & 1) ? h[j >> 1] : 0.f;
            acc[d] += v * gn;
        }
        w += gn;
    }
    *weight = w;
}
