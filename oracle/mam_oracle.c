/* CPU oracle for the Multiply-And-Max/min path, plain C.  TEST INFRASTRUCTURE ONLY: nothing in
 * the product links or loads this; tests and the bench's CPU-baseline leg do.
 *
 * Restates the reference checker `test/reference.py:3-25` (SSIGPRO/mamtorch) as loops:
 *   forward : p = fl32(a[m,k]*b[k,n]) (one rounded multiply, no fused multiply-add);
 *             strict '>' / '<' while k ascends, so the lowest k wins ties and -0.0 == +0.0,
 *             exactly what torch.max/torch.min return on CPU; y = max + min + bias[n].
 *   backward: every output sends g*b[k,n] to agrad[m,k] and g*a[m,k] to bgrad[k,n] for
 *             k = argmax and k = argmin (twice when they coincide).
 * Build with -ffp-contract=off so the compiler cannot fuse the multiply into anything.
 * Pinned against stored outputs of the reference by tests/test_oracle.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* b_is_nk = 0: b is [K,N] row-major (operand of the torch op); 1: b is W[N,K] row-major. */
void mam_oracle_forward(const float* a, const float* b, int b_is_nk, const float* bias,
                        float* y, int64_t* argmax, int64_t* argmin,
                        int64_t M, int64_t K, int64_t N)
{
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float* vmax = (float*)malloc(sizeof(float) * (size_t)N * 2);
        float* vmin = vmax + N;
        int64_t* imax = argmax + m * N;
        int64_t* imin = argmin + m * N;
        for (int64_t n = 0; n < N; ++n) { vmax[n] = -INFINITY; vmin[n] = INFINITY; imax[n] = 0; imin[n] = 0; }
        for (int64_t k = 0; k < K; ++k) {
            const float x = a[m * K + k];
            for (int64_t n = 0; n < N; ++n) {
                const float w = b_is_nk ? b[n * K + k] : b[k * N + n];
                volatile float pv = x * w;          /* force the fp32 rounding */
                const float p = pv;
                if (p > vmax[n]) { vmax[n] = p; imax[n] = k; }
                if (p < vmin[n]) { vmin[n] = p; imin[n] = k; }
            }
        }
        for (int64_t n = 0; n < N; ++n) {
            float s = vmax[n] + vmin[n];
            if (bias) s = s + bias[n];
            y[m * N + n] = s;
        }
        free(vmax);
    }
}

/* agrad[M,K] and bgrad (same layout as b) are overwritten. Sequential in (m,n): deterministic. */
void mam_oracle_backward(const float* a, const float* b, int b_is_nk, const float* g,
                         const int64_t* argmax, const int64_t* argmin,
                         float* agrad, float* bgrad, int64_t M, int64_t K, int64_t N)
{
    memset(agrad, 0, sizeof(float) * (size_t)(M * K));
    memset(bgrad, 0, sizeof(float) * (size_t)(K * N));
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            const float gv = g[m * N + n];
            for (int side = 0; side < 2; ++side) {
                const int64_t k = side ? argmin[m * N + n] : argmax[m * N + n];
                const int64_t bi = b_is_nk ? n * K + k : k * N + n;
                agrad[m * K + k] += b[bi] * gv;
                bgrad[bi] += a[m * K + k] * gv;
            }
        }
}

int mam_oracle_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
