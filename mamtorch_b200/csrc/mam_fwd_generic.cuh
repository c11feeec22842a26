// Any-shape exact MAM forward: the fallback for operands the TMA path cannot describe
// (K not a multiple of 4, pointers not 16-byte aligned, tiny problems) and an independent
// on-device cross-check of the fast path.
//
// Replaces fullyconnected_cuda_kernel of the reference
// (mamtorch/kernel/v1/csrc/cuda/fullyconnected.cu:33-175): same contract -- exact fp32 max+min with
// the lowest k winning ties through strict compares in ascending k -- but it reads a[M,K] and
// b[K,N] (or W[N,K]) in place (no transposed / padded copies), initialises the running extremes
// with -inf/+inf, and handles ragged edges by clamping the load coordinates: a replicated element
// can tie but never beat the original, so it never changes a value or an index.
#pragma once
#include "mam_ptx.cuh"

namespace mamb200 {

struct EpilogueArgs {
    const float* bias;   // [N] or nullptr
    const float* dense;  // [M,N] precomputed a.b or nullptr
    float alpha;         // scale of (max+min); used only when blend != 0
    float beta;          // scale of dense
    int blend;           // 0: y = (max+min) [+ bias]
    // output dropout, applied last: element i = m*N+n is kept (and scaled) where mam_drop_keeps(seed, i, threshold)
    unsigned long long drop_seed;
    unsigned drop_threshold;   // rate * 2^32
    float drop_scale;          // 1 / (1 - rate); 0 = no dropout
};

// The keep / drop decision of element `idx` under `seed`: a counter-based generator (the splitmix64 mixing
// function on seed + idx * golden ratio), so that the same mask is formed again wherever it is needed --
// forward epilogue, backward, weight drop -- without ever being stored.  Dropped with probability
// threshold / 2^32.
__device__ __forceinline__ bool mam_drop_keeps(unsigned long long seed, unsigned long long idx, unsigned threshold) {
    unsigned long long z = seed + idx * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (unsigned)(z >> 32) >= threshold;
}

// out[i] = in[i] * scale where element i is kept, else 0 (in == out is fine)
__global__ void __launch_bounds__(256)
mam_drop_kernel(const float* __restrict__ in, float* __restrict__ out, long long n, unsigned long long seed,
                unsigned threshold, float scale) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) out[i] = mam_drop_keeps(seed, (unsigned long long)i, threshold) ? __fmul_rn(in[i], scale) : 0.f;
}

// y = alpha*(vmax+vmin) + beta*dense + bias, every step individually rounded (no contraction),
// in the order of the reference's host glue (mamtorch/kernel/v3/csrc/cuda/fullyconnected.cu:153-160).
__device__ __forceinline__ float mam_epilogue_term(float s, const EpilogueArgs& e, long long m, long long n,
                                                   long long N) {
    if (e.blend) {
        s = __fmul_rn(s, e.alpha);
        if (e.dense) s = __fadd_rn(s, __fmul_rn(e.dense[m * N + n], e.beta));
    }
    if (e.bias) s = __fadd_rn(s, e.bias[n]);
    if (e.drop_scale != 0.f)
        s = mam_drop_keeps(e.drop_seed, (unsigned long long)(m * N + n), e.drop_threshold) ? __fmul_rn(s, e.drop_scale)
                                                                                           : 0.f;
    return s;
}
__device__ __forceinline__ float mam_epilogue(float vmax, float vmin, const EpilogueArgs& e,
                                              long long m, long long n, long long N) {
    return mam_epilogue_term(__fadd_rn(vmax, vmin), e, m, n, N);
}

constexpr int GEN_TILE = 64;
constexpr int GEN_BK = 16;

template <bool B_NK>
__global__ void __launch_bounds__(256)
mam_fwd_generic_kernel(const float* __restrict__ a, const float* __restrict__ b,
                       float* __restrict__ y, int* __restrict__ argmax, int* __restrict__ argmin,
                       long long M, long long K, long long N, EpilogueArgs ep) {
    __shared__ float As[GEN_BK][GEN_TILE + 1];
    __shared__ float Bs[GEN_BK][GEN_TILE + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = (long long)blockIdx.y * GEN_TILE, n0 = (long long)blockIdx.x * GEN_TILE;

    float vmax[4][4], vmin[4][4];
    int imax[4][4], imin[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            vmax[i][j] = -INFINITY;
            vmin[i][j] = INFINITY;
            imax[i][j] = 0;
            imin[i][j] = 0;
        }

    for (long long k0 = 0; k0 < K; k0 += GEN_BK) {
        // A tile: 64 rows x 16 k, k fastest in memory
        {
            const int kk = threadIdx.x & 15, r = threadIdx.x >> 4;
            const long long kc = min(k0 + kk, K - 1);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const long long mc = min(m0 + r + 16 * p, M - 1);
                As[kk][r + 16 * p] = a[mc * K + kc];
            }
        }
        if (B_NK) {
            const int kk = threadIdx.x & 15, r = threadIdx.x >> 4;
            const long long kc = min(k0 + kk, K - 1);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const long long nc = min(n0 + r + 16 * p, N - 1);
                Bs[kk][r + 16 * p] = b[nc * K + kc];
            }
        } else {
            const int nn = threadIdx.x & 63, r = threadIdx.x >> 6;
            const long long nc = min(n0 + nn, N - 1);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const long long kc = min(k0 + r + 4 * p, K - 1);
                Bs[r + 4 * p][nn] = b[kc * N + nc];
            }
        }
        __syncthreads();
        const int kend = (int)min((long long)GEN_BK, K - k0);
        for (int kk = 0; kk < kend; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx + 16 * j];
            const int k = (int)(k0 + kk);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p = __fmul_rn(av[i], bv[j]);
                    if (p > vmax[i][j]) { vmax[i][j] = p; imax[i][j] = k; }
                    if (p < vmin[i][j]) { vmin[i][j] = p; imin[i][j] = k; }
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long n = n0 + tx + 16 * j;
            if (n >= N) continue;
            y[m * N + n] = mam_epilogue(vmax[i][j], vmin[i][j], ep, m, n, N);
            if (argmax) argmax[m * N + n] = imax[i][j];
            if (argmin) argmin[m * N + n] = imin[i][j];
        }
    }
}

// out[c][r] = in[r][c]; in is [R,C] row-major.  Used to turn the op-level b[K,N] into the
// K-contiguous W[N,K] the tiled kernels want, and back for gradients.
__global__ void __launch_bounds__(256)
mam_transpose_kernel(const float* __restrict__ in, float* __restrict__ out, long long R, long long C) {
    __shared__ float t[32][33];
    const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long r = r0 + ty + 8 * p, c = c0 + tx;
        if (r < R && c < C) t[ty + 8 * p][tx] = in[r * C + c];
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long c = c0 + ty + 8 * p, r = r0 + tx;
        if (r < R && c < C) out[c * R + r] = t[tx][ty + 8 * p];
    }
}

// out[b][c][r] = in[b][r][c] for `batch` matrices [R,C] stored back to back (blockIdx.z = b).  With R = channels
// and C = H*W this turns an image batch [B,C,H,W] into the channels-last [B,H,W,C] the im2col-mode loads read.
__global__ void __launch_bounds__(256)
mam_transpose_batched_kernel(const float* __restrict__ in, float* __restrict__ out, long long R, long long C) {
    __shared__ float t[32][33];
    const long long base = (long long)blockIdx.z * R * C;
    const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long r = r0 + ty + 8 * p, c = c0 + tx;
        if (r < R && c < C) t[ty + 8 * p][tx] = in[base + r * C + c];
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const long long c = c0 + ty + 8 * p, r = r0 + tx;
        if (r < R && c < C) out[base + c * R + r] = t[tx][ty + 8 * p];
    }
}

}  // namespace mamb200
