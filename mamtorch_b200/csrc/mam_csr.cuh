// Pruned-weight kernels on CSR rows of W[N,K].
//
//  * mam_csr_fwd_kernel: MAM forward that touches only the stored weights.  The reference has no
//    sparse MAM: its pruning examples zero dense weights in place and run the dense kernels
//    (examples/vitb16_imagenet1k/pruning_utils.py:105-116), so the contract is "same result as the
//    dense layer on W with zeros at the pruned positions".  A pruned position still contributes a
//    product of +-0 at its k, therefore every row with fewer than K stored entries gets one
//    implicit candidate: value 0 at k0 = the lowest column that is not stored.  It beats a negative
//    explicit maximum, and on an exact tie with an explicit zero product the lower k wins.
//  * mam_spmm_csr_kernel: C = A_csr . B in the ordinary sum semiring, the operation behind
//    torch.ops.mamtorch_kernel_sparsev1.cusparsemm (mamtorch/sparse/kernel/v1/csrc/cuda/cusparsemm_csr.cu:19-77,
//    there a cuSPARSE call with a leaked per-call workspace).
//
// Forward layout: a CTA parks R rows of a in shared memory and its 8 warps stream the whole CSR
// once; a warp owns 32 consecutive outputs n at a time, its lanes stride over the stored entries
// of row n (coalesced), gather a[r][col] from shared memory and keep per-lane extremes with strict
// compares (ascending col per lane, so the lowest k survives).  Warp-wide, the value is reduced
// with redux.sync.max/min.f32 (sm_100a) and the index with a redux.sync.min.u32 over the lanes that
// hold the extreme.  Results are staged in shared memory and written 32 outputs at a time.
#pragma once
#include "mam_ptx.cuh"

namespace mamb200 {

__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float warp_min_f32(float v) {
    float r;
    asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ unsigned warp_min_u32(unsigned v) {
    unsigned r;
    asm volatile("redux.sync.min.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}

constexpr int CSR_WARPS = 16;
constexpr int CSR_UNROLL = 4;   // stored entries in flight per lane

template <int R>
__global__ void __launch_bounds__(CSR_WARPS * 32)
mam_csr_fwd_kernel(const float* __restrict__ a, const long long* __restrict__ crow,
                   const long long* __restrict__ col, const float* __restrict__ val,
                   const float* __restrict__ bias, float* __restrict__ y, int* __restrict__ argmax,
                   int* __restrict__ argmin, long long M, long long K, long long N) {
    extern __shared__ float csr_smem[];
    float* a_s = csr_smem;                                  // [R][K]
    float* o_s = csr_smem + (size_t)R * K;                  // [warps][3][R][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long m0 = (long long)blockIdx.x * R;
    for (long long i = tid; i < (long long)R * K; i += CSR_WARPS * 32) {
        const long long r = i / K, k = i - r * K;
        a_s[i] = (m0 + r < M) ? a[(m0 + r) * K + k] : 0.f;
    }
    __syncthreads();
    float* oy = o_s + (size_t)warp * 3 * R * 32;
    int* omax = reinterpret_cast<int*>(oy + R * 32);
    int* omin = omax + R * 32;
    const unsigned NONE = 0x7fffffffu;

    const long long nblocks = (N + 31) / 32;
    for (long long blk = warp; blk < nblocks; blk += CSR_WARPS) {
        const long long nbase = blk * 32;
        const int ncols = (int)min(32LL, N - nbase);
        // row extents of the whole 32-row block in one coalesced load; broadcast per row below
        const long long my_s = crow[min(nbase + lane, N)], my_e = crow[min(nbase + lane + 1, N)];
        for (int j = 0; j < ncols; ++j) {
            const long long n = nbase + j;
            const long long s = __shfl_sync(0xffffffffu, my_s, j), e = __shfl_sync(0xffffffffu, my_e, j);
            const int nnz = (int)(e - s);
            float vmax[R], vmin[R];
            unsigned kmax[R], kmin[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                vmax[r] = -INFINITY;
                vmin[r] = INFINITY;
                kmax[r] = NONE;
                kmin[r] = NONE;
            }
            unsigned gap = NONE;  // first position t whose stored column is not t: column t is missing
            for (int t0 = lane; t0 < nnz; t0 += 32 * CSR_UNROLL) {
                // issue all loads of this batch before touching any of them
                unsigned c[CSR_UNROLL];
                float v[CSR_UNROLL];
#pragma unroll
                for (int u = 0; u < CSR_UNROLL; ++u) {
                    const int t = t0 + 32 * u;
                    const bool in = t < nnz;
                    c[u] = in ? (unsigned)col[s + t] : 0u;
                    v[u] = in ? val[s + t] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < CSR_UNROLL; ++u) {
                    const int t = t0 + 32 * u;
                    if (t < nnz) {
                        if (c[u] != (unsigned)t) gap = min(gap, (unsigned)t);
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const float p = __fmul_rn(a_s[(size_t)r * K + c[u]], v[u]);
                            if (p > vmax[r]) { vmax[r] = p; kmax[r] = c[u]; }
                            if (p < vmin[r]) { vmin[r] = p; kmin[r] = c[u]; }
                        }
                    }
                }
            }
            gap = warp_min_u32(gap);
            const bool implicit = nnz < K;                  // at least one pruned position
            const unsigned k0 = gap == NONE ? (unsigned)nnz : gap;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float gmax = warp_max_f32(vmax[r]);
                unsigned imax = warp_min_u32(vmax[r] == gmax ? kmax[r] : NONE);
                float gmin = warp_min_f32(vmin[r]);
                unsigned imin = warp_min_u32(vmin[r] == gmin ? kmin[r] : NONE);
                if (implicit) {
                    if (0.f > gmax) { gmax = 0.f; imax = k0; } else if (0.f == gmax) imax = min(imax, k0);
                    if (0.f < gmin) { gmin = 0.f; imin = k0; } else if (0.f == gmin) imin = min(imin, k0);
                }
                if (lane == 0) {
                    float out = __fadd_rn(gmax, gmin);
                    if (bias) out = __fadd_rn(out, bias[n]);
                    oy[r * 32 + j] = out;
                    omax[r * 32 + j] = (int)min(imax, (unsigned)(K - 1));
                    omin[r * 32 + j] = (int)min(imin, (unsigned)(K - 1));
                }
            }
        }
        __syncwarp();
        if (lane < ncols) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (m0 + r < M) {
                    const long long o = (m0 + r) * N + nbase + lane;
                    y[o] = oy[r * 32 + lane];
                    if (argmax) argmax[o] = omax[r * 32 + lane];
                    if (argmin) argmin[o] = omin[r * 32 + lane];
                }
            }
        }
        __syncwarp();
    }
}

// C[n, j] = sum over stored (n,k) of val * B[k, j];  B is [K, Mc] row-major, C is [N, Mc].
__global__ void __launch_bounds__(128)
mam_spmm_csr_kernel(const long long* __restrict__ crow, const long long* __restrict__ col,
                    const float* __restrict__ val, const float* __restrict__ b, float* __restrict__ c,
                    long long N, long long Mc) {
    const long long n = blockIdx.y;
    const long long j = (long long)blockIdx.x * 128 + threadIdx.x;
    if (n >= N || j >= Mc) return;
    const long long s = crow[n], e = crow[n + 1];
    float acc = 0.f;
    for (long long t = s; t < e; ++t) acc = fmaf(val[t], b[col[t] * Mc + j], acc);
    c[n * Mc + j] = acc;
}

// The same product, four columns per thread (B and C rows 16-byte aligned, Mc % 4 == 0) and four stored entries
// in flight: every row of B a stored entry names is fetched with 16-byte loads, 2 KB per CTA and entry, and the
// four fetches are issued before the first is used.  The additions stay in ascending column order, so the sums
// are the ones of the kernel above bit for bit.  This is the form for very sparse operands, where the product
// is bound by the L2 traffic of the gathered B rows (nnz * Mc * 4 bytes) and nothing is there to reuse.
__global__ void __launch_bounds__(128)
mam_spmm_csr_v4_kernel(const long long* __restrict__ crow, const long long* __restrict__ col,
                       const float* __restrict__ val, const float* __restrict__ b, float* __restrict__ c,
                       long long N, long long Mc) {
    const long long n = blockIdx.y;
    const long long j = ((long long)blockIdx.x * 128 + threadIdx.x) * 4;
    if (n >= N || j >= Mc) return;
    const long long s = crow[n], e = crow[n + 1];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    long long t = s;
    for (; t + 4 <= e; t += 4) {
        float v[4];
        float4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            v[u] = val[t + u];
            x[u] = *reinterpret_cast<const float4*>(b + col[t + u] * Mc + j);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc.x = fmaf(v[u], x[u].x, acc.x);
            acc.y = fmaf(v[u], x[u].y, acc.y);
            acc.z = fmaf(v[u], x[u].z, acc.z);
            acc.w = fmaf(v[u], x[u].w, acc.w);
        }
    }
    for (; t < e; ++t) {
        const float v = val[t];
        const float4 x = *reinterpret_cast<const float4*>(b + col[t] * Mc + j);
        acc.x = fmaf(v, x.x, acc.x);
        acc.y = fmaf(v, x.y, acc.y);
        acc.z = fmaf(v, x.z, acc.z);
        acc.w = fmaf(v, x.w, acc.w);
    }
    *reinterpret_cast<float4*>(c + n * Mc + j) = acc;
}

}  // namespace mamb200
