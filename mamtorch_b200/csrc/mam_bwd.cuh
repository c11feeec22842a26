// Selected-pair backward of the MAM layer and the per-weight selection count.
//
// Replaces fullyconnected_backward_cuda_kernel of the reference
// (mamtorch/kernel/v4/csrc/cuda/fullyconnected_backward.cu:23-78; identical in v1), which runs one
// thread per 16x16 patch of outputs and issues four dependent global atomics per output.
// Here a CTA owns a block of rows of a: it sweeps all N outputs of those rows with coalesced reads
// of grad / argmax / argmin, accumulates the rows' da in shared memory (written out once, no
// global atomics, no zero-fill pass) and sends the dW contributions to L2 with red.global.add.f32.
// Sums are formed in a different order than the reference's, so gradients agree to rounding
// (1e-5 relative in the tests), not bit for bit.
#pragma once
#include "mam_conv.cuh"
#include "mam_ptx.cuh"

namespace mamb200 {

constexpr int BWD_THREADS = 256;

// One dW term on its way to L2.  Plain form: an fp32 reduction into dw[wi].  FUSED form: `dw` is a scratch array
// of 16-byte records {dW sum, max hits, min hits, unused} in the weight operand's layout, and the term travels
// with the selection hit it stands for in ONE 16-byte vector reduction -- the same number of L2 operations as
// the plain form, and no second sweep over the index matrices for the counts.  The counts are sums of 1.0f,
// exact below 2^24 hits per weight and call; mam_bwd_unpack_kernel splits the records afterwards.
template <bool FUSED, bool IS_MAX>
__device__ __forceinline__ void dw_term(float* dw, long long wi, float term) {
    if constexpr (FUSED) {
        asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dw + wi * 4), "f"(term),
                     "f"(IS_MAX ? 1.f : 0.f), "f"(IS_MAX ? 0.f : 1.f), "f"(0.f)
                     : "memory");
    } else {
        atomicAdd(&dw[wi], term);
    }
}

// acc[i] = {dW sum, max hits, min hits, -} for element i of the weight operand's layout -> dw[i] and, added into
// the caller's [N,K] matrices, the hits.
template <bool B_NK>
__global__ void __launch_bounds__(256)
mam_bwd_unpack_kernel(const float4* __restrict__ acc, float* __restrict__ dw, int* __restrict__ hit_max,
                      int* __restrict__ hit_min, long long K, long long N) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= K * N) return;
    const float4 v = acc[i];
    dw[i] = v.x;
    const long long j = B_NK ? i : (i % N) * K + i / N;
    if (v.y != 0.f) hit_max[j] += (int)v.y;
    if (v.z != 0.f) hit_min[j] += (int)v.z;
}

// B_NK: w is W[N,K] and dw has the same layout; otherwise b[K,N].
// DA_KM: da is written transposed, da[k*M + m] (what the convolution's fold kernel wants: unit stride
// along the output pixels); a CTA's rows are consecutive, so every k still gets one whole sector.
// CONV: a is not a matrix of patch rows but the convolution input x[B,C,H,W] itself; row m is output
// pixel (b, ho, wo) and a[m][k] is read where the patch element k = (c*kH+kh)*kW+kw lives in x (zero
// in the padding), so the patch rows need not be kept for the backward.
template <bool B_NK, bool DA_KM = false, bool CONV = false, bool FUSED = false, bool SLICED = false>
__global__ void __launch_bounds__(BWD_THREADS)
mam_bwd_kernel(const float* __restrict__ a, const float* __restrict__ w, const float* __restrict__ g,
               const int* __restrict__ argmax, const int* __restrict__ argmin,
               float* __restrict__ da, float* __restrict__ dw,
               long long M, long long K, long long N, int rows_per_cta, float scale, ConvGeom cg, int slices) {
    // SLICED: argmax / argmin hold one [M,N] matrix per slice of K (the module's `splits`), `slices` of them;
    // every slice routes the same upstream gradient through its own selected pairs.  (A template parameter, so
    // that the ordinary kernel keeps the loop nest the compiler schedules best.)
    extern __shared__ float da_s[];  // [rows_per_cta][K]
    const long long m0 = (long long)blockIdx.x * rows_per_cta;
    const int rows = (int)min((long long)rows_per_cta, M - m0);
    for (long long i = threadIdx.x; i < (long long)rows * K; i += BWD_THREADS) da_s[i] = 0.f;
    __syncthreads();
    for (int r = 0; r < rows; ++r) {
        const long long m = m0 + r;
        const float* arow = a + m * K;
        // CONV: where this output pixel's patch starts in the input
        const float* xb = a;
        int h0 = 0, w0 = 0;
        if constexpr (CONV) {
            const int wo = (int)(m % cg.Wo);
            const long long t = m / cg.Wo;
            const int ho = (int)(t % cg.Ho);
            xb = a + (t / cg.Ho) * (long long)cg.C * cg.H * cg.W;
            h0 = ho * cg.sh - cg.ph;
            w0 = wo * cg.sw - cg.pw;
        }
        auto a_at = [&](int k) -> float {
            if constexpr (CONV) {
                const int taps = cg.kH * cg.kW;
                const int c = k / taps, rr = k - c * taps;
                const int kh = rr / cg.kW, kw = rr - kh * cg.kW;
                const int h = h0 + kh, ww = w0 + kw;
                if ((unsigned)h >= (unsigned)cg.H || (unsigned)ww >= (unsigned)cg.W) return 0.f;
                return xb[((long long)c * cg.H + h) * cg.W + ww];
            } else {
                return arow[k];
            }
        };
        float* dar = da_s + (long long)r * K;
        for (int sl = 0; sl < (SLICED ? slices : 1); ++sl) {
        const int* amax_row = argmax + (SLICED ? (long long)sl * M * N : 0) + m * N;
        const int* amin_row = argmin + (SLICED ? (long long)sl * M * N : 0) + m * N;
        for (long long n = threadIdx.x; n < N; n += BWD_THREADS) {
            const float gv = __fmul_rn(g[m * N + n], scale);
            int k1 = amax_row[n], k2 = amin_row[n];
            // an index outside [0,K) cannot come from the forward; skip it rather than fault
            const bool ok1 = (unsigned)k1 < (unsigned long long)K, ok2 = (unsigned)k2 < (unsigned long long)K;
            if (ok1) {
                const long long wi = B_NK ? n * K + k1 : (long long)k1 * N + n;
                atomicAdd(&dar[k1], __fmul_rn(w[wi], gv));
                dw_term<FUSED, true>(dw, wi, __fmul_rn(a_at(k1), gv));
            }
            if (ok2) {
                const long long wi = B_NK ? n * K + k2 : (long long)k2 * N + n;
                atomicAdd(&dar[k2], __fmul_rn(w[wi], gv));
                dw_term<FUSED, false>(dw, wi, __fmul_rn(a_at(k2), gv));
            }
        }
        }
    }
    __syncthreads();
    if constexpr (DA_KM) {
        for (long long i = threadIdx.x; i < (long long)rows * K; i += BWD_THREADS) {
            const long long k = i / rows;
            const int r = (int)(i - k * rows);
            da[k * M + m0 + r] = da_s[(long long)r * K + k];
        }
    } else {
        for (long long i = threadIdx.x; i < (long long)rows * K; i += BWD_THREADS) da[m0 * K + i] = da_s[i];
    }
}

// ---------------------------------------------------------------------------------------------
// Row-per-warp form of the same pass.
//
// In the form above all warps of a CTA add into the same rows of da, so every addition is a
// floating-point shared-memory atomic -- a compare-and-swap loop on this hardware, and more than half
// of the kernel's load/store wavefronts.  Here every warp owns ONE row of a: its da row lives in
// shared memory and only that warp touches it, so the additions are plain read-modify-writes.  What is
// left to settle is two lanes of the same instruction naming the same k (about half of the 32-lane
// groups hold one such pair at K = 768): match.any groups the lanes by k, the lowest lane of a group
// collects the other lanes' terms by shuffle and adds the sum once.  A_SMEM also parks the warp's row
// of a in shared memory, so that the two selected activations per output are shared-memory gathers
// instead of scattered reads of a 3 KB row through L1.  The dW terms still go to L2 as
// red.global.add.f32 (their addresses are distinct inside a warp by construction: 32 different n).
constexpr int BWD_RW_UNROLL = 4;   // outputs in flight per lane

__device__ __forceinline__ void warp_row_add(float* row, int k, bool ok, float v, int lane) {
    // lanes with nothing to add get keys of their own so that they join no group
    const unsigned key = ok ? (unsigned)k : (0x80000000u | (unsigned)lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const bool leader = (__ffs(peers) - 1) == lane;
    unsigned todo = leader ? (peers & (peers - 1)) : 0u;   // the group's other lanes
    float s = v;
    while (__any_sync(0xffffffffu, todo != 0u)) {
        const int src = todo ? __ffs(todo) - 1 : lane;
        const float t = __shfl_sync(0xffffffffu, v, src);
        if (todo) {
            s += t;
            todo &= todo - 1;
        }
    }
    if (ok && leader) row[k] += s;
    __syncwarp();
}

template <bool B_NK, bool A_SMEM, bool FUSED = false, bool SLICED = false>
__global__ void __launch_bounds__(BWD_THREADS)
mam_bwd_rowwarp_kernel(const float* __restrict__ a, const float* __restrict__ w, const float* __restrict__ g,
                       const int* __restrict__ argmax, const int* __restrict__ argmin,
                       float* __restrict__ da, float* __restrict__ dw,
                       long long M, long long K, long long N, float scale, int slices) {
    extern __shared__ float rw_s[];   // per warp: da row [K] (+ a row [K])
    constexpr int WARPS = BWD_THREADS / 32, U = BWD_RW_UNROLL;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long m = (long long)blockIdx.x * WARPS + warp;
    if (m >= M) return;   // a whole warp leaves; nothing below synchronises across warps
    float* dar = rw_s + (size_t)warp * (size_t)K * (A_SMEM ? 2 : 1);
    float* as = dar + K;
    const float* arow = a + m * K;
    for (long long k = lane; k < K; k += 32) {
        dar[k] = 0.f;
        if constexpr (A_SMEM) as[k] = arow[k];
    }
    __syncwarp();
    const float* grow = g + m * N;
    for (int sl = 0; sl < (SLICED ? slices : 1); ++sl) {   // SLICED: one [M,N] pair of index matrices per slice of K
    const int* r1 = argmax + (SLICED ? (long long)sl * M * N : 0) + m * N;
    const int* r2 = argmin + (SLICED ? (long long)sl * M * N : 0) + m * N;
    for (long long nb = 0; nb < N; nb += 32 * U) {
        float gv[U], t1[U], t2[U];
        int k1[U], k2[U];
        bool ok1[U], ok2[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long n = nb + u * 32 + lane;
            gv[u] = 0.f;
            k1[u] = -1;
            k2[u] = -1;
            if (n < N) {
                gv[u] = __fmul_rn(grow[n], scale);
                k1[u] = r1[n];
                k2[u] = r2[n];
            }
            // an index outside [0,K) cannot come from the forward; skip it rather than fault
            ok1[u] = (unsigned)k1[u] < (unsigned long long)K;
            ok2[u] = (unsigned)k2[u] < (unsigned long long)K;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long n = nb + u * 32 + lane;
            t1[u] = 0.f;
            t2[u] = 0.f;
            if (ok1[u]) {
                const long long wi = B_NK ? n * K + k1[u] : (long long)k1[u] * N + n;
                t1[u] = __fmul_rn(w[wi], gv[u]);
                dw_term<FUSED, true>(dw, wi, __fmul_rn(A_SMEM ? as[k1[u]] : arow[k1[u]], gv[u]));
            }
            if (ok2[u]) {
                const long long wi = B_NK ? n * K + k2[u] : (long long)k2[u] * N + n;
                t2[u] = __fmul_rn(w[wi], gv[u]);
                dw_term<FUSED, false>(dw, wi, __fmul_rn(A_SMEM ? as[k2[u]] : arow[k2[u]], gv[u]));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            warp_row_add(dar, k1[u], ok1[u], t1[u], lane);
            warp_row_add(dar, k2[u], ok2[u], t2[u], lane);
        }
    }
    }
    for (long long k = lane; k < K; k += 32) da[m * K + k] = dar[k];
}

// ---------------------------------------------------------------------------------------------
// Two-kernel form of the backward used when both operands fit the shared-memory budgets.
//
// fp32 atomics are the cost of this pass (shared memory ~1.7 lane-ops/clk/SM, L2 reductions ~0.8),
// so neither gradient goes through global atomics here:
//   mam_bwd_dx_kernel : a CTA owns rows of a, accumulates their da in shared memory (as above,
//                       without the dW reductions);
//   mam_bwd_dw_kernel : a CTA owns `cols` consecutive outputs n, keeps their dW rows [cols][K] --
//                       and, when asked, their max/min hit counters -- in shared memory, sweeps
//                       all M rows, then writes each dW row once.  The selection count rides
//                       along for free (integer shared-memory atomics are ~7x faster than fp32).
// grad and the indices are read twice (once per kernel); both reads are streaming.
template <bool B_NK>
__global__ void __launch_bounds__(BWD_THREADS)
mam_bwd_dx_kernel(const float* __restrict__ w, const float* __restrict__ g,
                  const int* __restrict__ argmax, const int* __restrict__ argmin,
                  float* __restrict__ da, long long M, long long K, long long N, int rows_per_cta, float scale) {
    extern __shared__ float da_s[];  // [rows_per_cta][K]
    const long long m0 = (long long)blockIdx.x * rows_per_cta;
    const int rows = (int)min((long long)rows_per_cta, M - m0);
    for (long long i = threadIdx.x; i < (long long)rows * K; i += BWD_THREADS) da_s[i] = 0.f;
    __syncthreads();
    for (int r = 0; r < rows; ++r) {
        const long long m = m0 + r;
        float* dar = da_s + (long long)r * K;
        for (long long n = threadIdx.x; n < N; n += BWD_THREADS) {
            const float gv = __fmul_rn(g[m * N + n], scale);
            const int k1 = argmax[m * N + n], k2 = argmin[m * N + n];
            if ((unsigned)k1 < (unsigned long long)K)
                atomicAdd(&dar[k1], __fmul_rn(w[B_NK ? n * K + k1 : (long long)k1 * N + n], gv));
            if ((unsigned)k2 < (unsigned long long)K)
                atomicAdd(&dar[k2], __fmul_rn(w[B_NK ? n * K + k2 : (long long)k2 * N + n], gv));
        }
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < (long long)rows * K; i += BWD_THREADS) da[m0 * K + i] = da_s[i];
}

// COUNT: also accumulate hit_max / hit_min ([N,K] int32, added to the caller's matrices).
template <bool B_NK, bool COUNT>
__global__ void __launch_bounds__(BWD_THREADS)
mam_bwd_dw_kernel(const float* __restrict__ a, const float* __restrict__ g,
                  const int* __restrict__ argmax, const int* __restrict__ argmin,
                  float* __restrict__ dw, int* __restrict__ hit_max, int* __restrict__ hit_min,
                  long long M, long long K, long long N, int cols, float scale) {
    extern __shared__ float dw_s[];                                  // [cols][K] fp32
    int* cmax_s = reinterpret_cast<int*>(dw_s + (size_t)cols * K);   // [cols][K] (COUNT only)
    int* cmin_s = cmax_s + (size_t)cols * K;
    const long long n0 = (long long)blockIdx.x * cols;
    const int nc = (int)min((long long)cols, N - n0);
    const long long tot = (long long)cols * K * (COUNT ? 3 : 1);
    for (long long i = threadIdx.x; i < tot; i += BWD_THREADS) reinterpret_cast<int*>(dw_s)[i] = 0;
    __syncthreads();
    const long long work = M * nc;  // c = t % nc fastest: the nc values of a row are read together
    for (long long t = threadIdx.x; t < work; t += BWD_THREADS) {
        const long long m = t / nc;
        const int c = (int)(t - m * nc);
        const long long o = m * N + n0 + c;
        const float gv = __fmul_rn(g[o], scale);
        const int k1 = argmax[o], k2 = argmin[o];
        const float* arow = a + m * K;
        if ((unsigned)k1 < (unsigned long long)K) {
            atomicAdd(&dw_s[(long long)c * K + k1], __fmul_rn(arow[k1], gv));
            if (COUNT) atomicAdd(&cmax_s[(long long)c * K + k1], 1);
        }
        if ((unsigned)k2 < (unsigned long long)K) {
            atomicAdd(&dw_s[(long long)c * K + k2], __fmul_rn(arow[k2], gv));
            if (COUNT) atomicAdd(&cmin_s[(long long)c * K + k2], 1);
        }
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < (long long)nc * K; i += BWD_THREADS) {
        const long long c = i / K, k = i - c * K;
        const long long n = n0 + c;
        if (B_NK) dw[n * K + k] = dw_s[i]; else dw[k * N + n] = dw_s[i];
        if (COUNT) {
            const int vmax = cmax_s[i], vmin = cmin_s[i];
            if (vmax) hit_max[n * K + k] += vmax;
            if (vmin) hit_min[n * K + k] += vmin;
        }
    }
}

// True selection counts: cnt_max[n,k] += #rows with argmax[m,n]==k, same for min.  A CTA owns
// COLS consecutive outputs n (COLS*4 bytes = one 32-byte sector of each index row when COLS is 8)
// and one slice of the rows; it keeps the [COLS][K] int32 counters for max and for min in shared
// memory (integer shared-memory atomics run ~7x faster than fp32 ones), sweeps its rows with
// SEL_UNROLL independent loads in flight per thread (the sweep is a pure stream: without them it
// is bound by load latency, not by HBM), then adds its non-zero counters to the caller's [N,K]
// matrices -- atomically, because the CTAs of the other row slices add into the same entries.
// The module-level rule of the reference (mamtorch/nn/v4/fullyconnected.py:114-131) is derived
// from these on the host side: +1 where cnt_max>0, +1 where cnt_min>0.
constexpr int SEL_THREADS = 256;
constexpr int SEL_UNROLL = 8;

template <int COLS>
__global__ void __launch_bounds__(SEL_THREADS)
mam_selcount_kernel(const int* __restrict__ argmax, const int* __restrict__ argmin,
                    int* __restrict__ cnt_max, int* __restrict__ cnt_min,
                    long long M, long long K, long long N, long long rows_per_slice) {
    extern __shared__ int cnt_s[];  // [2][COLS][K]
    const long long n0 = (long long)blockIdx.x * COLS;
    const int nc = (int)min((long long)COLS, N - n0);
    const long long m_begin = (long long)blockIdx.y * rows_per_slice;
    const long long m_end = min(M, m_begin + rows_per_slice);
    const long long tot = 2LL * COLS * K;
    for (long long i = threadIdx.x; i < tot; i += SEL_THREADS) cnt_s[i] = 0;
    __syncthreads();
    constexpr int ROWS_PER_PASS = SEL_THREADS / COLS;
    const int c = threadIdx.x % COLS, r = threadIdx.x / COLS;
    int* my_max = cnt_s + (long long)c * K;
    int* my_min = cnt_s + ((long long)COLS + c) * K;
    if (c < nc) {
        const int* pmax = argmax + n0 + c;
        const int* pmin = argmin + n0 + c;
        for (long long m = m_begin + r; m < m_end; m += (long long)ROWS_PER_PASS * SEL_UNROLL) {
            int k1[SEL_UNROLL], k2[SEL_UNROLL];
#pragma unroll
            for (int u = 0; u < SEL_UNROLL; ++u) {
                const long long mm = m + (long long)u * ROWS_PER_PASS;
                k1[u] = -1;
                k2[u] = -1;
                if (mm < m_end) {
                    k1[u] = __ldg(pmax + mm * N);
                    k2[u] = __ldg(pmin + mm * N);
                }
            }
#pragma unroll
            for (int u = 0; u < SEL_UNROLL; ++u) {
                // an index outside [0,K) cannot come from the forward; skip it rather than fault
                if ((unsigned)k1[u] < (unsigned long long)K) atomicAdd(&my_max[k1[u]], 1);
                if ((unsigned)k2[u] < (unsigned long long)K) atomicAdd(&my_min[k2[u]], 1);
            }
        }
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < (long long)nc * K; i += SEL_THREADS) {
        const int vmax = cnt_s[i], vmin = cnt_s[(long long)COLS * K + i];
        if (vmax) atomicAdd(&cnt_max[n0 * K + i], vmax);
        if (vmin) atomicAdd(&cnt_min[n0 * K + i], vmin);
    }
}

// count[n,k] += (hit_max[n,k] > 0) + (hit_min[n,k] > 0): one update_selection_count() call of the
// reference module, which adds both indicators into max_selection_count
// (mamtorch/nn/v4/fullyconnected.py:125-129).
__global__ void mam_selcount_indicator_kernel(const int* __restrict__ hit_max, const int* __restrict__ hit_min,
                                              int* __restrict__ count, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) count[i] += (hit_max[i] > 0) + (hit_min[i] > 0);
}

}  // namespace mamb200
