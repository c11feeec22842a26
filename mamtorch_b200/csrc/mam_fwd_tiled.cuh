// Tiled MAM forward for sm_100a: TMA-staged operands, register-blocked max/min accumulation.
//
// Computes, for a[M,K] and W[N,K] (both K-contiguous), s[m,n] = max_k p + min_k p with
// p = fl32(a[m,k]*W[n,k]).  It stands where the reference launches
//   fullyconnected_fast_cuda_kernel   (mamtorch/kernel/v4/csrc/cuda/fullyconnected_fast_kernel.cu:29-161)
//   fullyconnected_cuda_kernel        (mamtorch/kernel/v1/csrc/cuda/fullyconnected.cu:33-175)
// but shares nothing with their structure:
//
//  * Operands arrive by TMA (cp.async.bulk.tensor, no multicast) as [rows][32 floats] boxes in the
//    128-byte swizzle, through a STAGES-deep full/empty mbarrier ring.  Thread 0 issues the
//    copies STAGES-2 chunks ahead of the chunk being computed; the kernel is persistent, so
//    the next tile's first chunks are already in flight during the epilogue of the current
//    one.  Every barrier wait is bounded.
//  * Each consumer thread owns a TM x TN block of outputs.  Per four k it issues TM+TN LDS.128
//    (bank-conflict free under the swizzle), 2*TM*TN packed multiplies (mul.rn.f32x2, each half
//    rounded like a scalar fp32 multiply) and 4*TM*TN three-input max/min -- one ALU-pipe
//    instruction per (m,n,k) unit, which is the floor on this machine because fp32 min/max issue
//    at 64 lanes/clk/SM.
//  * TRACK=true also records, per output, the 32-wide k chunk in which the running max (min)
//    last strictly increased (decreased): extremes are formed per chunk in registers and merged
//    into the running value with one compare; the chunk id goes to a per-thread shared-memory
//    slot through a predicated store.  Strict compares over ascending chunks keep the FIRST chunk
//    that attains the final value, so a later scan of only that chunk (mam_resolve_kernel) yields
//    the exact lowest-k index -- the tie rule of the reference -- without per-k index tracking.
#pragma once
#include <cuda.h>
#include "mam_fwd_generic.cuh"

namespace mamb200 {

constexpr int FWD_BK = 32;  // floats per row per stage = one 128-byte swizzle span

template <int TM_, int TN_, int WM_, int WN_, int STAGES_, bool TRACK_>
struct FwdCfg {
    static constexpr int TM = TM_, TN = TN_, WM = WM_, WN = WN_, STAGES = STAGES_;
    static constexpr bool TRACK = TRACK_;
    static constexpr int BM = WM * 4 * TM;   // rows of a per tile
    static constexpr int BN = WN * 8 * TN;   // rows of W per tile
    static constexpr int CONSUMER_WARPS = WM * WN;
    static constexpr int CONSUMERS = CONSUMER_WARPS * 32;
    static constexpr int THREADS = CONSUMERS;       // no separate producer warp: a 9th warp would
                                                    // put 3 warps on one SM sub-partition and cap
                                                    // every thread at 168 registers
    static constexpr int LOOKAHEAD = STAGES - 2;    // chunks in flight ahead of the one computed
    static constexpr int A_BYTES = BM * FWD_BK * 4;
    static constexpr int W_BYTES = BN * FWD_BK * 4;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
    static constexpr int ID_BYTES = TRACK ? 2 * TM * TN * CONSUMERS * 2 : 0;
    static constexpr int BAR_BYTES = 2 * STAGES * 8;
    static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * STAGE_BYTES + BAR_BYTES + ID_BYTES;
    static_assert(TM % 2 == 0, "row swizzle keys assume an even TM");
    static_assert(BM <= 256 && BN <= 256, "TMA box rows");
    static_assert(STAGES >= 3, "need one stage of slack so the issuing warp never waits on its peers");
};

struct FwdParams {
    float* y;
    int* cid_max;  // TRACK: chunk ids (later resolved in place to exact k)
    int* cid_min;
    long long M, K, N;
    EpilogueArgs ep;
    float one;     // 1.0f kept opaque to the compiler (see merge below)
    int* error;    // set to 1 when a bounded wait gave up
};

__device__ __forceinline__ ulonglong2 lds128(const unsigned char* p) {
    return *reinterpret_cast<const ulonglong2*>(p);
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
mam_fwd_tiled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                     const FwdParams prm) {
    constexpr int TM = Cfg::TM, TN = Cfg::TN, STAGES = Cfg::STAGES;
    constexpr bool TRACK = Cfg::TRACK;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    unsigned char* ids = smem + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], Cfg::CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    const long long M = prm.M, K = prm.K, N = prm.N;
    const int ntm = (int)((M + Cfg::BM - 1) / Cfg::BM), ntn = (int)((N + Cfg::BN - 1) / Cfg::BN);
    const long long ntiles = (long long)ntm * ntn;
    const int nk = (int)((K + FWD_BK - 1) / FWD_BK);
    const int tail_quads = (int)((K - (long long)(nk - 1) * FWD_BK) / 4);  // K % 4 == 0 is a precondition

    // ------------------------------------------------------------ producer role (thread 0 only)
    // Thread 0 walks the same (tile, chunk) sequence as the consumers, LOOKAHEAD chunks ahead.
    // The stage it refills held the chunk computed two iterations ago, so the empty-barrier wait
    // below is satisfied unless a peer warp lags by more than a whole chunk.
    long long p_tile = blockIdx.x;
    int p_kc = 0, p_stage = 0;
    uint32_t p_phase = 0;
    auto produce_one = [&]() -> bool {
        if (p_tile >= ntiles) return true;
        if (!mbar_wait_bounded(&empty_bar[p_stage], p_phase ^ 1u)) return false;
        const int tm = (int)(p_tile / ntn), tn = (int)(p_tile % ntn);
        mbar_expect_tx(&full_bar[p_stage], Cfg::STAGE_BYTES);
        unsigned char* sa = smem + p_stage * Cfg::STAGE_BYTES;
        tma_load_2d(sa, &tmA, &full_bar[p_stage], p_kc * FWD_BK, tm * Cfg::BM);
        tma_load_2d(sa + Cfg::A_BYTES, &tmW, &full_bar[p_stage], p_kc * FWD_BK, tn * Cfg::BN);
        if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1u; }
        if (++p_kc == nk) { p_kc = 0; p_tile += gridDim.x; }
        return true;
    };
    if (tid == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
        for (int i = 0; i < Cfg::LOOKAHEAD; ++i) produce_one();
    }

    // ---------------------------------------------------------------- consumers
    const int wm = warp / Cfg::WN, wn = warp % Cfg::WN;
    const int lane_m = lane >> 3, lane_n = lane & 7;
    // byte offsets of this thread's first A row / W row inside a stage; further rows are +i*512 / +j*1024
    const uint32_t a_row0 = (uint32_t)(wm * 4 * TM + lane_m) * 128u;
    const uint32_t w_row0 = (uint32_t)Cfg::A_BYTES + (uint32_t)(wn * 8 * TN + lane_n) * 128u;
    // swizzle: 16-byte group q of row r sits at group q ^ (r & 7).  Rows of this thread have
    // (r & 7) = lane_m (even i), lane_m + 4 (odd i) for A and lane_n for W.
    const uint32_t a_key = (uint32_t)lane_m << 4, w_key = (uint32_t)lane_n << 4;
    const uint32_t id_addr = smem_u32(ids) + (uint32_t)tid * 2u;

    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;

    for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        const int tm = (int)(tile / ntn), tn = (int)(tile % ntn);
        float vmax[TM][TN], vmin[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                vmax[i][j] = -INFINITY;
                vmin[i][j] = INFINITY;
            }
        if constexpr (TRACK) {
#pragma unroll
            for (int s = 0; s < 2 * TM * TN; ++s) {
                const uint32_t addr = id_addr + (uint32_t)(s * Cfg::CONSUMERS * 2);
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)0) : "memory");
            }
        }

        for (int kc = 0; kc < nk; ++kc) {
            if (tid == 0 && !produce_one()) atomicExch(prm.error, 1);
            if (!mbar_wait_bounded(&full_bar[stage], phase)) {
                atomicExch(prm.error, 1);
                ok = false;
                break;
            }
            const unsigned char* sbase = smem + stage * Cfg::STAGE_BYTES;
            const unsigned char* ap = sbase + a_row0;
            const unsigned char* wp = sbase + w_row0;
            float lmax[TRACK ? TM : 1][TRACK ? TN : 1], lmin[TRACK ? TM : 1][TRACK ? TN : 1];

            auto quad = [&](const int q, const bool first) {
                const uint32_t xa0 = ((uint32_t)q << 4) ^ a_key;
                const uint32_t xa1 = xa0 ^ 64u;
                const uint32_t xw = ((uint32_t)q << 4) ^ w_key;
                ulonglong2 av[TM];
#pragma unroll
                for (int i = 0; i < TM; ++i) av[i] = lds128(ap + ((i & 1) ? xa1 : xa0) + i * 512);
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const ulonglong2 wv = lds128(wp + xw + j * 1024);
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        float p0, p1, p2, p3;
                        unpack2(mul2(av[i].x, wv.x), p0, p1);
                        unpack2(mul2(av[i].y, wv.y), p2, p3);
                        if constexpr (TRACK) {
                            if (first) {
                                lmax[i][j] = fmaxf(p0, p1);
                                lmin[i][j] = fminf(p0, p1);
                            } else {
                                lmax[i][j] = fmax3(lmax[i][j], p0, p1);
                                lmin[i][j] = fmin3(lmin[i][j], p0, p1);
                            }
                            lmax[i][j] = fmax3(lmax[i][j], p2, p3);
                            lmin[i][j] = fmin3(lmin[i][j], p2, p3);
                        } else {
                            vmax[i][j] = fmax3(fmax3(vmax[i][j], p0, p1), p2, p3);
                            vmin[i][j] = fmin3(fmin3(vmin[i][j], p0, p1), p2, p3);
                        }
                    }
                }
            };

            if (kc + 1 < nk || tail_quads == FWD_BK / 4) {
                quad(0, true);
#pragma unroll
                for (int q = 1; q < FWD_BK / 4; ++q) quad(q, false);
            } else {
                quad(0, true);
                for (int q = 1; q < tail_quads; ++q) quad(q, false);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }

            if constexpr (TRACK) {
                // merge the chunk extremes into the running ones; one ALU compare per accumulator.
                // The value move is a multiply by an opaque 1.0 (exact for every input, keeps the
                // sign of zero) so that it issues on the FMA pipe rather than the saturated ALU pipe.
                const unsigned short kid = (unsigned short)kc;
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        const uint32_t amax = id_addr + (uint32_t)(((i * TN + j) * 2 + 0) * Cfg::CONSUMERS * 2);
                        const uint32_t amin = id_addr + (uint32_t)(((i * TN + j) * 2 + 1) * Cfg::CONSUMERS * 2);
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.gt.f32 p, %1, %0;\n\t"
                            "@p mul.rn.f32 %0, %1, %2;\n\t"
                            "@p st.shared.u16 [%3], %4;\n\t}"
                            : "+f"(vmax[i][j])
                            : "f"(lmax[i][j]), "f"(prm.one), "r"(amax), "h"(kid)
                            : "memory");
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.lt.f32 p, %1, %0;\n\t"
                            "@p mul.rn.f32 %0, %1, %2;\n\t"
                            "@p st.shared.u16 [%3], %4;\n\t}"
                            : "+f"(vmin[i][j])
                            : "f"(lmin[i][j]), "f"(prm.one), "r"(amin), "h"(kid)
                            : "memory");
                    }
            }
        }
        if (!ok) break;

        // ------------------------------------------------------------ epilogue
        const long long mrow0 = (long long)tm * Cfg::BM + wm * 4 * TM + lane_m;
        const long long ncol0 = (long long)tn * Cfg::BN + wn * 8 * TN + lane_n;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const long long m = mrow0 + i * 4;
            if (m >= M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const long long n = ncol0 + j * 8;
                if (n >= N) continue;
                prm.y[m * N + n] = mam_epilogue(vmax[i][j], vmin[i][j], prm.ep, m, n, N);
                if constexpr (TRACK) {
                    unsigned short cmax, cmin;
                    const uint32_t amax = id_addr + (uint32_t)(((i * TN + j) * 2 + 0) * Cfg::CONSUMERS * 2);
                    const uint32_t amin = id_addr + (uint32_t)(((i * TN + j) * 2 + 1) * Cfg::CONSUMERS * 2);
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmax) : "r"(amax) : "memory");
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmin) : "r"(amin) : "memory");
                    prm.cid_max[m * N + n] = (int)cmax;
                    prm.cid_min[m * N + n] = (int)cmin;
                }
            }
        }
    }
}

// Turns chunk ids into exact indices: scans the one 32-wide chunk recorded for each output with
// strict compares in ascending k.  The chunk's own extreme equals the global one (that is why the
// chunk was recorded), so no target value has to be carried over from the main kernel.
__global__ void __launch_bounds__(256)
mam_resolve_kernel(const float* __restrict__ a, const float* __restrict__ w,
                   int* __restrict__ argmax, int* __restrict__ argmin,
                   long long M, long long K, long long N) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * N) return;
    const long long m = idx / N, n = idx % N;
    const int nk = (int)((K + FWD_BK - 1) / FWD_BK);
    const float* ar = a + m * K;
    const float* wr = w + n * K;
    {
        int c = min(max(argmax[idx], 0), nk - 1);
        const int k0 = c * FWD_BK, k1 = (int)min((long long)k0 + FWD_BK, K);
        float best = -INFINITY;
        int bk = k0;
        for (int k = k0; k < k1; ++k) {
            const float p = __fmul_rn(ar[k], wr[k]);
            if (p > best) { best = p; bk = k; }
        }
        argmax[idx] = bk;
    }
    {
        int c = min(max(argmin[idx], 0), nk - 1);
        const int k0 = c * FWD_BK, k1 = (int)min((long long)k0 + FWD_BK, K);
        float best = INFINITY;
        int bk = k0;
        for (int k = k0; k < k1; ++k) {
            const float p = __fmul_rn(ar[k], wr[k]);
            if (p < best) { best = p; bk = k; }
        }
        argmin[idx] = bk;
    }
}

}  // namespace mamb200
