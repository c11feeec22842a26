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
#include <type_traits>
#include "mam_fwd_generic.cuh"

namespace mamb200 {

constexpr int FWD_BK = 32;  // floats per row per stage = one 128-byte swizzle span

template <int TM_, int TN_, int WM_, int WN_, int STAGES_, bool TRACK_, int UQ_ = 8, bool BATCH_ = false,
          bool MUL2_ = true, bool SPLIT_ = false, bool ROW8_ = false>
struct FwdCfg {
    // Which rows of the tile a thread owns.  false: row(i) = warp_m*4*TM + lane_m + 4*i -- consecutive rows
    // alternate between two swizzle keys, so every group of four k needs two a-addresses.  true: a pair of
    // warps interleaves inside 32-row groups, row(i) = (warp_m/2)*8*TM + 8*i + (warp_m%2)*4 + lane_m -- all rows
    // of a thread share (row & 7), one a-address per group of four k, the rest immediate offsets.
    static constexpr bool ROW8 = ROW8_;
    static_assert(!ROW8_ || (WM_ % 2 == 0), "paired warps");
    // K cut into slices of prm.split_chunks chunks: y = sum over slices of (max + min) of the slice, added in
    // ascending slice order -- the module's `splits` (mamtorch/nn/v4/fullyconnected.py:164-176) in one launch
    // With TRACK the slices' partial sums are banked in y itself (there is no room for a third accumulator set)
    // and every slice leaves its own chunk ids: prm.cid_max holds one [M,N] matrix per slice.
    static constexpr bool SPLIT = SPLIT_;
    static constexpr bool MUL2 = MUL2_;     // packed mul.rn.f32x2 (true) or four scalar multiplies
    static constexpr int UQ = UQ_;          // 16-byte k groups per unrolled loop body
    static constexpr bool BATCH = BATCH_;   // form all products of a W row before any max/min
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

// Patch rows of a convolution read straight from the channels-last input by im2col-mode TMA instead
// of from a materialised [M, K] matrix.  Row m is output pixel (n, ho, wo), m = (n*Ho + ho)*Wo + wo;
// column k' = (kh + kH*kw)*C + c (channels fastest, then kh, then kw: the order of the reference's
// convolution text, mamtorch/kernel/backup/mamconv2d_forward.txt:128), so a 32-wide chunk is 32
// channels of one filter tap.  c32 = C / 32 (0: not a convolution).
struct Im2colRows {
    int c32, C, kH, kW, Ho, Wo, sh, sw, ph, pw;
};

// Where the issuing thread stands in the (tile, chunk) sequence of a convolution: base pixel of the tile
// and the filter tap / channel block of the next chunk.  Decoding a tile costs three integer divisions,
// stepping to the next chunk none -- the issuing thread also computes, and its warp must not fall behind
// the others by a division sequence per chunk.
struct Im2colCursor {
    int n, h, w;        // image and base pixel (top-left patch corner) of the tile's first row
    int cc, kh, kw;     // channel block and tap of the next chunk
    long long m0_of;    // the tile (its first row) that n, h, w belong to; -1: none yet
    // (cc, kh, kw) step with every chunk in every thread (warp-uniform counters); (n, h, w) cost three divisions
    // and are formed only by a thread that issues a copy, once per tile it issues for
    __device__ __forceinline__ void reset() { cc = kh = kw = 0; m0_of = -1; n = h = w = 0; }
    __device__ __forceinline__ void locate(const Im2colRows& cv, long long m0) {
        if (m0_of == m0) return;
        m0_of = m0;
        const int hw = cv.Ho * cv.Wo;
        n = (int)(m0 / hw);
        const int rem = (int)(m0 - (long long)n * hw);
        const int ho = rem / cv.Wo;
        h = ho * cv.sh - cv.ph;
        w = (rem - ho * cv.Wo) * cv.sw - cv.pw;
    }
    __device__ __forceinline__ void load(void* dst, const void* tmap, uint64_t* bar) const {
        tma_load_im2col_4d(dst, tmap, bar, cc * 32, w, h, n, (uint16_t)kw, (uint16_t)kh);
    }
    // to the next chunk; `wrap`: that chunk is the first of the next tile
    __device__ __forceinline__ void advance(const Im2colRows& cv, bool wrap) {
        if (wrap) {
            cc = kh = kw = 0;
        } else if (++cc == cv.c32) {
            cc = 0;
            if (++kh == cv.kH) { kh = 0; ++kw; }
        }
    }
};

struct FwdParams {
    float* y;
    int* cid_max;  // TRACK: receives (max chunk id) | (min chunk id) << 16; the resolver turns it into the exact
    int* cid_min;  //        argmax in place and writes the argmin here
    long long M, K, N;
    EpilogueArgs ep;
    float one;     // 1.0f kept opaque to the compiler (see merge below)
    int* error;    // set to 1 when a bounded wait gave up
    Im2colRows conv;  // c32 != 0: tmA is an im2col-mode map of the channels-last convolution input
    int split_chunks; // Cfg::SPLIT: 32-wide chunks per slice of K
};

// compile-time loop: f receives std::integral_constant<int, I>, so I can feed "n" asm operands
template <int I, int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// LDS.128 from a 32-bit shared-window address plus a compile-time byte offset.  Going through a
// generic pointer instead costs two integer adds per load on the ALU pipe -- the pipe the max/min
// instructions saturate.
template <int OFF>
__device__ __forceinline__ ulonglong2 lds128_at(uint32_t addr) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2+%3];" : "=l"(v.x), "=l"(v.y) : "r"(addr), "n"(OFF));
    return v;
}

// Shared-memory accesses of the resolver by 32-bit shared-window address.  The kernels carve their dynamic
// shared memory up through integer arithmetic (1024-byte alignment), after which the compiler no longer
// knows that the pointers are shared memory and would emit generic loads, stores and atomics.
__device__ __forceinline__ ulonglong2 lds128_s(uint32_t addr) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds32_s(uint32_t addr) {
    int v;
    asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ unsigned lds16_s(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32_s(uint32_t addr, int v) {
    asm volatile("st.shared.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts16_s(uint32_t addr, unsigned v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}
__device__ __forceinline__ int atoms_add_s(uint32_t addr, int v) {
    int old;
    asm volatile("atom.shared.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}

// CONV: the a-operand is fetched by im2col-mode TMA (tmA is an im2col map, prm.conv describes the geometry).
template <class Cfg, bool CONV = false>
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

    // ------------------------------------------------------------ producer role
    // The loads run LOOKAHEAD chunks ahead of the chunk being computed, over the same (tile, chunk) sequence
    // as the consumers.  The stage a load refills held the chunk computed two iterations ago, so the
    // empty-barrier wait below is satisfied unless a peer warp lags by more than a whole chunk.  EVERY thread
    // steps the producer's position (warp-uniform counters); who issues the copies rotates over the warps, chunk
    // by chunk, so that the few dozen instructions of an issue do not make one warp -- and with it the whole CTA,
    // which moves at the pace of its slowest warp -- permanently slower than the others.
    long long p_tile = blockIdx.x;
    int p_kc = 0, p_stage = 0;
    uint32_t p_phase = 0;
    [[maybe_unused]] Im2colCursor p_cur;
    if constexpr (CONV) p_cur.reset();
    auto produce_one = [&](const bool issue) -> bool {
        if (p_tile >= ntiles) return true;
        bool ok = true;
        if (issue) {
            ok = mbar_wait_bounded(&empty_bar[p_stage], p_phase ^ 1u);
            if (ok) {
                const int tm = (int)(p_tile / ntn), tn = (int)(p_tile % ntn);
                mbar_expect_tx(&full_bar[p_stage], Cfg::STAGE_BYTES);
                unsigned char* sa = smem + p_stage * Cfg::STAGE_BYTES;
                if constexpr (CONV) {
                    p_cur.locate(prm.conv, (long long)tm * Cfg::BM);
                    p_cur.load(sa, &tmA, &full_bar[p_stage]);
                } else {
                    tma_load_2d(sa, &tmA, &full_bar[p_stage], p_kc * FWD_BK, tm * Cfg::BM);
                }
                tma_load_2d(sa + Cfg::A_BYTES, &tmW, &full_bar[p_stage], p_kc * FWD_BK, tn * Cfg::BN);
            }
        }
        if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1u; }
        const bool wrap = ++p_kc == nk;
        if (wrap) { p_kc = 0; p_tile += gridDim.x; }
        if constexpr (CONV) p_cur.advance(prm.conv, wrap);
        return ok;
    };
    if (tid == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    for (int i = 0; i < Cfg::LOOKAHEAD; ++i) produce_one(tid == 0);

    // ---------------------------------------------------------------- consumers
    const int wm = warp / Cfg::WN, wn = warp % Cfg::WN;
    const int lane_m = lane >> 3, lane_n = lane & 7;
    // byte offsets of this thread's first A row / W row inside a stage; further rows are +i*512 / +j*1024
    // first row of a this thread owns inside the tile, and the distance between its rows
    const int a_first = Cfg::ROW8 ? (wm >> 1) * 8 * TM + (wm & 1) * 4 + lane_m : wm * 4 * TM + lane_m;
    constexpr int A_ROW_STEP = Cfg::ROW8 ? 8 : 4;
    const uint32_t a_row0 = (uint32_t)a_first * 128u;
    const uint32_t w_row0 = (uint32_t)Cfg::A_BYTES + (uint32_t)(wn * 8 * TN + lane_n) * 128u;
    // swizzle: 16-byte group q of row r sits at group q ^ (r & 7).  Rows of this thread have
    // (r & 7) = lane_m (even i), lane_m + 4 (odd i) for A and lane_n for W.
    const uint32_t a_key = (uint32_t)(Cfg::ROW8 ? (a_first & 7) : lane_m) << 4, w_key = (uint32_t)lane_n << 4;
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

        float ysum[(Cfg::SPLIT && !TRACK) ? TM : 1][(Cfg::SPLIT && !TRACK) ? TN : 1];
        int next_split = prm.split_chunks;
        if constexpr (Cfg::SPLIT && !TRACK) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) ysum[i][j] = 0.f;
        }
        [[maybe_unused]] int slice_base = 0;   // first chunk of the current slice (TRACK: ids are slice-relative)
        for (int kc = 0; kc < nk; ++kc) {
            if constexpr (Cfg::SPLIT) {
                if (kc == next_split) {   // a slice of K ends: bank its max + min, start the next one
                    next_split += prm.split_chunks;
                    if constexpr (TRACK) {
                        const long long slice = kc / prm.split_chunks - 1;   // the slice that just ended
                        const long long mrow0 = (long long)tm * Cfg::BM + a_first;
                        const long long ncol0 = (long long)tn * Cfg::BN + wn * 8 * TN + lane_n;
                        slice_base = kc;
#pragma unroll
                        for (int i = 0; i < TM; ++i)
#pragma unroll
                            for (int j = 0; j < TN; ++j) {
                                const long long m = mrow0 + i * A_ROW_STEP, n = ncol0 + j * 8;
                                const uint32_t amax = id_addr + (uint32_t)(((i * TN + j) * 2 + 0) * Cfg::CONSUMERS * 2);
                                const uint32_t amin = id_addr + (uint32_t)(((i * TN + j) * 2 + 1) * Cfg::CONSUMERS * 2);
                                if (m < M && n < N) {
                                    const float t = __fadd_rn(vmax[i][j], vmin[i][j]);
                                    float* yp = prm.y + m * N + n;
                                    // the first slice stands alone (0 + t would turn -0 into +0)
                                    *yp = slice == 0 ? t : __fadd_rn(*yp, t);
                                    unsigned short cmax, cmin;
                                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmax) : "r"(amax) : "memory");
                                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmin) : "r"(amin) : "memory");
                                    prm.cid_max[slice * M * N + m * N + n] = (int)((unsigned)cmax | ((unsigned)cmin << 16));
                                }
                                asm volatile("st.shared.u16 [%0], %1;" ::"r"(amax), "h"((unsigned short)0) : "memory");
                                asm volatile("st.shared.u16 [%0], %1;" ::"r"(amin), "h"((unsigned short)0) : "memory");
                                vmax[i][j] = -INFINITY;
                                vmin[i][j] = INFINITY;
                            }
                    } else {
#pragma unroll
                        for (int i = 0; i < TM; ++i)
#pragma unroll
                            for (int j = 0; j < TN; ++j) {
                                const float t = __fadd_rn(vmax[i][j], vmin[i][j]);
                                // the first slice stands alone (0 + t would turn -0 into +0)
                                ysum[i][j] = (kc == prm.split_chunks) ? t : __fadd_rn(ysum[i][j], t);
                                vmax[i][j] = -INFINITY;
                                vmin[i][j] = INFINITY;
                            }
                    }
                }
            }
            const bool my_turn = lane == 0 && warp == kc % Cfg::CONSUMER_WARPS;
            if (!produce_one(my_turn)) atomicExch(prm.error, 1);
            if (!mbar_wait_bounded(&full_bar[stage], phase)) {
                atomicExch(prm.error, 1);
                ok = false;
                break;
            }
            const uint32_t sbase = smem_u32(smem) + (uint32_t)(stage * Cfg::STAGE_BYTES);
            const uint32_t ap = sbase + a_row0;
            const uint32_t wp = sbase + w_row0;
            float lmax[TRACK ? TM : 1][TRACK ? TN : 1], lmin[TRACK ? TM : 1][TRACK ? TN : 1];

            // qoff = 16 * (index of the group of four k inside the chunk)
            auto quad = [&](const uint32_t qoff, const bool first) {
                // ap and wp are 128-byte aligned and the swizzled group offset is < 128, so OR is ADD
                // and each address is one three-input logic op
                const uint32_t xa0 = ap | (qoff ^ a_key);
                const uint32_t xa1 = xa0 ^ 64u;
                const uint32_t xw = wp | (qoff ^ w_key);
                ulonglong2 av[TM];
                static_for<0, TM>([&](auto ic) {
                    constexpr int i = decltype(ic)::value;
                    if constexpr (Cfg::ROW8) av[i] = lds128_at<i * 1024>(xa0);
                    else av[i] = lds128_at<i * 512>((i & 1) ? xa1 : xa0);
                });
                static_for<0, TN>([&](auto jc) {
                    constexpr int j = decltype(jc)::value;
                    const ulonglong2 wv = lds128_at<j * 1024>(xw);
                    float p[TM][4];
                    auto products = [&](int i) {
                        if constexpr (Cfg::MUL2) {
                            unpack2(mul2(av[i].x, wv.x), p[i][0], p[i][1]);
                            unpack2(mul2(av[i].y, wv.y), p[i][2], p[i][3]);
                        } else {
                            float a0, a1, a2, a3, w0, w1, w2, w3;
                            unpack2(av[i].x, a0, a1);
                            unpack2(av[i].y, a2, a3);
                            unpack2(wv.x, w0, w1);
                            unpack2(wv.y, w2, w3);
                            p[i][0] = __fmul_rn(a0, w0);
                            p[i][1] = __fmul_rn(a1, w1);
                            p[i][2] = __fmul_rn(a2, w2);
                            p[i][3] = __fmul_rn(a3, w3);
                        }
                    };
                    if constexpr (Cfg::BATCH) {
#pragma unroll
                        for (int i = 0; i < TM; ++i) products(i);
                    }
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        if constexpr (!Cfg::BATCH) products(i);
                        if constexpr (TRACK) {
                            if (first) {
                                lmax[i][j] = fmaxf(p[i][0], p[i][1]);
                                lmin[i][j] = fminf(p[i][0], p[i][1]);
                            } else {
                                lmax[i][j] = fmax3(lmax[i][j], p[i][0], p[i][1]);
                                lmin[i][j] = fmin3(lmin[i][j], p[i][0], p[i][1]);
                            }
                            lmax[i][j] = fmax3(lmax[i][j], p[i][2], p[i][3]);
                            lmin[i][j] = fmin3(lmin[i][j], p[i][2], p[i][3]);
                        } else {
                            vmax[i][j] = fmax3(fmax3(vmax[i][j], p[i][0], p[i][1]), p[i][2], p[i][3]);
                            vmin[i][j] = fmin3(fmin3(vmin[i][j], p[i][0], p[i][1]), p[i][2], p[i][3]);
                        }
                    }
                });
            };

            // one code path for full and ragged chunks: the first group is peeled (it initialises
            // the chunk-local extremes), the rest run in a loop unrolled UQ groups at a time so
            // that the body stays inside the instruction cache
            const int nq = (kc + 1 < nk) ? FWD_BK / 4 : tail_quads;
            quad(0u, true);
            const uint32_t qend = (uint32_t)nq << 4;
#pragma unroll(Cfg::UQ)
            for (uint32_t qoff = 16u; qoff < qend; qoff += 16u) quad(qoff, false);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }

            if constexpr (TRACK) {
                // merge the chunk extremes into the running ones; one ALU compare per accumulator.
                // The value move is a multiply by an opaque 1.0 (exact for every input, keeps the
                // sign of zero) so that it issues on the FMA pipe rather than the saturated ALU pipe.
                const unsigned short kid = (unsigned short)(Cfg::SPLIT ? kc - slice_base : kc);
                static_for<0, TM * TN>([&](auto slot) {
                    constexpr int S = decltype(slot)::value;
                    constexpr int i = S / TN, j = S % TN;
                    // slot addresses are id_addr + compile-time offsets: no address arithmetic
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.gt.f32 p, %1, %0;\n\t"
                        "@p mul.rn.f32 %0, %1, %2;\n\t"
                        "@p st.shared.u16 [%3+%5], %4;\n\t}"
                        : "+f"(vmax[i][j])
                        : "f"(lmax[i][j]), "f"(prm.one), "r"(id_addr), "h"(kid), "n"((S * 2 + 0) * Cfg::CONSUMERS * 2)
                        : "memory");
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.lt.f32 p, %1, %0;\n\t"
                        "@p mul.rn.f32 %0, %1, %2;\n\t"
                        "@p st.shared.u16 [%3+%5], %4;\n\t}"
                        : "+f"(vmin[i][j])
                        : "f"(lmin[i][j]), "f"(prm.one), "r"(id_addr), "h"(kid), "n"((S * 2 + 1) * Cfg::CONSUMERS * 2)
                        : "memory");
                });
            }
        }
        if (!ok) break;

        // ------------------------------------------------------------ epilogue
        const long long mrow0 = (long long)tm * Cfg::BM + a_first;
        const long long ncol0 = (long long)tn * Cfg::BN + wn * 8 * TN + lane_n;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const long long m = mrow0 + i * A_ROW_STEP;
            if (m >= M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const long long n = ncol0 + j * 8;
                if (n >= N) continue;
                if constexpr (Cfg::SPLIT && TRACK)   // the earlier slices' sum waits in y
                    prm.y[m * N + n] = mam_epilogue_term(
                        __fadd_rn(prm.y[m * N + n], __fadd_rn(vmax[i][j], vmin[i][j])), prm.ep, m, n, N);
                else if constexpr (Cfg::SPLIT)
                    prm.y[m * N + n] = mam_epilogue_term(
                        __fadd_rn(ysum[i][j], __fadd_rn(vmax[i][j], vmin[i][j])), prm.ep, m, n, N);
                else
                    prm.y[m * N + n] = mam_epilogue(vmax[i][j], vmin[i][j], prm.ep, m, n, N);
                if constexpr (TRACK) {
                    unsigned short cmax, cmin;
                    const uint32_t amax = id_addr + (uint32_t)(((i * TN + j) * 2 + 0) * Cfg::CONSUMERS * 2);
                    const uint32_t amin = id_addr + (uint32_t)(((i * TN + j) * 2 + 1) * Cfg::CONSUMERS * 2);
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmax) : "r"(amax) : "memory");
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(cmin) : "r"(amin) : "memory");
                    // both chunk ids in one word (K / 32 < 65535): the resolver reads half as much
                    const long long last_slice = Cfg::SPLIT ? (long long)((nk - 1) / prm.split_chunks) : 0;
                    prm.cid_max[last_slice * M * N + m * N + n] = (int)((unsigned)cmax | ((unsigned)cmin << 16));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Index resolution, tiled: chunk ids -> exact lowest-k indices.
//
// Every output carries two tasks (its max chunk and its min chunk); a task rescans one 32-wide
// chunk of one a-row against one W-row.  A CTA owns an RM x RN tile of outputs.  It counting-sorts
// the tile's 2*RM*RN tasks by chunk in shared memory (integer shared-memory atomics), then
// streams the tile's operand chunks through a TMA ring like the main kernel's, and for chunk c
// its threads split the tasks of bucket c between them, each taking a run of consecutive tasks.
//
// Shared-memory bandwidth is the floor here (every task reads its own 2 x 128 bytes), so the
// stage is NOT swizzled: lane L reads the eight 16-byte groups of its rows in the rotated order
// (q + L) & 7, which puts the eight lanes of every quarter-warp on eight different bank groups
// whatever rows they hold.  Group extremes therefore sit in rotated registers; the pick below
// recovers the lowest true group index among those equal to the chunk extreme.
// A min task negates its a-values (exact) and then runs the same max search as a max task.
struct ResolveCfg {
    static constexpr int RM = 64, RN = 128, STAGES = 3, THREADS = 256, WARPS = 8;
    static constexpr int NK_MAX = 2048;  // K <= 65536
    static constexpr int A_BYTES = RM * FWD_BK * 4, W_BYTES = RN * FWD_BK * 4;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
    static constexpr int TASKS = 2 * RM * RN;
    // Bucket counters: `segments` per chunk (see pass A of the kernel), as many as keep the two counter arrays
    // under ~8 KB, so that three stages still leave room for two CTAs per SM at ordinary K (at most 113 KB up to
    // K = 32000; 121 KB and one CTA per SM at the 65536 limit).
    __host__ __device__ static constexpr int nk_pad(int nk) { return (nk + 3) & ~3; }
    __host__ __device__ static constexpr int segments(int nk) {
        int s = WARPS;
        while (s > 1 && s * nk > 1000) s >>= 1;
        return s;
    }
    static constexpr int smem_bytes(int nk) {
        return 1024 + STAGES * STAGE_BYTES + 2 * STAGES * 8 + 64 + TASKS * 2 + (2 * nk_pad(nk * segments(nk)) + 8) * 4;
    }
    static constexpr int LOOKAHEAD = STAGES - 1;
};

template <bool CONV>
__global__ void __launch_bounds__(ResolveCfg::THREADS, 2)
mam_resolve_tiled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                         int* __restrict__ argmax, int* __restrict__ argmin,
                         long long M, long long K, long long N, int* error, const Im2colRows conv, int k_offset) {
    using C = ResolveCfg;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    unsigned short* tasks = reinterpret_cast<unsigned short*>(smem + C::STAGES * C::STAGE_BYTES + 2 * C::STAGES * 8 + 64);
    const int nk_for_layout = (int)((K + FWD_BK - 1) / FWD_BK);
    const int segs = C::segments(nk_for_layout);              // counters per chunk
    const int entries = nk_for_layout * segs;
    int* cursor = reinterpret_cast<int*>(tasks + C::TASKS);  // [entries]   tasks per (chunk, segment)
    int* start = cursor + C::nk_pad(entries) + 4;             // [entries+1] where each (chunk, segment) begins
    __shared__ int warp_sums[C::WARPS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nk = (int)((K + FWD_BK - 1) / FWD_BK);
    const int tail_quads = (int)((K - (long long)(nk - 1) * FWD_BK) / 4);
    const int ntn = (int)((N + C::RN - 1) / C::RN);
    const long long m0 = (long long)(blockIdx.x / ntn) * C::RM, n0 = (long long)(blockIdx.x % ntn) * C::RN;

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], C::WARPS);
        }
        mbar_fence_init();
    }
    const uint32_t cursor_s = smem_u32(cursor), start_s = smem_u32(start), tasks_s = smem_u32(tasks);
    for (int i = tid; i < entries; i += C::THREADS) sts32_s(cursor_s + 4u * i, 0);
    __syncthreads();

    // producer: every thread steps the position, the warp that issues the copies rotates chunk by chunk (as in
    // the main kernel)
    int p_kc = 0, p_stage = 0;
    uint32_t p_phase = 0;
    [[maybe_unused]] Im2colCursor p_cur;
    if constexpr (CONV) p_cur.reset();
    auto produce_one = [&](const bool issue) -> bool {
        if (p_kc >= nk) return true;
        bool good = true;
        if (issue) {
            good = mbar_wait_bounded(&empty_bar[p_stage], p_phase ^ 1u);
            if (good) {
                mbar_expect_tx(&full_bar[p_stage], C::STAGE_BYTES);
                unsigned char* sa = smem + p_stage * C::STAGE_BYTES;
                if constexpr (CONV) {
                    p_cur.locate(conv, m0);
                    p_cur.load(sa, &tmA, &full_bar[p_stage]);
                } else {
                    tma_load_2d(sa, &tmA, &full_bar[p_stage], p_kc * FWD_BK, (int)m0);
                }
                tma_load_2d(sa + C::A_BYTES, &tmW, &full_bar[p_stage], p_kc * FWD_BK, (int)n0);
            }
        }
        if (++p_stage == C::STAGES) { p_stage = 0; p_phase ^= 1u; }
        ++p_kc;
        if constexpr (CONV) p_cur.advance(conv, false);
        return good;
    };
    if (tid == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    for (int i = 0; i < C::LOOKAHEAD; ++i) produce_one(tid == 0);

    // ---- pass A: read this thread's chunk ids once (all loads in flight together) and take a place in the
    // bucket of each: the value an integer shared-memory atomic returns IS the task's rank, so the sort needs
    // one round of atomics, not a counting round and a placing round.  Every warp owns RM / WARPS consecutive
    // a-rows and walks them in order; counters are kept per (chunk, segment), a segment being the rows of one
    // warp (of two or more warps where K has too many chunks for 8 counters each), and a warp's atomics on one
    // address take effect in program order.  A bucket is therefore laid out segment by segment and, inside a
    // segment, a-row by a-row: tasks that are neighbours in a bucket mostly share their a-row, which pass C
    // turns into register reuse.  No barrier is needed until all ranks are taken.
    constexpr int ROWS_PER_WARP = C::RM / C::WARPS;          // 8
    constexpr int COLS_PER_LANE = C::RN / 32;                // 4
    constexpr int IDS = ROWS_PER_WARP * COLS_PER_LANE;       // (max, min) pairs per thread
    const int seg = (warp * segs) / C::WARPS;
    unsigned ids[IDS];   // (max chunk) | (min chunk) << 16; 0xffffffff = outside the matrix
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
        for (int q = 0; q < COLS_PER_LANE; ++q) {
            const long long m = m0 + warp * ROWS_PER_WARP + r, n = n0 + q * 32 + lane;
            unsigned v = 0xffffffffu;
            if (m < M && n < N) {
                const unsigned packed = (unsigned)argmax[m * N + n];   // as the main kernel left it
                const int c1 = min((int)(packed & 0xffffu), nk - 1);
                const int c2 = min((int)(packed >> 16), nk - 1);
                v = (unsigned)c1 | ((unsigned)c2 << 16);
            }
            ids[r * COLS_PER_LANE + q] = v;
        }
    unsigned rk[IDS];    // (rank of the max task) | (rank of the min task) << 16; ranks < 2*RM*RN = 16384
#pragma unroll
    for (int i = 0; i < IDS; ++i) {
        rk[i] = 0u;
        if (ids[i] != 0xffffffffu) {
            const unsigned r1 = (unsigned)atoms_add_s(cursor_s + 4u * ((ids[i] & 0xffffu) * segs + seg), 1);
            const unsigned r2 = (unsigned)atoms_add_s(cursor_s + 4u * ((ids[i] >> 16) * segs + seg), 1);
            rk[i] = r1 | (r2 << 16);
        }
    }
    __syncthreads();
    // ---- exclusive scan of the nk * segs counts, chunk-major (at most NK_MAX = 8 * THREADS of them)
    {
        constexpr int PER = C::NK_MAX / C::THREADS;
        int v[PER], sum = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int idx = tid * PER + i;
            v[i] = idx < entries ? lds32_s(cursor_s + 4u * idx) : 0;
            sum += v[i];
        }
        int incl = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int base = 0;
        for (int w2 = 0; w2 < warp; ++w2) base += warp_sums[w2];
        int run = base + incl - sum;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int idx = tid * PER + i;
            if (idx < entries) sts32_s(start_s + 4u * idx, run);
            run += v[i];
        }
        if (tid == C::THREADS - 1) sts32_s(start_s + 4u * entries, run);
    }
    __syncthreads();
    // ---- pass B: every task code goes to (start of its bucket segment) + (its rank); plain stores.
    // code = (row * RN + column) << 1 | (1 for a min task)
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
        for (int q = 0; q < COLS_PER_LANE; ++q) {
            const int i = r * COLS_PER_LANE + q;
            const unsigned o = (unsigned)((warp * ROWS_PER_WARP + r) * C::RN + q * 32 + lane);
            if (ids[i] != 0xffffffffu) {
                const int p1 = lds32_s(start_s + 4u * ((ids[i] & 0xffffu) * segs + seg)) + (int)(rk[i] & 0xffffu);
                const int p2 = lds32_s(start_s + 4u * ((ids[i] >> 16) * segs + seg)) + (int)(rk[i] >> 16);
                sts16_s(tasks_s + 2u * p1, o << 1);
                sts16_s(tasks_s + 2u * p2, (o << 1) | 1u);
            }
        }
    __syncthreads();

    // ---- pass C: stream the chunks, resolve the tasks of each.  A thread takes a run of consecutive tasks
    // of the bucket; consecutive tasks mostly share their a-row (see pass A), whose chunk then stays in
    // registers and only the W-row is read again.
    int stage = 0;
    uint32_t phase = 0;
    [[maybe_unused]] int r_cc = 0, r_kh = 0, r_kw = 0;   // convolution: channel block and tap of the chunk being resolved
    for (int kc = 0; kc < nk; ++kc) {
        if (!produce_one(lane == 0 && warp == kc % C::WARPS)) atomicExch(error, 1);
        if (!mbar_wait_bounded(&full_bar[stage], phase)) {
            atomicExch(error, 1);
            return;
        }
        const uint32_t As = smem_u32(smem) + (uint32_t)(stage * C::STAGE_BYTES);
        const uint32_t Ws = As + (uint32_t)C::A_BYTES;
        const int nq = (kc + 1 < nk) ? FWD_BK / 4 : tail_quads;
        // Convolution rows: the chunk is 32 channels of one tap; indices leave in the numbering
        // k = (c*kH + kh)*kW + kw of weight.view(F, -1), i.e. kout = kout0 + e * kH*kW for element e.
        int kout0 = kc * FWD_BK, kout_step = 1;
        if constexpr (CONV) {   // (r_cc, r_kh, r_kw) step with the chunks: no divisions in the loop
            kout_step = conv.kH * conv.kW;
            kout0 = r_cc * 32 * kout_step + r_kh * conv.kW + r_kw;
            if (++r_cc == conv.c32) {
                r_cc = 0;
                if (++r_kh == conv.kH) { r_kh = 0; ++r_kw; }
            }
        }
        const int b0 = lds32_s(start_s + 4u * (kc * segs)), b1 = lds32_s(start_s + 4u * ((kc + 1) * segs));
        const int per = (b1 - b0 + C::THREADS - 1) / C::THREADS;   // tasks per thread in this chunk
        const int t_first = b0 + tid * per;
        const int t_last = min(t_first + per, b1);
        // the a-row's chunk, rotated: register r holds true 16-byte group (r + lane) & 7
        ulonglong2 areg[FWD_BK / 4];
        int cached_ra = -1;
        for (int t = t_first; t < t_last; ++t) {
            const unsigned code = lds16_s(tasks_s + 2u * t);
            const int o = (int)(code >> 1);
            const int ra = o / C::RN, rw = o % C::RN;
            const float sgn = (code & 1u) ? -1.0f : 1.0f;
            const f32x2_t sgn2 = pack2(sgn, sgn);
            const uint32_t ap = As + (uint32_t)ra * 128u;
            const uint32_t wp = Ws + (uint32_t)rw * 128u;
            if (ra != cached_ra) {
                cached_ra = ra;
#pragma unroll
                for (int r = 0; r < FWD_BK / 4; ++r) areg[r] = lds128_s(ap + ((uint32_t)((r + lane) & 7) << 4));
            }
            float qm[FWD_BK / 4];
#pragma unroll
            for (int r = 0; r < FWD_BK / 4; ++r) {
                const ulonglong2 wv = lds128_s(wp + ((uint32_t)((r + lane) & 7) << 4));
                float p0, p1, p2, p3;
                // a min task looks for the maximum of the negated products (the sign flip is exact)
                unpack2(mul2(mul2(areg[r].x, sgn2), wv.x), p0, p1);
                unpack2(mul2(mul2(areg[r].y, sgn2), wv.y), p2, p3);
                qm[r] = fmaxf(fmax3(p0, p1, p2), p3);
            }
            // groups at or beyond nq (ragged last chunk) hold zero fill: exclude them
            float best = -INFINITY;
#pragma unroll
            for (int r = 0; r < FWD_BK / 4; ++r) {
                const int gq = (r + lane) & 7;
                if (gq >= nq) qm[r] = -INFINITY;
                best = fmaxf(best, qm[r]);
            }
            int bq = FWD_BK / 4;
#pragma unroll
            for (int r = 0; r < FWD_BK / 4; ++r) {
                const int gq = (r + lane) & 7;
                if (qm[r] == best) bq = min(bq, gq);
            }
            bq = min(bq, nq - 1);  // only reachable when every product is NaN
            // first element of group bq equal to the extreme
            const ulonglong2 av = lds128_s(ap + ((uint32_t)bq << 4));
            const ulonglong2 wv = lds128_s(wp + ((uint32_t)bq << 4));
            float p0, p1, p2, p3;
            unpack2(mul2(mul2(av.x, sgn2), wv.x), p0, p1);
            unpack2(mul2(mul2(av.y, sgn2), wv.y), p2, p3);
            int e = 3;
            if (p2 == best) e = 2;
            if (p1 == best) e = 1;
            if (p0 == best) e = 0;
            // k_offset: the problem is a slice of a wider K (slices of the module's `splits`); indices leave
            // in the numbering of the whole row
            const int kbest = CONV ? kout0 + (bq * 4 + e) * kout_step : kout0 + bq * 4 + e + k_offset;
            const long long m = m0 + ra, n = n0 + rw;
            if (code & 1u) argmin[m * N + n] = kbest; else argmax[m * N + n] = kbest;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
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
    const unsigned packed = (unsigned)argmax[idx];   // (max chunk id) | (min chunk id) << 16
    {
        int c = min((int)(packed & 0xffffu), nk - 1);
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
        int c = min((int)(packed >> 16), nk - 1);
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
